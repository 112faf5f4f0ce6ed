"""Stand-alone kernels of the kernel sweep (MSM Mpts/s, NTT / fold GB/s, fp64 head forward), device-timed
with CUDA events on the backend's stream.  Measurement code used by bench.py; not on the proving path."""
import ctypes

import numpy as np


def _sz(v):
    return ctypes.c_size_t(int(v))


def _c_uint(v):
    return ctypes.c_uint(int(v))


def _stream_of(be, device):
    import torch

    return torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", device))


def run_sweep(be, device, small=False, budget_gb=40.0):
    """The kernel sweep: G1 MSM 2^16..2^26 (plain, and against a resident table of shifted bases while the
    table fits `budget_gb`), Fr NTT / inverse NTT / coset NTT 2^16..2^26 at batch 1, 4, 16, 64 (while
    n * batch <= 2^28), coset LDE with blow-up 2, sumcheck fold 2^20..2^26; each line with its time, its
    rate (Mpts/s or GB/s of algorithmic bytes) and the fraction of the integer-pipe roof measured in the
    same run.  Inputs are generated on the device: scalars and vectors are the powers of a seeded
    challenge (uniform-looking field elements), MSM bases are [k_i] G for such k_i."""
    import torch

    import pyref

    from project_b200 import KIND_FR, KIND_FR_MONT, KIND_G1
    from project_b200.lib import measure_mac_peak

    stream = _stream_of(be, device)
    rng = np.random.default_rng(1234)
    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()
    mac_peak = measure_mac_peak(device, 2, 20000)       # 8x8-limb products per second
    fr_mul_roof = mac_peak * 64.0 / 136.0               # Montgomery multiplications in Fr (136 limb products each)
    fp_mul_roof = mac_peak * 64.0 / 300.0               # ... in Fp (12 limbs: 300 limb products each)

    def timed_ms(fn, reps=3):
        fn()
        be.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(reps):
            fn()
        stop.record(stream)
        be.synchronize()
        return start.elapsed_time(stop) / reps

    def challenge(seed):
        c = np.zeros(32, dtype=np.uint8)
        c[:8] = np.frombuffer(np.uint64((0x9E3779B97F4A7C15 * seed) % (1 << 64) | 1).tobytes(), dtype=np.uint8)
        c[8:16] = np.frombuffer(np.uint64((0xC2B2AE3D27D4EB4F * seed) % (1 << 64)).tobytes(), dtype=np.uint8)
        return c

    def device_vector(n, seed):
        """n field elements c^0, c^1, ... (Montgomery form) built on the device"""
        return be.powers(challenge(seed), n)

    out = {"integer_roof": {"limb_products_per_s": mac_peak * 64, "fr_mults_per_s": fr_mul_roof, "fp_mults_per_s": fp_mul_roof,
                            "note": "8x8-limb multiply-accumulate rate measured on register operands; a Montgomery multiplication costs 136 (Fr) / 300 (Fp) limb products"}}
    sizes = (12, 14) if small else (16, 18, 20, 22, 24, 26)

    # ---- MSM -------------------------------------------------------------------------------------------
    msm = []
    for lg in sizes:
        n = 1 << lg
        scalars = device_vector(n, 1)
        multipliers = device_vector(n, 2)
        points = be.g1_fixed_base_mul(G, multipliers, n)
        multipliers.free()
        ms = timed_ms(lambda: be.msm(scalars, points, n), reps=2 if lg >= 24 else 3)
        c = min(16, max(8, lg - 6))
        windows = -(-256 // c)
        adds = n * windows * 10 + 2 * (1 << (c - 1)) * windows * 14  # Fp multiplications: mixed additions + bucket reduction
        entry = {"log2n": lg, "ms": ms, "Mpts_per_s": n / ms / 1e3, "window_bits": c,
                 "integer_roof_frac": adds / (ms * 1e-3) / fp_mul_roof}
        wb = be.msm_window_bits(n)
        table_points = int(be.lib.gzk_msm_table_points(_sz(n), _c_uint(wb)))
        if table_points * 96 / 1e9 <= budget_gb:
            table, wb = be.msm_precompute(points, n)
            ms = timed_ms(lambda: be.msm_precomputed(scalars, table, n, wb), reps=2 if lg >= 24 else 3)
            w2 = table_points // n
            adds = n * w2 * 10 + 2 * (1 << (wb - 1)) * 14
            entry["resident_table"] = {"window_bits": wb, "table_GB": table_points * 96 / 1e9, "ms": ms, "Mpts_per_s": n / ms / 1e3,
                                       "integer_roof_frac": adds / (ms * 1e-3) / fp_mul_roof}
            table.free()
        else:
            entry["resident_table"] = f"table of shifted bases would take {table_points * 96 / 1e9:.0f} GB (budget {budget_gb:.0f} GB)"
        msm.append(entry)
        scalars.free()
        points.free()
    out["msm"] = msm

    # ---- NTT / inverse / coset / LDE -------------------------------------------------------------------
    ntt = []
    shift = np.zeros(32, dtype=np.uint8)
    shift[0] = 5
    for lg in sizes:
        n = 1 << lg
        for batch in ((1, 4) if small else (1, 4, 16, 64)):
            if n * batch > (1 << 28):
                continue
            vec = device_vector(n * batch, 3)
            res = be.alloc(KIND_FR_MONT, n * batch)
            passes = 1 + (max(0, lg - 10) + 7) // 8
            mults = batch * ((n // 2) * lg + n * (passes - 1))
            entry = {"log2n": lg, "batch": batch}
            for name, kw in (("forward", {}), ("inverse", {"inverse": True}), ("coset_forward", {"coset_shift": shift})):
                ms = timed_ms(lambda: be.ntt(vec, lg, batch=batch, out=res, **kw), reps=2 if n * batch >= (1 << 26) else 3)
                extra = batch * n if name != "forward" else 0  # the scaling by 1/n or by the coset powers
                entry[name] = {"ms": ms, "GB_per_s": 2 * 32 * n * batch / ms / 1e6, "integer_roof_frac": (mults + extra) / (ms * 1e-3) / fr_mul_roof}
            ntt.append(entry)
            vec.free()
            res.free()
    out["ntt"] = ntt
    lde = []
    for lg in sizes:
        if lg + 1 > 27:
            continue
        n = 1 << lg
        vec = device_vector(n, 4)
        wide = be.alloc(KIND_FR_MONT, 2 * n)
        ms = timed_ms(lambda: be.coset_lde(vec, lg, 1, shift, out=wide), reps=2)
        wide.free()
        lde.append({"log2n": lg, "blowup": 2, "ms": ms, "GB_per_s": 32 * n * 3 / ms / 1e6})
        vec.free()
    out["coset_lde"] = lde

    # ---- sumcheck fold ----------------------------------------------------------------------------------
    fold = []
    for lg in ((12, 14) if small else (20, 22, 24, 26)):
        n = 1 << lg
        vec = device_vector(n, 5)  # Montgomery table
        half = be.alloc(KIND_FR_MONT, n // 2)
        r = challenge(6)
        ms = timed_ms(lambda: be.fold(vec, n, r, out=half))
        fold.append({"log2n": lg, "ms": ms, "GB_per_s": 48 * n / ms / 1e6, "integer_roof_frac": (n // 2) / (ms * 1e-3) / fr_mul_roof,
                     "forms": "table kept in Montgomery form (1 multiplication per output)"})
        vec.free()
        half.free()
    out["fold"] = fold

    # ---- CPU stand-ins on the host cores (the reference has no MSM, NTT or fold: these are the oracle's) ------
    try:
        import time

        import oracle_lib as ora

        cpu = {}
        m = 1 << 10
        sc = rng.integers(0, 256, size=(m, 32), dtype=np.uint8)
        sc[:, 31] &= 0x3F
        pts = ora.g1_mul_same_base(G, sc[:64])
        pts = np.tile(pts, (m // 64, 1))
        t0 = time.perf_counter()
        ora.g1_msm_naive(pts, sc)
        cpu["msm_naive_2p10"] = {"ms": (time.perf_counter() - t0) * 1e3, "note": "double-and-add per point, one thread"}
        v = rng.integers(0, 256, size=(1 << 16, 32), dtype=np.uint8)
        v[:, 31] &= 0x3F
        t0 = time.perf_counter()
        ora.ntt(v)
        cpu["ntt_2p16"] = {"ms": (time.perf_counter() - t0) * 1e3, "note": "radix-2 transform, one thread"}
        t0 = time.perf_counter()
        ora.fold(v, sc[0])
        cpu["fold_2p16"] = {"ms": (time.perf_counter() - t0) * 1e3, "note": "one thread"}
        out["cpu_stand_ins"] = cpu
    except Exception as e:  # the sweep numbers do not depend on the stand-ins
        out["cpu_stand_ins"] = f"unavailable: {e}"

    # ---- fp64 forward of one attention head at the mid-size graph's shape (time only: not a roofline target) ---
    from project_b200 import KIND_F64, KIND_U32, incoming_lists

    nodes, inner, width, directed = (512, 32, 8, 2000) if small else (19717, 500, 8, 88648)
    src = np.concatenate([rng.integers(0, nodes, size=directed), np.arange(nodes)]).astype(np.uint32)
    dst = np.concatenate([rng.integers(0, nodes, size=directed), np.arange(nodes)]).astype(np.uint32)
    order = np.argsort(dst, kind="stable")
    src, dst = src[order], dst[order]
    ptr, inc = incoming_lists(src, dst, nodes)
    feats = rng.exponential(1.0, size=(nodes, inner)) * (rng.random((nodes, inner)) < 0.1)
    up = lambda a, kind: be.upload(np.ascontiguousarray(a).reshape(-1), kind)
    args = (up(feats, KIND_F64), up(rng.uniform(-0.1, 0.1, size=(inner, width)), KIND_F64), up(rng.uniform(-1, 1, size=width), KIND_F64), 0.0,
            up(rng.uniform(-1, 1, size=width), KIND_F64), 0.0, up(np.zeros(width), KIND_F64), True, up(src, KIND_U32), up(dst, KIND_U32),
            nodes, inner, width, up(ptr, KIND_U32), up(inc, KIND_U32))
    trace = be.gat_head_forward(*args)

    def forward():
        be.gat_head_forward(*args, out=trace)
        be.synchronize()

    out["head_forward_fp64"] = {"nodes": nodes, "edges": int(src.size), "input_width": inner, "output_width": width, "ms": timed_ms(forward)}
    return out


def run_sweep_sharded(be, G, rank, world, device, small=False):
    """Sharded kernels over all ranks through the library's own communicator (gzk_comm_*): the row-sharded
    transform (two all-to-all exchanges), the point-range-sharded MSM (an all-gather of one point per rank),
    the row-sharded packed evaluation of an edge-shaped domain with the partial sums combined on the
    device, and - on 8 ranks - the evaluation phase of the 169k-node configuration, whose opened edge
    columns (294 x 2^26 rows) only fit when their rows are split over 8 GPUs.  Device-timed, max over ranks."""
    import torch
    import torch.distributed as dist

    from project_b200 import KIND_FR, KIND_FR_MONT, KIND_G1, KIND_I64, fr_sum, g1_sum, shard_rows
    from project_b200.lib import Comm

    stream = _stream_of(be, device)
    box = [Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Comm(be, world, rank, box[0])
    comm.set_timeout(120.0)
    be.set_deferred(True)

    def timed_ms(fn, reps=3):
        fn()
        be.synchronize()
        dist.barrier()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(reps):
            fn()
        stop.record(stream)
        be.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / reps], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def challenge(seed):
        c = np.zeros(32, dtype=np.uint8)
        c[:8] = np.frombuffer(np.uint64((0x9E3779B97F4A7C15 * seed) % (1 << 64) | 1).tobytes(), dtype=np.uint8)
        return c

    def all_ok(flag):
        verdict = torch.tensor([1 if flag else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)  # every rank learns the outcome: none is left waiting in a collective
        return int(verdict.item()) == 1

    out = {}
    # ---- row-sharded transform ---------------------------------------------------------------------------
    if world & (world - 1) == 0:
        lg = 14 if small else 24
        n = 1 << lg
        local = n // world
        vec = be.powers(challenge(100 + rank), local)
        work, res = be.alloc(KIND_FR_MONT, local), be.alloc(KIND_FR_MONT, local)
        ms = timed_ms(lambda: comm.ntt_sharded(vec, lg, work, res))
        # self-check without a CPU pass: X[0] (first element of rank 0's block) is the sum of all inputs
        sums = be.sumcheck_round_sums(vec, local)
        mine = be.upload(fr_sum(np.stack([sums[0], sums[1]])).reshape(1, 32), KIND_FR)
        total = be.alloc(KIND_FR, 1)
        comm.allgather_fr_sum(mine, 1, total)
        comm.wait()
        good = rank != 0 or np.array_equal(res.download(count=1)[0], total.download()[0])
        if not all_ok(good):
            raise RuntimeError("row-sharded transform: X[0] does not equal the sum of the inputs")
        out["ntt_sharded"] = {"log2n": lg, "ranks": world, "ms": ms, "GB_per_s": 2 * 32 * n / ms / 1e6, "field_mults_per_s": (n // 2) * lg / ms * 1e3,
                              "layout": "rows in, transposed out; 2 all-to-all exchanges inside gzk_ntt_sharded", "self_check": "ok"}
        for b in (vec, work, res):
            b.free()
    # ---- point-range-sharded MSM ---------------------------------------------------------------------------
    lg = 12 if small else 20
    n_local = 1 << lg
    scalars = be.powers(challenge(200 + rank), n_local)
    multipliers = be.powers(challenge(300 + rank), n_local)
    points = be.g1_fixed_base_mul(G, multipliers, n_local)
    table, wb = be.msm_precompute(points, n_local)  # each rank keeps the shifted copies of its own point range
    part_buf, all_buf = be.alloc(KIND_G1, 1), be.alloc(KIND_G1, world)

    def msm():
        part_buf.upload(be.msm_precomputed(scalars, table, n_local, wb).reshape(1, 96))
        comm.allgather(part_buf, 1, all_buf)
        comm.wait()
        return g1_sum(all_buf.download())

    ms = timed_ms(msm)
    out["msm_sharded"] = {"log2n_per_rank": lg, "ranks": world, "ms": ms, "Mpts_per_s": world * n_local / ms / 1e3,
                          "layout": "point range per rank, resident table of shifted bases, all-gather of one point per rank"}
    for b in (scalars, multipliers, points, table, part_buf, all_buf):
        b.free()

    # ---- row-sharded packed evaluation, partial sums combined on the device ----------------------------------
    def sharded_evaluation(log2n, k_field, k_int, label):
        n = 1 << log2n
        begin, end = shard_rows(n, world, rank, align=32)
        rows = end - begin
        w_first, w_count = (begin - 1) % n, min(rows + 1, n)
        cols = [be.powers(challenge(1000 + 17 * i + rank), rows) for i in range(k_field)]
        cols += [be.generated_column(1 + (i % 3), rows, 7 + i, rows, kind=KIND_I64) for i in range(k_int)]
        k = len(cols)
        tau = np.zeros(32, dtype=np.uint8)
        tau[0] = 28
        w_tau = be.bary_weights_range(log2n, tau, w_first, w_count)
        w_z = be.alloc(KIND_FR_MONT, w_count)
        partial, summed = be.alloc(KIND_FR_MONT, 4 * k), be.alloc(KIND_FR_MONT, 4 * k)
        counter = [0]

        def step():
            counter[0] += 1
            be.eval_batch_range_device(cols, rows, begin, log2n, w_tau, w_first, (0, 1), partial, 0)          # quotient: {tau, omega tau}
            be.bary_weights_range(log2n, challenge(5000 + counter[0]), w_first, w_count, out=w_z)              # fresh opening point
            be.eval_batch_range_device(cols, rows, begin, log2n, w_z, w_first, (0, 1), partial, 2 * k)        # openings: {z, omega z}
            comm.allgather_fr_sum(partial, 4 * k, summed)
            comm.wait()
            return summed.download()

        ms = timed_ms(step, reps=2)
        bytes_per_rank = sum(c.count * (8 if c.kind == KIND_I64 else 32) for c in cols)
        entry = {"domain": label, "log2n": log2n, "columns": k, "field_columns": k_field, "int64_columns": k_int, "ranks": world, "ms": ms,
                 "resident_GB_per_rank": bytes_per_rank / 1e9,
                 "step": "evaluation of every column at {tau, omega tau} and at a fresh {z, omega z} (weights at z computed per step), partial sums "
                         "summed over the ranks on the device (gzk_comm_allgather_fr_sum), one read-back"}
        for b in cols + [w_tau, w_z, partial, summed]:
            b.free()
        return entry

    try:
        out["eval_sharded_edge"] = sharded_evaluation(12 if small else 18, 8 if small else 375, 8 if small else 257, "edge domain of the mid-size configuration (632 opened columns, 2^18 rows)")
    except Exception as e:  # keep the other lines of the sweep
        out["eval_sharded_edge"] = f"failed: {e}"
    if world == 8 and not small:
        try:
            # the 169k-node configuration: 294 opened edge columns (about half of them small integers) x 2^26 rows
            out["b4_8gpu_evaluation"] = sharded_evaluation(26, 147, 147, "edge domain of the 169k-node configuration (294 opened columns, 2^26 rows)")
        except Exception as e:
            out["b4_8gpu_evaluation"] = f"failed: {e}"
    comm.close()
    return out

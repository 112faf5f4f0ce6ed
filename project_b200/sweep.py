"""Stand-alone kernels of the kernel sweep (MSM Mpts/s, NTT / fold GB/s, fp64 head forward), device-timed
with CUDA events on the backend's stream.  Measurement code used by bench.py; not on the proving path."""
import numpy as np


def _stream_of(be, device):
    import torch

    return torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", device))


def run_sweep(be, device, small=False):
    """Stand-alone kernels of the sweep at one representative size each (device-timed)."""
    import torch

    import pyref

    stream = _stream_of(be, device)
    rng = np.random.default_rng(1234)
    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()

    from project_b200 import KIND_FR

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

    def rand_fr(n):
        a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
        a[:, 31] &= 0x3F
        return a

    out = {}
    for lg in ((14,) if small else (20, 22)):
        n = 1 << lg
        scalars = be.upload(rand_fr(n), KIND_FR)
        points = be.g1_fixed_base_mul(G, be.upload(rand_fr(n), KIND_FR), n)
        ms = timed_ms(lambda: be.msm(scalars, points, n))
        entry = {"log2n": lg, "ms": ms, "Mpts_per_s": n / ms / 1e3}
        # the same MSM against the resident table of shifted bases (the SRS layout)
        table, wb = be.msm_precompute(points, n)
        ms = timed_ms(lambda: be.msm_precomputed(scalars, table, n, wb))
        entry["resident_table"] = {"window_bits": wb, "table_GB": table.count * 96 / 1e9, "ms": ms, "Mpts_per_s": n / ms / 1e3}
        out["msm" if lg <= 20 else f"msm_2p{lg}"] = entry
        for b in (scalars, points, table):
            b.free()
    lg = 14 if small else 22
    n = 1 << lg
    from project_b200 import KIND_FR_MONT

    vec = be.upload(rand_fr(n), KIND_FR)
    res = be.alloc(KIND_FR_MONT, n)
    ms = timed_ms(lambda: be.ntt(vec, lg, out=res))
    out["ntt"] = {"log2n": lg, "batch": 1, "ms": ms, "GB_per_s": 2 * 32 * n / ms / 1e6,
                  "field_mults_per_s": (n // 2) * lg / ms * 1e3}
    r = rand_fr(1)[0]
    ms = timed_ms(lambda: be.fold(vec, n, r, out=res))
    out["fold"] = {"log2n": lg, "ms": ms, "GB_per_s": 48 * n / ms / 1e6, "forms": "canonical table -> Montgomery output (2 multiplications per output)"}
    # a table kept in one form through the rounds of a sumcheck costs one multiplication per output
    half = be.alloc(KIND_FR, n // 2)
    ms = timed_ms(lambda: be.fold(vec, n, r, out=half))
    out["fold_same_form"] = {"log2n": lg, "ms": ms, "GB_per_s": 48 * n / ms / 1e6, "forms": "canonical table -> canonical output (1 multiplication per output)"}
    half.free()
    for b in (vec, res):
        b.free()
    # fp64 forward of one attention head at the mid-size graph's shape (time only: not a roofline target)
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

    ms = timed_ms(forward)
    out["head_forward_fp64"] = {"nodes": nodes, "edges": int(src.size), "input_width": inner, "output_width": width, "ms": ms}
    return out


def run_sweep_sharded(be, G, rank, world, device, small=False):
    """Sweep kernels over all ranks: the row-sharded transform (two all-to-all exchanges over
    NCCL) and the point-range-sharded MSM (one 96-byte all-gather); device-timed, max over ranks."""
    import torch
    import torch.distributed as dist

    from project_b200 import KIND_FR, KIND_FR_MONT, fr_sum, g1_sum
    from project_b200 import sharded_ntt as sn

    stream = _stream_of(be, device)

    rng = np.random.default_rng(1000 + rank)

    def rand_fr(n):
        a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
        a[:, 31] &= 0x3F
        return a

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

    out = {}
    if world & (world - 1) == 0:
        lg = 14 if small else 24
        n = 1 << lg
        local = n // world
        vec = be.upload(rand_fr(local), KIND_FR)
        work = (be.alloc(KIND_FR, local), be.alloc(KIND_FR_MONT, local))
        exchange = sn.NcclExchange(be, local, device)

        def transform():
            work[0].retag(KIND_FR)
            exchange.run(sn.forward(be, vec, lg, rank, world, work=work))

        ms = timed_ms(transform)
        # self-check without a CPU pass: X[0] (first element of rank 0's block) is the sum of all inputs
        sums = be.sumcheck_round_sums(vec, local)
        mine = torch.from_numpy(fr_sum(np.stack([sums[0], sums[1]]))).cuda()
        every = torch.empty((world, 32), dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(every, mine)
        good = 1
        if rank == 0 and not np.array_equal(work[1].download(count=1)[0], fr_sum(every.cpu().numpy())):
            good = 0
        verdict = torch.tensor([good], device="cuda", dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)  # every rank learns the outcome: none is left waiting in a collective
        if int(verdict.item()) == 0:
            raise RuntimeError("row-sharded transform: X[0] does not equal the sum of the inputs")
        be.timing_reset()
        be.timing_enable(True)
        transform()
        be.synchronize()
        families = {k: round(v[1], 3) for k, v in be.timing_report().items()}
        be.timing_enable(False)
        exchange.close()
        for b in work:
            b.free()
        out["ntt_sharded"] = {"log2n": lg, "ranks": world, "ms": ms, "GB_per_s": 2 * 32 * n / ms / 1e6,
                              "field_mults_per_s": (n // 2) * lg / ms * 1e3, "layout": "rows in, transposed out; 2 all-to-all exchanges",
                              "kernel_ms_one_transform": families}
        vec.free()
    lg = 12 if small else 20
    n_local = (1 << lg)
    scalars = be.upload(rand_fr(n_local), KIND_FR)
    points = be.g1_fixed_base_mul(G, be.upload(rand_fr(n_local), KIND_FR), n_local)

    table, wb = be.msm_precompute(points, n_local)  # each rank keeps the shifted copies of its own point range

    def msm():
        part = torch.from_numpy(be.msm_precomputed(scalars, table, n_local, wb).copy()).cuda()
        gathered = torch.empty((world, 96), dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(gathered, part)
        return g1_sum(gathered.cpu().numpy())

    ms = timed_ms(msm)
    out["msm_sharded"] = {"log2n_per_rank": lg, "ranks": world, "ms": ms, "Mpts_per_s": world * n_local / ms / 1e3,
                          "layout": "point range per rank, resident table of shifted bases, 96-byte all-gather"}
    scalars.free()
    points.free()
    table.free()
    return out



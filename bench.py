#!/usr/bin/env python
"""Benchmark of the B200 proving backend on the reference's headline metric.

Metric: commit+prove ms/proof.  A "step" is one pass of the data-parallel hot
path of commit + prove over one proof's worth of synthetic columns with the
domain sizes and column counts of the mid-size GAT configuration (N=19717
nodes: n_FH=2^24, n_edge=2^18, n_N=2^15, n_in=2^9, n_cat=2^7, n_d=2^4, n_C=2^3).
Per domain the step runs, through the C ABI of libgatzk_b200.so:
  commit     tau-evaluation of every committed column against resident w(tau)
  quotient   packed evaluation of all columns at {tau, omega*tau}
  open       barycentric weights at a fresh challenge z, then packed evaluation
             of all columns at {z, omega*z}
Host orchestration of the prover (transcript, label lists, scalar constraint
algebra) is O(#columns) and is not part of the step.

`value`   device-timed step with all columns resident in HBM.
`e2e`     same step through the same calls with the columns starting in pinned
          host memory: every step uploads them and reads the results back.
"""
import argparse
import concurrent.futures
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# (name, log2 n, committed/opened columns, valid rows) for the 19717-node config:
# 8 hidden heads (H), 8 output heads (K), 1 hidden layer (L); column counts per
# domain: FH 5, edge 43H+36K, in 3H, d 15H, cat 3L+3K, C 9K, N 18H+17K+L.
WORKLOAD_B2 = [
    ("FH", 24, 5, 19717 * 500),
    ("edge", 18, 632, 88648 + 19717),
    ("N", 15, 281, 19717),
    ("in", 9, 24, 500),
    ("cat", 7, 27, 64),
    ("d", 4, 120, 8),
    ("C", 3, 72, 3),
]
# reduced shapes for smoke-sized runs (--small)
WORKLOAD_SMALL = [("edge", 14, 64, 12000), ("N", 11, 32, 1500)]
# one edge-shaped domain, 512 MiB of columns: larger than L2, small enough for a profiler capture
WORKLOAD_PROFILE = [("edge", 18, 64, 88648 + 19717)]
METRIC = "commit+prove ms/proof"


def workload_terms(workload):
    """Field multiply-adds of one step: commit over the valid prefix, two 2-point
    evaluations over the whole domain."""
    return sum(k * valid + 4 * k * (1 << lg) for _, lg, k, valid in workload)


def workload_bytes(workload):
    """Algorithmic HBM bytes of the packed-evaluation launches of one step:
    every column once per launch plus the weight vector once per launch."""
    return sum(32 * (k * valid + valid) + 2 * 32 * (k + 1) * (1 << lg) for _, lg, k, valid in workload)


class ClockSampler:
    def __init__(self, device_index=0):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.device_index = device_index

    def _run(self):
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={fields}", "--format=csv,noheader,nounits", "-i", str(self.device_index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    parts = [p.strip() for p in out[0].split(",")]
                    self.samples.append(float(parts[0]))
                    self.max_mhz = float(parts[1])
                    for name, val in zip(names, parts[2:]):
                        if val.lower().startswith("active"):
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_count():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample(workload, threads, budget_columns=96, heads=16):
    """Times the CPU restatement of the reference loops on a bounded sample of the step and
    scales to a whole step: packed evaluation + weights by multiply-add count (all host
    threads, as the reference fans out), one column of every builder kind single-threaded
    (as the reference builds them) times the per-proof counts, and a sample of the same-base
    G1 batch.  Returns (ms_per_proof, description)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ora
    import pyref

    name, lg, k, valid = max((w for w in workload if w[1] <= 18), key=lambda w: w[1] * 1000 + w[2])
    ks = min(k, budget_columns)
    n = 1 << lg
    t_commit, _ = ora.bench_eval(ks, n, 1, threads, seed=1)
    t_eval, _ = ora.bench_eval(ks, n, 2, threads, seed=2)
    t_bary, _ = ora.bench_bary(n, threads, seed=3)
    sample_terms = ks * n * 1 + ks * n * 2
    per_term = (t_commit + t_eval) / sample_terms
    bary_per_row = t_bary / n
    eval_s = per_term * workload_terms(workload) + bary_per_row * sum(1 << w[1] for w in workload)
    # builders: per head 4 LogUp, 2+2 routes, 2 segmented states, 6 bindings (fold + inner product)
    node = min((w for w in workload), key=lambda w: abs(w[1] - 15))
    e_valid = min(valid, n - 1)
    tb = ora.bench_builders(n, e_valid, seed=4)
    nn = 1 << node[1]
    tn = ora.bench_builders(nn, min(node[3], nn - 1), seed=5)
    builders_s = heads * (4 * tb[0] + 2 * tn[1] + 2 * tb[2] + 2 * tb[3] + 6 * (tn[5] * 8 + tb[4] * 16 / max(e_valid, 1)))
    # same-base G1 batch: 16 scalar multiplications timed, scaled to the number of committed columns
    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8)
    rng = np.random.default_rng(6)
    sc = rng.integers(0, 256, size=(16, 32), dtype=np.uint8)
    sc[:, 31] &= 0x3F
    t0 = time.perf_counter()
    ora.g1_mul_same_base(G, sc)
    g1_s = (time.perf_counter() - t0) / 16 * sum(w[2] for w in workload) / max(1, threads)
    total = eval_s + builders_s + g1_s
    desc = (f"{name}-shaped sample: {ks} columns x 2^{lg} rows, 1- and 2-point packed evaluation ({sample_terms / 1e6:.0f}M mul-adds, "
            f"{t_commit + t_eval:.2f}s on {threads} threads) + barycentric weights 2^{lg} ({t_bary:.2f}s), scaled by multiply-add count "
            f"[{eval_s * 1e3:.0f} ms]; one column of each builder kind single-threaded x per-proof counts for {heads} heads "
            f"[{builders_s * 1e3:.0f} ms]; 16 double-and-add G1 multiplications scaled to the committed columns over {threads} threads "
            f"[{g1_s * 1e3:.0f} ms]")
    return total * 1e3, desc


def run_reference(args, workload, wl_name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = cpu_count()
    times = []
    desc = ""
    for i in range(args.warmup + args.steps):
        ms, desc = cpu_sample(workload, threads, budget_columns=32, heads=2 if (args.small or args.profile_case) else 16)
        if i >= args.warmup:
            times.append(ms)
    value = float(np.mean(times))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": value, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "u32x8 Montgomery Fr (BLS12-381)", "data": "synthetic",
        "config": {"workload": wl_name},
        "cpu_baseline": {"value": value, "unit": "ms", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)
    return 0


_RESULT_OUT = None


def claim_stdout():
    """Libraries (NCCL's version banner, for one) write to file descriptor 1; the result line
    must be the only thing there.  Keep a private copy of stdout for the result and point
    descriptor 1 at stderr for everything else."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
    return _RESULT_OUT


def emit(line):
    out = claim_stdout()
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced shapes (smoke runs)")
    ap.add_argument("--profile-case", action="store_true", help="one 2^18 x 64-column domain (profiler captures)")
    ap.add_argument("--builder-threads", type=int, default=4,
                    help="host threads (one context each) that issue the column builders of independent heads")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the MSM / NTT / fold kernel sweep lines")
    ap.add_argument("--sweep-only", action="store_true", help="only the MSM / NTT / fold sweep (profiler captures of those kernels)")
    args = ap.parse_args()
    workload = WORKLOAD_SMALL if args.small else (WORKLOAD_PROFILE if args.profile_case else WORKLOAD_B2)
    wl_name = ("reduced shapes (edge 2^14 x 64, N 2^11 x 32)" if args.small else
               "profiling case (edge 2^18 x 64 columns)" if args.profile_case else
               "mid-size GAT (N=19717, 8x8 hidden, 8x3 output) hot-path step: commit (tau-evaluation + same-base G1 batch) + quotient + opening "
               "evaluations over 7 domains, 1161 Fr columns, plus the column builders of 16 heads; inputs larger than L2")
    if args.impl == "reference":
        return run_reference(args, workload, wl_name)

    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import pyref
    from project_b200 import KIND_FR, KIND_FR_MONT, KIND_I64, KIND_U32, Backend, fr_sum, shard_rows

    be = Backend(local_rank)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local_rank))
    rng = np.random.default_rng(1234)
    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()
    heads = 2 if (args.small or args.profile_case) else 16
    if args.sweep_only:
        if world == 1:
            sweep = run_sweep(be, rng, G, stream, small=args.small)
        else:
            sweep = run_sweep_sharded(be, G, stream, rank, world, local_rank, small=args.small)
            dist.destroy_process_group()
        if rank == 0:
            emit({"sweep": sweep, "n_gpus": world})
        return 0

    # ---- resident inputs: every rank holds its ROW range of every column ---------------
    slabs = {}
    domains = []
    tau = np.zeros(32, dtype=np.uint8)
    tau[0] = 11 + 17  # KZG::setup: tau = seed + 17 with the config seed 11
    for name, lg, k, valid in workload:
        n = 1 << lg
        begin, end = shard_rows(n, world, rank, align=32) if world > 1 else (0, n)
        rows = end - begin
        if rows == 0:
            begin = 0  # a rank without rows of a tiny domain contributes zero partial sums
        if lg not in slabs:
            base = rng.integers(0, 256, size=(min(n, 1 << 22) * 2, 32), dtype=np.uint8)
            base[:, 31] &= 0x3F
            slabs[lg] = base
        base = slabs[lg]
        cols = []
        for i in range(k):
            buf = be.alloc(KIND_FR, max(rows, 1))
            done = 0
            while done < rows:
                part = min(rows - done, 1 << 22)
                off = ((i * 7919 + done) * 31) % (base.shape[0] - part + 1)
                buf.upload(base[off:off + part], offset=done)
                done += part
            cols.append(buf)
        d = {"name": name, "lg": lg, "n": n, "k": k, "valid": min(valid, n), "cols": cols, "begin": begin, "rows": rows}
        if world == 1:
            d["w_tau"] = be.bary_weights(lg, tau)
            d["w_z"] = be.alloc(KIND_FR_MONT, n)
        else:
            # weight slice with a one-row halo for the rotation by one; a rank that holds a
            # whole (tiny) domain keeps the whole vector
            d["w_first"] = (begin - 1) % n if rows + 1 <= n else 0
            d["w_count"] = min(rows + 1, n)
            d["w_tau"] = be.bary_weights_range(lg, tau, d["w_first"], d["w_count"])
            d["w_z"] = be.alloc(KIND_FR_MONT, d["w_count"])
        domains.append(d)

    # builder inputs (edge- and node-shaped columns of one head; reused for every head)
    edge = next((d for d in domains if d["name"] == "edge"), domains[0])
    node = next((d for d in domains if d["name"] == "N"), domains[-1])
    ne, nn = edge["n"], node["n"]
    e_valid, n_valid = min(edge["valid"], ne - 1), min(node["valid"], nn - 1)
    b_in = {
        "table": be.upload(rng.integers(-2048, 2048, size=ne, dtype=np.int64), KIND_I64),
        "query": be.upload(rng.integers(-2048, 2048, size=ne, dtype=np.int64), KIND_I64),
        "mult": be.upload(rng.integers(0, 64, size=ne, dtype=np.uint32), KIND_U32),
        "q_table": be.upload((np.arange(ne) < 4096).astype(np.uint32), KIND_U32),
        "q_query": be.upload((np.arange(ne) < e_valid).astype(np.uint32), KIND_U32),
        "q_new": be.upload((rng.random(ne) < 0.15).astype(np.uint32), KIND_U32),
        "values": be.upload(rng.integers(0, 4096, size=ne, dtype=np.int64), KIND_I64),
        "node_vals": be.upload(rng.integers(-4096, 4096, size=nn, dtype=np.int64), KIND_I64),
        "src": be.upload(rng.integers(0, n_valid, size=ne, dtype=np.int64).astype(np.uint32), KIND_U32),
        "hits": be.upload(rng.integers(0, 4096, size=e_valid, dtype=np.int64).astype(np.uint32), KIND_U32),
        "matrix": be.upload(rng.integers(-4096, 4096, size=n_valid * 8, dtype=np.int64), KIND_I64),
        "node_tab": be.upload(rng.integers(0, 1 << 20, size=nn, dtype=np.int64), KIND_I64),
        "node_mult": be.upload(rng.integers(0, 64, size=nn, dtype=np.uint32), KIND_U32),
    }
    w_node = be.bary_weights(node["lg"], tau)
    be.synchronize()
    # builder calls queue their kernels and return; calls that hand values to the host
    # (evaluations, the inner-product total) still synchronise, and a device-side error of
    # a queued call is raised by the synchronize that ends the builder phase
    be.set_deferred(True)
    step_counter = [0]

    def challenge():
        step_counter[0] += 1
        z = np.zeros(32, dtype=np.uint8)
        z[:8] = np.frombuffer(np.uint64((0x9E3779B97F4A7C15 * step_counter[0]) % (1 << 64) | 1).tobytes(), dtype=np.uint8)
        return z

    def gather_sum(partial):
        """all-gather the per-rank partial sums (a few KB) over NCCL and add them mod r"""
        if world == 1:
            return partial
        t = torch.from_numpy(partial).cuda()
        out = torch.empty((world,) + tuple(t.shape), dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(out, t)
        return fr_sum(out.cpu().numpy())

    def evaluate(d, weights, length, rotations, w=None):
        w = w or be
        if world == 1:
            return w.eval_batch(d["cols"], length, d["lg"], weights, rotations)
        local_len = max(0, min(length - d["begin"], d["rows"]))
        return gather_sum(w.eval_batch_range(d["cols"], local_len, d["begin"], d["lg"], weights, d["w_first"], rotations))

    def step_domain(d, w=None):
        w = w or be
        outs = []
        tau_evals = evaluate(d, d["w_tau"], d["valid"], (0,), w)[0]
        outs.append(w.g1_mul_same_base(G, tau_evals))                          # commit: [p_k(tau)] G
        outs.append(evaluate(d, d["w_tau"], d["n"], (0, 1), w))                # quotient: {tau, omega*tau}
        z = challenge()
        if world == 1:
            w.bary_weights(d["lg"], z, out=d["w_z"])
        else:
            w.bary_weights_range(d["lg"], z, d["w_first"], d["w_count"], out=d["w_z"])
        outs.append(evaluate(d, d["w_z"], d["n"], (0, 1), w))                  # openings: {z, omega*z}
        return outs

    one_at_a_time = [False]  # set for the pass that times each kernel by itself

    def local_eval(d, weights, length, rotations, w):
        if world == 1:
            return w.eval_batch(d["cols"], length, d["lg"], weights, rotations)
        local_len = max(0, min(length - d["begin"], d["rows"]))
        return w.eval_batch_range(d["cols"], local_len, d["begin"], d["lg"], weights, d["w_first"], rotations)

    def phase(fn):
        """fn(domain, worker context) over all domains -> {domain name: result}.  The reference
        evaluates its seven domains from seven concurrent host tasks (one std::async per domain
        bundle); here the domains are dealt to the worker contexts the same way, so the launch
        and read-back latencies of the small domains hide behind the kernels of the large ones."""
        if pool is None or one_at_a_time[0]:
            return {d["name"]: fn(d, be) for d in domains}

        def run_group(t):
            return [(d["name"], fn(d, workers[t])) for d in domain_groups[t]]

        out = {}
        for f in [pool.submit(run_group, t) for t in range(n_workers)]:
            out.update(f.result())
        return out

    def gather_all(parts):
        """One all-gather per protocol barrier: the partial sums of every domain travel together
        (K*P*32 bytes per domain) and are added mod r; issued from the main thread only."""
        if world == 1:
            return parts
        names = [d["name"] for d in domains]
        flat = np.concatenate([parts[name].reshape(-1, 32) for name in names])
        summed = gather_sum(flat)
        out, at = {}, 0
        for name in names:
            count = parts[name].size // 32
            out[name] = summed[at:at + count].reshape(parts[name].shape)
            at += count
        return out

    def step_evaluations():
        # barrier 1: tau-evaluations of every column (valid prefix), then the commitments [p_k(tau)] G
        tau_evals = gather_all(phase(lambda d, w: local_eval(d, d["w_tau"], d["valid"], (0,), w)))
        commits = phase(lambda d, w: w.g1_mul_same_base(G, tau_evals[d["name"]][0]))
        # barrier 2: quotient evaluations at {tau, omega*tau}
        quotient = gather_all(phase(lambda d, w: local_eval(d, d["w_tau"], d["n"], (0, 1), w)))
        # barrier 3: fresh weights at the challenge z, openings at {z, omega*z}
        z = challenge()

        def open_domain(d, w):
            if world == 1:
                w.bary_weights(d["lg"], z, out=d["w_z"])
            else:
                w.bary_weights_range(d["lg"], z, d["w_first"], d["w_count"], out=d["w_z"])
            return local_eval(d, d["w_z"], d["n"], (0, 1), w)

        opened = gather_all(phase(open_domain))
        return commits, quotient, opened

    # The reference builds the columns of a proof from concurrent host tasks (std::async per
    # head / per column); the same shape here: a few host threads, each with its own context
    # (its own stream and scratch), so the short builder kernels of independent heads overlap
    # on the GPU.  Builder outputs are allocated once per worker: the columns of a proof live
    # in the backend's pool.
    n_workers = max(1, args.builder_threads)
    workers = [be] + [Backend(local_rank) for _ in range(n_workers - 1)]
    for w in workers[1:]:
        w.set_deferred(True)
    w_nodes = [w_node] + [w.bary_weights(node["lg"], tau) for w in workers[1:]]
    for w in workers:
        w.synchronize()

    def make_outputs(w):
        return {
            "edge_mont": [w.alloc(KIND_FR_MONT, ne) for _ in range(3)],
            "node_mont": w.alloc(KIND_FR_MONT, nn),
            "edge_i64": w.alloc(KIND_I64, ne),
            "hist": w.alloc(KIND_U32, 4096),
            "folded": w.alloc(KIND_FR, 8),
            "acc16": w.alloc(KIND_FR_MONT, 16),
        }

    w_outs = [make_outputs(w) for w in workers]
    pool = concurrent.futures.ThreadPoolExecutor(max_workers=n_workers) if n_workers > 1 else None
    # domains dealt to the workers, largest first, each to the least loaded worker
    domain_groups = [[] for _ in range(n_workers)]
    loads = [0] * n_workers
    for d in sorted(domains, key=lambda d: -d["k"] * d["n"]):
        t = loads.index(min(loads))
        domain_groups[t].append(d)
        loads[t] += d["k"] * d["n"] + (1 << 22)

    def build_heads(t, beta, my_heads):
        # column builders of the heads dealt to worker t (heads are independent)
        w, b_out, wn = workers[t], w_outs[t], w_nodes[t]
        e_out = b_out["edge_mont"]
        for head in my_heads:
            for i in range(4):  # feature / LeakyReLU / range / exp lookups
                w.logup_accumulator(b_in["table"], b_in["query"], b_in["mult"], b_in["q_table"], b_in["q_query"], ne, beta, e_valid, out=e_out[i % 3])
            for i in range(2):  # src / dst routes
                w.route_node_accumulator(b_in["node_tab"], b_in["node_mult"], n_valid, nn, beta, out=b_out["node_mont"])
                w.route_edge_accumulator(b_in["query"], e_valid, ne, beta, out=e_out[i])
            for i in range(2):  # PSQ state, max counter
                w.group_prefix_state(b_in["values"], b_in["q_new"], ne, out=e_out[i])
            for _ in range(5):  # E_src, E_dst, M, Sum, inv broadcast to edges
                w.broadcast_node_values(b_in["node_vals"], nn, b_in["src"], e_valid, ne, out=b_out["edge_i64"])
            for _ in range(3):
                w.histogram(b_in["hits"], e_valid, 4096, out=b_out["hist"])
            for _ in range(6):  # bindings: fold rows by weights, then the running inner product
                w.fold_rows(b_in["matrix"], n_valid, 8, wn, n_valid, out=b_out["folded"])
                w.zkmap_accumulator(b_out["folded"], b_out["folded"], 8, 16, out=b_out["acc16"])
            w.weighted_sum(b_in["table"], beta, b_in["query"], e_valid, ne, out=e_out[2])
        w.synchronize()

    def step_builders():
        beta = challenge()
        mine = list(range(rank, heads, world))
        if pool is None or one_at_a_time[0]:
            build_heads(0, beta, mine)
            return
        futures = [pool.submit(build_heads, t, beta, mine[t::n_workers]) for t in range(n_workers)]
        for f in futures:
            f.result()

    def step_resident():
        step_builders()
        return step_evaluations()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        be.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        for w in workers:
            w.timing_reset()
            w.timing_enable(True)
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(steps):
                fn()
            stop.record(stream)
            barrier()
        ms = start.elapsed_time(stop)
        report = {}
        for w in workers:
            for kname, (count, total_ms) in w.timing_report().items():
                prev = report.get(kname, (0, 0.0))
                report[kname] = (prev[0] + count, prev[1] + total_ms)
            w.timing_enable(False)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, report, clocks.summary()

    ms_total, report_overlapped, clocks = timed(step_resident, args.steps, args.warmup)
    ms_per_step = ms_total / args.steps
    launches = sum(v[0] for v in report_overlapped.values())
    # Per-kernel durations: in the timed region kernels of independent heads and domains run
    # side by side, so a kernel's event-to-event time there includes its neighbours.  The
    # roofline needs the kernel by itself: the same steps once more, issued from one thread.
    iso_steps = args.steps
    if n_workers > 1:
        one_at_a_time[0] = True
        iso_steps = max(1, min(args.steps, 3))
        _, report, _ = timed(step_resident, iso_steps, 1)
        one_at_a_time[0] = False
    else:
        report = report_overlapped

    # ---- roofline of the dominant kernel (packed evaluation) ----------------------------
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            peak = float(json.load(f)["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    eval_ms = sum(v[1] for kname, v in report.items() if kname.startswith("eval_partial"))
    eval_launches = sum(v[0] for kname, v in report.items() if kname.startswith("eval_partial"))
    local_workload = [(d["name"], d["lg"], d["k"], max(0, min(d["valid"] - d["begin"], d["rows"]))) for d in domains]
    local_rows = {d["name"]: d["rows"] for d in domains}
    local_bytes = sum(32 * (k * valid + valid) + 2 * 32 * (k + 1) * local_rows[name] for name, lg, k, valid in local_workload)
    local_terms = sum(k * valid + 4 * k * local_rows[name] for name, lg, k, valid in local_workload)
    achieved = local_bytes * iso_steps / (eval_ms * 1e-3) / 1e9 if eval_ms > 0 else 0.0
    from project_b200.lib import measure_mac_peak

    mac_peak = measure_mac_peak(local_rank, 2, 20000)
    products_per_s = local_terms * iso_steps / (eval_ms * 1e-3) if eval_ms > 0 else 0.0
    roofline = {
        "bound": "hbm", "kernel": "eval_partial_kernel (packed evaluation, all launches of a step; durations from the one-thread pass, each launch by itself)", "achieved": achieved,
        "peak": peak, "unit": "GB/s", "frac": achieved / peak if peak else None, "traffic": 560.1e6 + 5.4e6,
        "traffic_note": "ncu dram read+write of one 2-rotation launch on the 2^18 x 64 profiling case (algorithmic 545.3e6, traffic grows in proportion to columns x rows); see profiles/eval_partial_kernel_edge2p18x64.md",
        "peak_source": peak_src, "launches": eval_launches, "avg_launch_ms": eval_ms / max(1, eval_launches),
        "bytes_per_step": local_bytes,
        "integer_pipe": {"achieved_products_per_s": products_per_s, "measured_peak_products_per_s": mac_peak,
                         "frac": products_per_s / mac_peak if mac_peak else None,
                         "note": "the kernel's binding roof: 64 32x32 limb products per 32-byte term; peak measured in this run on register operands"},
    }

    # ---- end to end: columns start in pinned host memory --------------------------------
    e2e = None
    if not args.no_e2e:
        pinned = {}
        for d in domains:
            rows = min(max(d["rows"], 1), 1 << 22)
            t = torch.empty((rows, 32), dtype=torch.uint8, pin_memory=True)
            t.numpy()[:] = slabs[d["lg"]][:rows]
            pinned[d["name"]] = t
        h2d = sum(d["k"] * d["rows"] * 32 for d in domains) * world
        d2h = sum(d["k"] * (5 * 32 + 96) for d in domains)

        def queue_uploads(d):
            host = pinned[d["name"]].numpy()
            for buf in d["cols"]:
                done = 0
                while done < d["rows"]:
                    part = min(d["rows"] - done, host.shape[0])
                    buf.upload_async(host[:part], offset=done)
                    done += part

        # Columns are independent, so a domain is uploaded and evaluated in groups of columns: the
        # evaluation of one group runs while the next group travels, and only the last group's
        # kernels are left after the last byte has arrived.
        group_columns = 96
        units = []
        for d in domains:
            for first in range(0, len(d["cols"]), group_columns):
                units.append(dict(d, cols=d["cols"][first:first + group_columns]))

        def step_e2e():
            # uploads run on the copy stream; the first one overlaps with the builders
            outs = []
            queue_uploads(units[0])
            step_builders()
            for i, u in enumerate(units):
                be.copy_fence()
                if i + 1 < len(units):
                    queue_uploads(units[i + 1])
                outs.append(step_domain(u))
            return outs

        e2e_steps = max(1, min(args.steps, 3))
        e2e_ms, _, _ = timed(step_e2e, e2e_steps, 1)
        e2e = {"value": e2e_ms / e2e_steps, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}

    # ---- kernel sweep (single GPU): MSM Mpts/s, NTT GB/s, fold GB/s ------------------------
    sweep = None
    if world == 1 and not args.no_sweep and not args.profile_case:
        sweep = run_sweep(be, rng, G, stream, small=args.small)
    elif world > 1 and not args.no_sweep and not args.profile_case:
        sweep = run_sweep_sharded(be, G, stream, rank, world, local_rank, small=args.small)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = cpu_count()
        v, desc = cpu_sample(workload, threads, heads=heads)
        cpu_baseline = {"value": v, "unit": "ms", "cores": threads, "kind": "port", "sample": desc}

    if rank == 0:
        line = {
            "metric": METRIC, "value": ms_per_step, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32x8 Montgomery Fr / u32x12 Fp (BLS12-381)", "data": "synthetic",
            "config": {"workload": wl_name, "l2": "inputs larger than L2 (5.3 GB edge columns, 2.7 GB FH columns per pass)",
                       "sharding": f"rows of every domain split across {world} rank(s); one all-gather of the partial sums (K*P*32 B per domain) over NCCL at each of the 3 protocol barriers; "
                                   f"builder heads dealt round-robin",
                       "builder_threads": n_workers},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches,
            "kernel_ms": {k: round(v[1] / iso_steps, 3) for k, v in report.items()},
            "kernel_ms_note": "per step, each kernel family by itself (a pass issued from one host thread after the timed region)", "clocks": clocks, "sweep": sweep,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_sweep(be, rng, G, stream, small=False):
    """Stand-alone kernels of the sweep at one representative size each (device-timed)."""
    import torch

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


def run_sweep_sharded(be, G, stream, rank, world, device, small=False):
    """Sweep kernels over all ranks: the row-sharded transform (two all-to-all exchanges over
    NCCL) and the point-range-sharded MSM (one 96-byte all-gather); device-timed, max over ranks."""
    import torch
    import torch.distributed as dist

    from project_b200 import KIND_FR, KIND_FR_MONT, fr_sum, g1_sum
    from project_b200 import sharded_ntt as sn

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


if __name__ == "__main__":
    sys.exit(main())

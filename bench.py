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


def cpu_sample(workload, threads, budget_columns=96):
    """Times the CPU restatement of the reference loops on a bounded sample of the
    step (the edge-shaped domain, `budget_columns` columns) and scales by the
    multiply-add count to a whole step.  Returns (ms_per_proof, description)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ora

    name, lg, k, valid = max((w for w in workload if w[1] <= 18), key=lambda w: w[1] * 1000 + w[2])
    ks = min(k, budget_columns)
    n = 1 << lg
    t_commit, _ = ora.bench_eval(ks, n, 1, threads, seed=1)
    t_eval, _ = ora.bench_eval(ks, n, 2, threads, seed=2)
    t_bary, _ = ora.bench_bary(n, threads, seed=3)
    sample_terms = ks * n * 1 + ks * n * 2
    per_term = (t_commit + t_eval) / sample_terms
    bary_per_row = t_bary / n
    total = per_term * workload_terms(workload) + bary_per_row * sum(1 << w[1] for w in workload)
    desc = (f"{name}-shaped sample: {ks} columns x 2^{lg} rows, 1- and 2-point packed evaluation "
            f"({sample_terms / 1e6:.0f}M mul-adds, {t_commit + t_eval:.2f}s) + barycentric weights 2^{lg} ({t_bary:.2f}s), "
            f"scaled by multiply-add count to one step")
    return total * 1e3, desc


def run_reference(args, workload, wl_name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = cpu_count()
    times = []
    desc = ""
    for i in range(args.warmup + args.steps):
        ms, desc = cpu_sample(workload, threads, budget_columns=32)
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
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced shapes (smoke runs)")
    ap.add_argument("--profile-case", action="store_true", help="one 2^18 x 64-column domain (profiler captures)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    workload = WORKLOAD_SMALL if args.small else (WORKLOAD_PROFILE if args.profile_case else WORKLOAD_B2)
    wl_name = ("reduced shapes (edge 2^14 x 64, N 2^11 x 32)" if args.small else
               "profiling case (edge 2^18 x 64 columns)" if args.profile_case else
               "mid-size GAT (N=19717, 8x8 hidden, 8x3 output) hot-path step: commit + quotient + opening evaluations over 7 domains, "
               "1161 Fr columns, inputs larger than L2")
    if args.impl == "reference":
        return run_reference(args, workload, wl_name)

    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from project_b200 import KIND_FR, KIND_FR_MONT, Backend

    be = Backend(local_rank)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local_rank))
    rng = np.random.default_rng(1234 + rank)

    # Shard: with N ranks every rank takes a contiguous 1/N slice of the columns of
    # every domain (independent inner products, no data-path collective).
    def my_columns(k):
        lo = (k * rank) // world
        hi = (k * (rank + 1)) // world
        return hi - lo

    # ---- resident inputs ----------------------------------------------------------
    slabs = {}
    domains = []
    tau = np.zeros(32, dtype=np.uint8)
    tau[0] = 11 + 17  # KZG::setup: tau = seed + 17 with the config seed 11
    for name, lg, k, valid in workload:
        n = 1 << lg
        kk = my_columns(k)
        if lg not in slabs:
            base = rng.integers(0, 256, size=(min(n, 1 << 22) * 4, 32), dtype=np.uint8)
            base[:, 31] &= 0x3F
            slabs[lg] = base
        base = slabs[lg]
        cols = []
        for i in range(kk):
            buf = be.alloc(KIND_FR, n)
            off = (i * 7919) % (base.shape[0] - min(n, 1 << 22) + 1) if n <= (1 << 22) else 0
            if n <= (1 << 22):
                buf.upload(base[off:off + n])
            else:
                for part in range(n >> 22):
                    o2 = ((i + part) * 104729) % (base.shape[0] - (1 << 22) + 1)
                    buf.upload(base[o2:o2 + (1 << 22)], offset=part << 22)
            cols.append(buf)
        w_tau = be.bary_weights(lg, tau)
        w_z = be.alloc(KIND_FR_MONT, n)
        domains.append({"name": name, "lg": lg, "n": n, "k": kk, "valid": min(valid, n), "cols": cols, "w_tau": w_tau, "w_z": w_z})
    be.synchronize()

    step_counter = [0]

    def challenge():
        step_counter[0] += 1
        z = np.zeros(32, dtype=np.uint8)
        z[:8] = np.frombuffer(np.uint64(0x9E3779B97F4A7C15 * step_counter[0] % (1 << 64) | 1).tobytes(), dtype=np.uint8)
        return z

    def step_resident():
        outs = []
        for d in domains:
            if d["k"] == 0:
                continue
            outs.append(be.eval_batch(d["cols"], d["valid"], d["lg"], d["w_tau"], (0,)))
            outs.append(be.eval_batch(d["cols"], d["n"], d["lg"], d["w_tau"], (0, 1)))
            be.bary_weights(d["lg"], challenge(), out=d["w_z"])
            outs.append(be.eval_batch(d["cols"], d["n"], d["lg"], d["w_z"], (0, 1)))
        return outs

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()
        be.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        be.timing_reset()
        be.timing_enable(True)
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(steps):
                fn()
            stop.record(stream)
            barrier()
        ms = start.elapsed_time(stop)
        report = be.timing_report()
        be.timing_enable(False)
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, report, clocks.summary()

    ms_total, report, clocks = timed(step_resident, args.steps, args.warmup)
    ms_per_step = ms_total / args.steps
    launches = sum(v[0] for v in report.values())

    # roofline of the dominant kernel family (packed evaluation, 2-point)
    fam = max(report.items(), key=lambda kv: kv[1][1])[0]
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            peak = float(json.load(f)["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    eval_ms = sum(v[1] for kname, v in report.items() if kname.startswith("eval_partial"))
    eval_launches = sum(v[0] for kname, v in report.items() if kname.startswith("eval_partial"))
    local_workload = [(d["name"], d["lg"], d["k"], d["valid"]) for d in domains if d["k"] > 0]
    eval_bytes = workload_bytes(local_workload) * args.steps
    achieved = eval_bytes / (eval_ms * 1e-3) / 1e9 if eval_ms > 0 else 0.0
    roofline = {
        "bound": "hbm", "kernel": "eval_partial_kernel (packed evaluation, all launches of the step)", "achieved": achieved,
        "peak": peak, "unit": "GB/s", "frac": achieved / peak if peak else None, "traffic": None,
        "peak_source": peak_src, "launches": eval_launches, "avg_launch_ms": eval_ms / max(1, eval_launches),
        "bytes_per_step": workload_bytes(local_workload),
        "field_muladds_per_s": workload_terms(local_workload) * args.steps / (eval_ms * 1e-3) if eval_ms > 0 else None,
    }

    # ---- end to end: columns start in pinned host memory ---------------------------
    e2e = None
    if not args.no_e2e:
        pinned = {}
        for d in domains:
            if d["k"] == 0:
                continue
            rows = min(d["n"], 1 << 22)
            t = torch.empty((rows, 32), dtype=torch.uint8, pin_memory=True)
            src = slabs[d["lg"]]
            t.numpy()[:] = src[:rows]
            pinned[d["name"]] = t
        h2d = sum(d["k"] * d["n"] * 32 for d in domains)
        d2h = sum(d["k"] * 5 * 32 for d in domains)

        def step_e2e():
            for d in domains:
                if d["k"] == 0:
                    continue
                host = pinned[d["name"]].numpy()
                rows = host.shape[0]
                for buf in d["cols"]:
                    for part in range(0, d["n"], rows):
                        buf.upload(host, offset=part)
            return step_resident()

        e2e_ms, _, _ = timed(step_e2e, max(1, min(args.steps, 3)), 1)
        e2e = {"value": e2e_ms / max(1, min(args.steps, 3)), "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = cpu_count()
        v, desc = cpu_sample(workload, threads)
        cpu_baseline = {"value": v, "unit": "ms", "cores": threads, "kind": "port", "sample": desc}

    if rank == 0:
        line = {
            "metric": METRIC, "value": ms_per_step, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32x8 Montgomery Fr (BLS12-381)", "data": "synthetic",
            "config": {"workload": wl_name, "l2": "inputs larger than L2 (5.3 GB edge columns, 2.7 GB FH columns per pass)",
                       "sharding": f"columns of every domain split across {world} rank(s), no data-path collective"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches,
            "kernel_ms": {k: round(v[1], 3) for k, v in report.items()}, "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

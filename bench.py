#!/usr/bin/env python
"""Benchmark of the B200 proving backend on the reference's headline metric.

Metric: commit+prove ms/proof.  A "step" is ONE proof: the whole commit + prove flow of the
multi-head GAT prover (project_b200/host/prover_flow.hpp).  The default workload is the
configuration the metric is quoted on, the 169k-node citation-style GAT (N=169343, about 2.5 M
edges with self loops, 128 features, two hidden layers of 3 heads x 256, one output head of 40
classes; domains n_FH=2^25, n_edge=2^26, n_N=2^18, n_in=2^10, n_cat=2^10, n_d=2^9, n_C=2^6): with
the edge-domain columns stored as prefixes it fits one GPU.  The mid-size configuration (b2:
N=19717, 8x8 hidden, 8x3 output) is measured beside it in `b2`.  The flow follows the reference's
schedule: fp64 forward pass and quantised witness of every head, then ONE Fiat-Shamir transcript
over the heads in order, per head the commit barriers of the reference (every barrier reads its
commitment points back to the host, hashes them and only then builds the next columns), then the
quotient evaluations at {tau, omega*tau}, fresh barycentric weights at the opening challenges and
the evaluations at {z, omega*z}.

`value`   device-timed step with the feature matrix already in HBM.
`e2e`     the same call with the feature matrix and the model parameters uploaded from host memory
          every step (results always come back to the host: that is how the transcript advances).
`--impl reference`  the same flow over the CPU restatement (oracle/), all host threads.  For b2
          and small: the whole workload every step.  For b4 (about seven minutes and 150 GB per
          proof on 16 cores): the same model on a graph of 1/16 of the nodes and edges, whole flow
          every step, time scaled by 16 (the flow's cost is linear in nodes and edges: measured
          26.3 s at 1/16 and 103.7 s at 1/4 on 16 cores).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "commit+prove ms/proof"
WORKLOADS = {
    # the configuration the metric is quoted on: citation-style graph, power-law out-degree, symmetrised, dense Gaussian features
    "b4": dict(seed=11, nodes=169343, directed_edges=1166243, feature_count=128, hidden=[(3, 256), (3, 256)], output_heads=1, class_count=40,
               power_law=True, symmetrize=True, feature_kind="gauss"),
    # mid-size GAT of the configuration list: power-law graph, 10 % dense exponential features
    "b2": dict(seed=11, nodes=19717, directed_edges=88648, feature_count=500, hidden=[(8, 8)], output_heads=8, class_count=3, density=0.1,
               power_law=True),
    # reduced shapes for smoke-sized runs and profiler captures
    "small": dict(seed=11, nodes=1500, directed_edges=6000, feature_count=64, hidden=[(2, 8)], output_heads=2, class_count=3, density=0.1,
                  power_law=True),
}
# workloads whose edge-domain columns are stored as prefixes (whole-domain vectors would not fit one device)
COMPACT = {"b4"}
# the CPU arm of b4 runs the same model on 1/CPU_SAMPLE_DIVISOR of the nodes and edges and scales the time
CPU_SAMPLE_DIVISOR = 16
WORKLOAD_NAMES = {
    "b4": "169k-node citation-style GAT (N=169343, 2.5M edges with self loops, 128 features, (3+3)x256 hidden, 1x40 output): one full "
          "commit+prove flow per step, 575 dynamic commitments, 40 Fiat-Shamir-chained commit barriers, 7 domains (FH 2^25, edge 2^26, N 2^18), "
          "edge-domain columns stored as prefixes",
    "b2": "mid-size GAT (N=19717, 500 features, 8x8 hidden, 8x3 output): one full commit+prove flow per step, 1212 dynamic commitments, "
          "69 Fiat-Shamir-chained commit barriers, 7 domains (FH 2^24, edge 2^18, N 2^15)",
    "small": "reduced shapes (N=1500, 64 features, 2x8 hidden, 2x3 output), same flow",
}


def cpu_sample_inputs(workload, proofs=1):
    """Inputs of the CPU arm and the factor its time is multiplied by.  The b4 sample shrinks further when many proofs are
    asked for, so that the whole run stays within a few minutes (a 1/16 graph takes about 26 s per proof on 16 cores)."""
    from project_b200 import synthetic

    shape = dict(WORKLOADS[workload])
    if workload != "b4":
        return synthetic.make_inputs(**shape), 1
    divisor = CPU_SAMPLE_DIVISOR if proofs <= 8 else 2 * CPU_SAMPLE_DIVISOR if proofs <= 16 else 4 * CPU_SAMPLE_DIVISOR
    shape["nodes"] //= divisor
    shape["directed_edges"] //= divisor
    return synthetic.make_inputs(**shape), divisor


def cpu_sample_text(workload, stats, threads, divisor=CPU_SAMPLE_DIVISOR):
    if workload == "b4":
        return (f"the whole commit+prove flow ({stats['dynamic_commitments']} commitments, {stats['commit_barriers']} barriers) of the same model on a "
                f"graph of 1/{divisor} of the nodes and edges ({WORKLOADS['b4']['nodes'] // divisor} nodes), over the CPU "
                f"restatement, {threads} host threads; time multiplied by {divisor} (cost linear in nodes and edges: 26.3 s at 1/16, "
                f"103.7 s at 1/4 measured on 16 cores; the full size needs about 150 GB of host memory and seven minutes per proof)")
    return (f"full workload every step: the whole commit+prove flow ({stats['dynamic_commitments']} commitments, {stats['commit_barriers']} barriers) "
            f"over the CPU restatement of the reference's leaves, {threads} host threads where the reference fans out, builders serial per column")


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


def generator_bytes():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import pyref

    return np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()


def config_of(args, world):
    return {"workload": WORKLOAD_NAMES[args.workload], "schedule": "fs_chain",
            "l2": "inputs larger than L2 (the columns of one proof are several GB; every barrier streams fresh columns)",
            "sharding": "one proof per rank (independent proofs, no data-path collective)" if world > 1 else "single GPU"}


def cpu_flow_run(inputs, steps, warmup, threads, compact=False):
    """The flow over the CPU restatement, whole workload every step.  Returns (mean ms per proof, per-step list, stats)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ora
    from project_b200.flow import Flow

    flow = Flow(ora.lib(), "ora_flow_", threads, inputs, generator_bytes(), compact_columns=compact)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        flow.prove()
        if i >= warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    stats = flow.stats()
    flow.close()
    return float(np.mean(times)), times, stats


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = cpu_count()
    warmup = args.warmup if args.workload != "b4" else min(args.warmup, 1)  # the CPU flow has no warm-up effect worth 26 s a step
    inputs, factor = cpu_sample_inputs(args.workload, proofs=args.steps + warmup)
    value, times, stats = cpu_flow_run(inputs, args.steps, warmup, threads, compact=args.workload in COMPACT)
    value *= factor
    sample = cpu_sample_text(args.workload, stats, threads, factor)
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup,
        "ms_per_step": value, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "u32x8 Montgomery Fr / u32x12 Fp (BLS12-381)", "data": "synthetic", "config": config_of(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": "ms", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
        "step_ms": [round(t * factor, 1) for t in times],
    })
    return 0


def self_check(flow, ora, columns=8):
    """After the timed region: tau-evaluations of committed N-domain and edge-domain columns recomputed by
    the CPU restatement from the columns themselves and compared with what the flow committed to."""
    listing = {}
    for line in flow.dump().splitlines():
        parts = line.split(" ")
        if parts[0] == "tau_eval":
            listing[parts[1]] = parts[2]
    tau = np.zeros(32, dtype=np.uint8)
    tau[0] = 11 + 17
    sizes = flow.stats()["domains"]
    checked = 0
    for domain in ("N", "edge"):
        n = sizes[domain]
        if n > (1 << 18):
            continue
        weights = ora.bary_weights(tau, n)
        labels = flow.domain_labels(domain)
        step = max(1, len(labels) // columns)
        for label in labels[::step][:columns]:
            kind, values = flow.column(label)
            if kind in (2, 3):
                values = ora.fr_from_i64(values.astype(np.int64))
            want = ora.commit_tau_eval(values[None, :, :].copy(), weights[:values.shape[0]].copy())[0]
            if want.tobytes().hex() != listing[label]:
                return f"mismatch in {label}"
            checked += 1
    return "ok" if checked >= columns else f"only {checked} columns checked"


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="b4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-b2", action="store_true", help="skip the mid-size configuration measured beside b4")
    ap.add_argument("--small", action="store_true", help="same as --workload small")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-msm", action="store_true", help="skip the MSM-commitment measurement")
    ap.add_argument("--no-sweep", action="store_true", help="skip the MSM / NTT / fold kernel sweep lines")
    ap.add_argument("--sweep-only", action="store_true", help="only the MSM / NTT / fold sweep")
    ap.add_argument("--profile-case", default=None, help="run one small single-kernel case (project_b200/profile_cases.py) and exit")
    args = ap.parse_args()
    if args.small:
        args.workload = "small"
    if args.profile_case is not None:
        from project_b200 import profile_cases

        emit({"profile_case": args.profile_case, "launches_and_us_per_launch": profile_cases.run_case(args.profile_case)})
        return 0
    from project_b200 import synthetic

    if args.impl == "reference":
        return run_reference(args)
    inputs = synthetic.make_inputs(**WORKLOADS[args.workload])
    compact = args.workload in COMPACT

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
    from project_b200 import Backend, load_library
    from project_b200.flow import gpu_flow

    lib = load_library()
    G = generator_bytes()
    small = args.workload == "small"
    if args.sweep_only:
        from project_b200 import sweep as sw

        be = Backend(local_rank)
        result = sw.run_sweep(be, local_rank, small=small) if world == 1 else sw.run_sweep_sharded(be, G, rank, world, local_rank, small=small)
        if world > 1:
            dist.destroy_process_group()
        if rank == 0:
            emit({"sweep": result, "n_gpus": world})
        return 0

    flow = gpu_flow(local_rank, inputs, G, compact_columns=compact)
    ctx = flow.context()
    lib.gzk_ctx_stream.restype = ctypes.c_void_p
    stream = torch.cuda.ExternalStream(lib.gzk_ctx_stream(ctx), device=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, stream=stream):
        for _ in range(warmup):
            fn()
        barrier()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(steps):
                fn()
            stop.record(stream)
            barrier()
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks.summary()

    def contexts():
        return [ctx] + flow.side_contexts()  # the side contexts (streams) appear with the first proof

    def timing_report():
        out = {}
        for c in contexts():
            for i in range(lib.gzk_timing_family_count(c)):
                name, launches, ms = ctypes.c_char_p(), ctypes.c_uint64(), ctypes.c_double()
                lib.gzk_timing_get(c, i, ctypes.byref(name), ctypes.byref(launches), ctypes.byref(ms))
                seen = out.get(name.value.decode(), (0, 0.0))
                out[name.value.decode()] = (seen[0] + int(launches.value), seen[1] + float(ms.value))
        return out

    flow.prove(inputs_resident=True)  # untimed: buffers, work areas and side contexts come into being
    for c in contexts():
        lib.gzk_timing_reset(c)
    ms_total, clocks = timed(lambda: flow.prove(inputs_resident=True), args.steps, args.warmup)
    ms_per_step = ms_total / args.steps / world  # `world` independent proofs run side by side
    launches_per_step = sum(v[0] for v in timing_report().values()) // (args.steps + args.warmup)
    stats = flow.stats()
    free_bytes, total_bytes = torch.cuda.mem_get_info()
    resident_gb = (total_bytes - free_bytes) / 1e9  # columns of one proof, tables, weights, pooled buffers

    # per-kernel durations: one more proof with every launch bracketed by CUDA events
    for c in contexts():
        lib.gzk_timing_reset(c)
        lib.gzk_timing_enable(c, 1)
    flow.prove(inputs_resident=True)
    report = timing_report()
    work = (ctypes.c_uint64 * 3)()
    lib.gzk_eval_work_counters(ctx, work)
    for c in contexts():
        lib.gzk_timing_enable(c, 0)
    kernel_ms = {k: round(v[1], 3) for k, v in sorted(report.items(), key=lambda kv: -kv[1][1]) if v[0]}

    # ---- roofline of the dominant kernel family (packed evaluation) --------------------------------
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            peak = float(json.load(f)["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    from project_b200.lib import measure_mac_peak

    eval_ms = sum(v[1] for k, v in report.items() if k.startswith("eval_partial"))
    eval_launches = sum(v[0] for k, v in report.items() if k.startswith("eval_partial"))
    achieved = work[0] / (eval_ms * 1e-3) / 1e9 if eval_ms > 0 else 0.0
    mac_peak = measure_mac_peak(local_rank, 2, 20000)  # 8x8-limb products per second
    limb_rate = work[1] / (eval_ms * 1e-3) if eval_ms > 0 else 0.0
    field_terms = max(0, (work[1] - 8 * work[2]) // 56)  # terms of field-element columns (64 limb products each; 8 for the others)
    roofline = {
        "bound": "hbm",
        "kernel": "eval_partial_kernel / eval_integers_kernel (packed evaluation: commit tau-evaluations, quotient and opening evaluations; "
                  "all launches of one proof, each timed by itself)",
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if peak else None,
        "traffic": (537.0e6 + 4.5e6) / 536.9e6 * work[0] / max(1, eval_launches),
        "traffic_note": "average launch of this run: its algorithmic bytes times the ratio ncu measured on a 2^22-row, 3-column launch "
                        "(dram read+write 541.5e6 against 536.9e6 algorithmic; traffic grows in proportion to columns x rows); "
                        "profiles/eval_partial_kernel_2p22_rows.md",
        "peak_source": peak_src, "launches": eval_launches, "avg_launch_ms": eval_ms / max(1, eval_launches), "bytes_per_step": int(work[0]),
        "tensor": {"u8_products_per_s": field_terms * 1024 / (eval_ms * 1e-3) if eval_ms > 0 else 0.0,
                   "note": "field-element columns: the 32 x 32 byte products of a row, summed over the rows, are one matrix product "
                           "(mma.sync m16n8k32 u8 -> s32); the tensor pipe is 28-33 % busy in the ncu capture, memory and the byte "
                           "transposition bound the kernel"},
        "integer_pipe": {"limb_products_per_s_if_on_the_integer_pipe": limb_rate, "measured_peak_limb_products_per_s": mac_peak * 64,
                         "ratio": limb_rate / (mac_peak * 64) if mac_peak else None,
                         "note": "what the same sums would need of the integer pipe (64 32x32-bit products per term of a field-element column, 8 for a "
                                 "small-integer column) against its measured peak: that pipe bounded this kernel at 0.48 before the field-element "
                                 "columns moved to the tensor cores; it still bounds the weight, scan and matrix kernels"},
    }

    # ---- end to end: the feature matrix and the parameters travel from the host every step ---------
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, min(args.steps, 3))
        e2e_ms, _ = timed(lambda: flow.prove(inputs_resident=False), e2e_steps, 1)
        s = flow.stats()
        e2e = {"value": e2e_ms / e2e_steps / world, "unit": "ms", "h2d_bytes_per_step": s["h2d_bytes"], "d2h_bytes_per_step": s["d2h_bytes"]}

    # ---- honest-prover commitments: every column also committed as an MSM against the resident SRS ----
    commit_msm = None
    if not args.no_msm and not compact:
        flow.set_msm_commit(True)
        flow.prove(inputs_resident=True)  # builds the SRS tables (set-up, not timed)
        before = flow.set_msm_commit(True)
        msm_ms, _ = timed(lambda: flow.prove(inputs_resident=True), 1, 0)
        after = flow.set_msm_commit(False)
        commit_msm = {"ms_per_proof_added": msm_ms / world - ms_per_step, "msm_commitments": after[0] - before[0], "mismatches_vs_trapdoor": after[1],
                      "note": "one Pippenger MSM per committed column against the resident table of shifted SRS bases (Lagrange basis of the "
                              "column's domain, monomial basis for the matrices), each compared with the trapdoor point [p(tau)] G; "
                              "small-integer columns are widened to field elements first, MSMs are not batched across columns"}

    # ---- self-check against the CPU restatement (after the timed regions) --------------------------
    import oracle_lib as ora

    check = self_check(flow, ora)
    if world > 1:
        verdict = torch.tensor([1 if check == "ok" else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
        if int(verdict.item()) == 0 and check == "ok":
            check = "another rank failed"

    flow.close()
    del flow
    # ---- the mid-size configuration beside the headline one ------------------------------------------
    b2 = None
    if args.workload == "b4" and not args.no_b2:
        flow2 = gpu_flow(local_rank, synthetic.make_inputs(**WORKLOADS["b2"]), G)
        stream2 = torch.cuda.ExternalStream(lib.gzk_ctx_stream(flow2.context()), device=torch.device("cuda", local_rank))
        ms2, _ = timed(lambda: flow2.prove(inputs_resident=True), args.steps, args.warmup, stream2)
        e2e2, _ = timed(lambda: flow2.prove(inputs_resident=False), 2, 1, stream2)
        stats2 = flow2.stats()
        b2 = {"workload": WORKLOAD_NAMES["b2"], "ms_per_proof": ms2 / args.steps / world, "e2e_ms_per_proof": e2e2 / 2 / world,
              "dynamic_commitments": stats2["dynamic_commitments"], "commit_barriers": stats2["commit_barriers"], "self_check": self_check(flow2, ora)}
        if not args.no_msm:
            flow2.set_msm_commit(True)
            flow2.prove(inputs_resident=True)  # builds the SRS tables (set-up, not timed)
            before = flow2.set_msm_commit(True)
            msm_ms, _ = timed(lambda: flow2.prove(inputs_resident=True), 1, 0, stream2)
            after = flow2.set_msm_commit(False)
            b2["commit_msm"] = {"ms_per_proof_added": msm_ms / world - b2["ms_per_proof"], "msm_commitments": after[0] - before[0],
                                "mismatches_vs_trapdoor": after[1],
                                "note": "every committed column also committed as a Pippenger MSM against the resident SRS table and compared "
                                        "with the trapdoor point [p(tau)] G"}
        flow2.close()
        del flow2
    sweep = None
    if not args.no_sweep:
        from project_b200 import sweep as sw

        be = Backend(local_rank)
        sweep = sw.run_sweep(be, local_rank, small=small) if world == 1 else sw.run_sweep_sharded(be, G, rank, world, local_rank, small=small)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = cpu_count()
        cpu_inputs, factor = cpu_sample_inputs(args.workload)
        v, _, cstats = cpu_flow_run(cpu_inputs, 1, 0, threads, compact=compact)
        cpu_baseline = {"value": v * factor, "unit": "ms", "cores": threads, "kind": "port", "sample": "one proof: " + cpu_sample_text(args.workload, cstats, threads, factor)}

    if rank == 0:
        emit({
            "metric": METRIC, "value": ms_per_step, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32x8 Montgomery Fr / u32x12 Fp (BLS12-381)", "data": "synthetic", "config": config_of(args, world),
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "self_check": check, "proof": {k: stats[k] for k in ("commit_barriers", "challenges", "dynamic_commitments", "opened_columns", "domains")},
            "kernel_ms": kernel_ms, "kernel_ms_note": "one proof, every launch bracketed by CUDA events (sums per kernel family)",
            "clocks": clocks, "resident_gb": resident_gb, "commit_msm": commit_msm, "b2": b2, "sweep": sweep,
        })
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

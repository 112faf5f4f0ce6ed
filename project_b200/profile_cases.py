"""Small single-kernel cases for profiler captures: each case runs one kernel family of the proof flow a few
times on inputs larger than L2 but a few hundred MB at most, so that a capture of one to three launches ends by
itself in a minute or two.  `python bench.py --profile-case NAME` runs one of them and prints the per-launch
times the library's own event timers saw (never a number to quote from a run under a profiler)."""
import numpy as np

from . import KIND_F64, KIND_FR, KIND_FR_MONT, KIND_I64, KIND_U32, Backend

CASES = ("eval", "eval_int", "logup_indexed", "bary", "matrix", "combine", "multiplicity", "project", "ntt", "msm", "scan_batch")


def _challenge(seed):
    x = np.zeros(32, dtype=np.uint8)
    x[:8] = np.frombuffer((0x9E3779B97F4A7C15 ^ seed).to_bytes(8, "little"), dtype=np.uint8)
    return x


def run_case(name, device=0, repeats=2):
    be = Backend(device)
    be.set_deferred(True)
    rng = np.random.default_rng(7)
    x = _challenge(1)
    one = np.frombuffer((1).to_bytes(32, "little"), dtype=np.uint8)

    def ints(n, lo=-1000, hi=1000):
        return be.upload(rng.integers(lo, hi, size=n, dtype=np.int64), KIND_I64)

    def field_column(n):
        a, b = ints(n), ints(n)
        return be.linear_combination([a, b], np.concatenate([one, x]), n, n)

    if name in ("eval", "eval_int"):
        # 2^22 rows: 3 field-element columns (384 MiB) or 8 small-integer columns (256 MiB), one and two points
        log2n, n = 22, 1 << 22
        w = be.bary_weights(log2n, x)
        cols = [field_column(n) for _ in range(3)] if name == "eval" else [ints(n) for _ in range(8)]
        out = be.alloc(KIND_FR, 2 * len(cols))
        run = lambda: (be.eval_batch_range_device(cols, n, 0, log2n, w, 0, (0,), out), be.eval_batch_range_device(cols, n, 0, log2n, w, 0, (0, 1), out))
    elif name == "logup_indexed":
        # a 24 579-row banded table (the ELU table's shape) hit by 2^22 queries, most of them near the centre
        band, xs, n = 3, 8193, 1 << 22
        valid = n - 7
        table_x = np.repeat(np.arange(-4096, 4097, dtype=np.int64), band)
        table_y = table_x * 5 + np.tile(np.arange(band, dtype=np.int64), xs) - 1
        pick = np.clip(rng.normal(xs * band / 2, 600, size=valid).astype(np.int64), 0, xs * band - 1)
        pad = lambda v: np.concatenate([v, np.zeros(n - v.size, dtype=np.int64)])
        bx, by = be.upload(pad(table_x[pick]), KIND_I64), be.upload(pad(table_y[pick]), KIND_I64)
        btx, bty = be.upload(pad(table_x), KIND_I64), be.upload(pad(table_y), KIND_I64)
        mult = be.banded_lookup_multiplicity(bx, by, valid, -4096, band, bty, xs * band, n)
        table = be.linear_combination([btx, bty], np.concatenate([one, x]), xs * band, n)
        out = be.alloc(KIND_FR_MONT, n)
        beta = np.zeros(32, dtype=np.uint8)
        beta[:16] = rng.integers(0, 256, size=16, dtype=np.uint8)
        run = lambda: be.logup_accumulator_indexed(table, mult, bx, by, valid, -4096, band, bty, xs * band, n, beta, out=out)
    elif name == "bary":
        out = be.alloc(KIND_FR_MONT, 1 << 22)
        run = lambda: be.bary_weights(22, x, out=out)
    elif name == "matrix":
        # 65 536 x 256 small-integer matrix (128 MiB): row fold, row linear form, Horner as one polynomial
        rows, cols = 65536, 256
        m = ints(rows * cols)
        w = be.bary_weights(16, x)
        powers = be.powers(x, cols)
        folded = be.alloc(KIND_FR, cols)
        run = lambda: (be.fold_rows(m, rows, cols, w, rows, out=folded), be.linear_form_rows(m, rows, cols, powers).free(), be.matrix_horner(m, rows, cols, x))
    elif name == "combine":
        n = 1 << 23
        a, b = ints(n), ints(n)
        out = be.alloc(KIND_FR_MONT, n)
        run = lambda: be.linear_combination([a, b], np.concatenate([one, x]), n, n, out=out)
    elif name == "multiplicity":
        band, xs, n = 3, 8193, 1 << 24
        table_x = np.repeat(np.arange(-4096, 4097, dtype=np.int64), band)
        table_y = table_x * 5 + np.tile(np.arange(band, dtype=np.int64), xs) - 1
        pick = np.clip(rng.normal(xs * band / 2, 600, size=n).astype(np.int64), 0, xs * band - 1)
        bx, by = be.upload(table_x[pick], KIND_I64), be.upload(table_y[pick], KIND_I64)
        bty = be.upload(table_y, KIND_I64)
        out = be.alloc(KIND_U32, n)
        run = lambda: be.banded_lookup_multiplicity(bx, by, n, -4096, band, bty, xs * band, n, out=out)
    elif name == "project":
        # one attention head of 65 536 nodes, 128 -> 256, 8 incoming edges per node plus a hub of 20 000
        nodes, inner, width = 65536, 128, 256
        src = np.concatenate([rng.integers(0, nodes, size=nodes * 8), rng.integers(0, nodes, size=20000), np.arange(nodes)]).astype(np.uint32)
        dst = np.concatenate([rng.integers(0, nodes, size=nodes * 8), np.zeros(20000, dtype=np.int64), np.arange(nodes)]).astype(np.uint32)
        order = np.argsort(dst, kind="stable")
        src, dst = src[order], dst[order]
        in_ptr = np.zeros(nodes + 1, dtype=np.uint32)
        np.cumsum(np.bincount(dst, minlength=nodes), out=in_ptr[1:])
        f64 = lambda a: be.upload(np.ascontiguousarray(a, dtype=np.float64), KIND_F64)
        u32 = lambda a: be.upload(np.ascontiguousarray(a, dtype=np.uint32), KIND_U32)
        args = (f64(rng.standard_normal(nodes * inner)), f64(rng.uniform(-0.1, 0.1, size=inner * width)), f64(rng.uniform(-0.5, 0.5, size=width)), 0.01,
                f64(rng.uniform(-0.5, 0.5, size=width)), -0.02, None, True, u32(src), u32(dst), nodes, inner, width, u32(in_ptr), u32(src))
        trace = be.gat_head_forward(*args)
        run = lambda: be.gat_head_forward(*args, out=trace)
    elif name == "ntt":
        v = field_column(1 << 22)
        run = lambda: be.ntt(v, 22)
    elif name == "scan_batch":
        # the independent running sums between two Fiat-Shamir points of one head of the mid-size configuration: four
        # LogUp accumulators, three route accumulators and two segmented states over 2^18 rows, one batched call
        from .lib import SCAN_GROUP_PREFIX, SCAN_LOGUP, SCAN_ROUTE_EDGE, SCAN_ROUTE_NODE

        n, valid = 1 << 18, (1 << 18) - 37
        sel = np.zeros(n, dtype=np.uint32)
        sel[:valid] = 1
        starts = (rng.random(n) < 0.1).astype(np.uint32)
        starts[0] = 1
        bsel, bstarts = be.upload(sel, KIND_U32), be.upload(starts, KIND_U32)
        mult = be.upload(rng.integers(0, 4, size=n, dtype=np.uint32), KIND_U32)
        fields = [field_column(n) for _ in range(8)]
        outs = [be.alloc(KIND_FR_MONT, n) for _ in range(9)]
        beta = np.zeros(32, dtype=np.uint8)  # unrelated to the multiplier inside the field columns
        beta[:16] = rng.integers(0, 256, size=16, dtype=np.uint8)
        jobs = [(SCAN_LOGUP, [fields[0], fields[1], mult, bsel, bsel], valid, n, beta, outs[0]),
                (SCAN_LOGUP, [fields[2], fields[3], mult, bsel, bsel], valid, n, beta, outs[1]),
                (SCAN_LOGUP, [fields[4], fields[5], mult, bsel, bsel], valid, n, beta, outs[2]),
                (SCAN_LOGUP, [fields[6], fields[7], mult, bsel, bsel], valid, n, beta, outs[3]),
                (SCAN_ROUTE_NODE, [fields[0], mult], valid, n, beta, outs[4]),
                (SCAN_ROUTE_EDGE, [fields[1]], valid, n, beta, outs[5]),
                (SCAN_ROUTE_EDGE, [fields[3]], valid, n, beta, outs[6]),
                (SCAN_GROUP_PREFIX, [fields[5], bstarts], n, n, None, outs[7]),
                (SCAN_GROUP_PREFIX, [mult, bstarts], n, n, None, outs[8])]
        run = lambda: be.running_sums_batch(jobs)
    elif name == "msm":
        # 2^20 points (the Lagrange SRS of a 2^20 domain) against uniform-looking scalars: plain Pippenger
        import os
        import sys

        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tests"))
        import pyref

        G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()
        srs = be.srs_lagrange(20, G, x)
        scalars = field_column(1 << 20)
        run = lambda: be.msm(scalars, srs, 1 << 20)
    else:
        raise SystemExit(f"unknown profile case {name}; one of {CASES}")
    run()
    be.synchronize()
    be.timing_reset()
    be.timing_enable(True)
    for _ in range(repeats):
        run()
    be.synchronize()
    report = {k: (v[0], round(v[1] / max(1, v[0]) * 1e3, 1)) for k, v in be.timing_report().items() if v[0]}
    be.timing_enable(False)
    be.close()
    return report

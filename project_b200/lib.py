"""ctypes binding of libgatzk_b200.so (include/gatzk_b200.h).

There is no fallback: if the shared library is absent or no sm_100 GPU is
usable, construction raises.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgatzk_b200.so")

KIND_FR, KIND_FR_MONT, KIND_I64, KIND_U32, KIND_F64, KIND_G1 = 0, 1, 2, 3, 4, 5
_KIND_DTYPE = {KIND_FR: (np.uint8, 32), KIND_FR_MONT: (np.uint8, 32), KIND_I64: (np.int64, 1), KIND_U32: (np.uint32, 1), KIND_F64: (np.float64, 1), KIND_G1: (np.uint8, 96)}

_lib = None


class GzkError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"gatzk_b200 error {code}: {message}")
        self.code = code


def load_library():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m project_b200.build` (needs nvcc); there is no CPU fallback"
            )
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.gzk_last_error.restype = ctypes.c_char_p
        _lib.gzk_last_error.argtypes = [ctypes.c_void_p]
        _lib.gzk_msm_table_points.restype = ctypes.c_size_t
        _lib.gzk_msm_window_bits.restype = ctypes.c_uint
        _lib.gzk_buf_count.restype = ctypes.c_size_t
        _lib.gzk_buf_count.argtypes = [ctypes.c_void_p]
        _lib.gzk_buf_kind.argtypes = [ctypes.c_void_p]
        _lib.gzk_buf_device_ptr.restype = ctypes.c_void_p
        _lib.gzk_buf_device_ptr.argtypes = [ctypes.c_void_p]
        _lib.gzk_ctx_stream.restype = ctypes.c_void_p
        _lib.gzk_ctx_stream.argtypes = [ctypes.c_void_p]
        _lib.gzk_ctx_destroy.restype = None
        _lib.gzk_ctx_destroy.argtypes = [ctypes.c_void_p]
        _lib.gzk_timing_family_count.argtypes = [ctypes.c_void_p]
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _sz(v):
    return ctypes.c_size_t(int(v))


def _fr(x):
    a = np.ascontiguousarray(x, dtype=np.uint8).reshape(-1)
    assert a.size == 32, "expected one 32-byte field element"
    return a


class _ScanJob(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int), ("c0", ctypes.c_void_p), ("c1", ctypes.c_void_p), ("c2", ctypes.c_void_p), ("c3", ctypes.c_void_p),
                ("c4", ctypes.c_void_p), ("count", ctypes.c_size_t), ("domain_size", ctypes.c_size_t), ("beta", ctypes.c_void_p), ("out", ctypes.c_void_p)]


SCAN_LOGUP, SCAN_ROUTE_NODE, SCAN_ROUTE_EDGE, SCAN_ZKMAP, SCAN_GROUP_PREFIX = 0, 1, 2, 3, 4


class _GatHead(ctypes.Structure):
    _fields_ = [("features", ctypes.c_void_p), ("input_width", ctypes.c_uint32), ("output_width", ctypes.c_uint32),
                ("seq_kernel", ctypes.c_void_p), ("attn_src_kernel", ctypes.c_void_p), ("attn_dst_kernel", ctypes.c_void_p),
                ("attn_src_bias", ctypes.c_double), ("attn_dst_bias", ctypes.c_double), ("output_bias", ctypes.c_void_p),
                ("output_bias_count", ctypes.c_size_t), ("apply_activation", ctypes.c_int)]


class _GatGraph(ctypes.Structure):
    _fields_ = [("node_count", ctypes.c_size_t), ("edge_count", ctypes.c_size_t), ("edge_src", ctypes.c_void_p), ("edge_dst", ctypes.c_void_p),
                ("incoming_count", ctypes.c_size_t), ("incoming_ptr", ctypes.c_void_p), ("incoming_src", ctypes.c_void_p)]


class _GatTrace(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in ("H_prime", "E_src", "E_dst", "M", "Sum", "inv", "S", "Z", "Delta", "U", "alpha",
                                                     "H_agg_pre_bias", "H_agg")]


def incoming_lists(edge_src, edge_dst, node_count):
    """The per-destination source lists the reference builds on the host (src/model/gat.cpp:521-538): sources in edge order,
    the node itself appended when it has no self loop.  Returns (ptr[node_count + 1], src[...]) as uint32 arrays."""
    lists = [[] for _ in range(node_count)]
    for s, d in zip(np.asarray(edge_src).tolist(), np.asarray(edge_dst).tolist()):
        lists[d].append(s)
    for d in range(node_count):
        if d not in lists[d]:
            lists[d].append(d)
    ptr = np.zeros(node_count + 1, dtype=np.uint32)
    ptr[1:] = np.cumsum([len(x) for x in lists])
    src = np.array([s for x in lists for s in x], dtype=np.uint32)
    return ptr, src


class Buffer:
    def __init__(self, backend, handle, kind, count):
        self.backend, self.handle, self.kind, self.count = backend, handle, kind, count

    def upload(self, host, offset=0):
        dtype, width = _KIND_DTYPE[self.kind]
        a = np.ascontiguousarray(host, dtype=dtype)
        count = a.size // width
        self.backend._check(self.backend.lib.gzk_buf_upload(self.backend.ctx, self.handle, _sz(offset), _ptr(a), _sz(count)))
        return self

    def upload_async(self, host, offset=0):
        """Queue the copy on the copy stream; `host` must stay alive until Backend.copy_fence + synchronize."""
        dtype, width = _KIND_DTYPE[self.kind]
        a = np.ascontiguousarray(host, dtype=dtype)
        self.backend._check(self.backend.lib.gzk_buf_upload_async(self.backend.ctx, self.handle, _sz(offset), _ptr(a), _sz(a.size // width)))
        return self

    def download(self, offset=0, count=None):
        dtype, width = _KIND_DTYPE[self.kind]
        count = self.count - offset if count is None else count
        out = np.zeros((count, width) if width > 1 else (count,), dtype=dtype)
        self.backend._check(self.backend.lib.gzk_buf_download(self.backend.ctx, self.handle, _sz(offset), _ptr(out), _sz(count)))
        return out

    def retag(self, kind):
        """Declare the 32-byte form (KIND_FR / KIND_FR_MONT) a refilled work buffer now holds."""
        if self.backend.lib.gzk_buf_retag(self.handle, int(kind)) != 0:
            raise ValueError("retag: only between the two field-element kinds")
        self.kind = kind
        return self

    @property
    def device_ptr(self):
        return self.backend.lib.gzk_buf_device_ptr(self.handle)

    def free(self):
        if self.handle is not None:
            self.backend._check(self.backend.lib.gzk_buf_free(self.backend.ctx, self.handle))
            self.handle = None


class Backend:
    """One context on one GPU; thin, argument-for-argument view of the C ABI."""

    def __init__(self, device=0):
        self.lib = load_library()
        ctx = ctypes.c_void_p()
        rc = self.lib.gzk_ctx_create(int(device), ctypes.byref(ctx))
        if rc != 0:
            raise GzkError(rc, "gzk_ctx_create failed: no usable sm_100 CUDA device (there is no CPU fallback)")
        self.ctx = ctx

    def close(self):
        if self.ctx:
            self.lib.gzk_ctx_destroy(self.ctx)
            self.ctx = None

    def _check(self, rc):
        if rc != 0:
            raise GzkError(rc, self.lib.gzk_last_error(self.ctx).decode())

    def set_deferred(self, on=True):
        self._check(self.lib.gzk_ctx_set_deferred(self.ctx, int(bool(on))))

    def copy_fence(self):
        self._check(self.lib.gzk_copy_fence(self.ctx))

    def synchronize(self):
        self._check(self.lib.gzk_ctx_synchronize(self.ctx))

    def wait_for(self, other):
        """Everything queued on this context from now on runs after what `other` (same GPU) has queued so far."""
        self._check(self.lib.gzk_ctx_wait_for(self.ctx, other.ctx))

    def timing_enable(self, on=True):
        self._check(self.lib.gzk_timing_enable(self.ctx, int(bool(on))))

    def timing_reset(self):
        self._check(self.lib.gzk_timing_reset(self.ctx))

    def timing_report(self):
        """{family: (launches, total_ms)} since the last reset."""
        out = {}
        for i in range(self.lib.gzk_timing_family_count(self.ctx)):
            name = ctypes.c_char_p()
            launches = ctypes.c_uint64()
            ms = ctypes.c_double()
            self._check(self.lib.gzk_timing_get(self.ctx, i, ctypes.byref(name), ctypes.byref(launches), ctypes.byref(ms)))
            out[name.value.decode()] = (int(launches.value), float(ms.value))
        return out


    @property
    def stream(self):
        return self.lib.gzk_ctx_stream(self.ctx)

    def alloc(self, kind, count):
        h = ctypes.c_void_p()
        self._check(self.lib.gzk_buf_alloc(self.ctx, int(kind), _sz(count), ctypes.byref(h)))
        return Buffer(self, h, kind, count)

    def upload(self, host, kind=KIND_FR):
        dtype, width = _KIND_DTYPE[kind]
        a = np.ascontiguousarray(host, dtype=dtype)
        return self.alloc(kind, a.size // width).upload(a)

    def root_of_unity(self, size):
        out = np.zeros(32, dtype=np.uint8)
        self._check(self.lib.gzk_root_of_unity(self.ctx, ctypes.c_uint64(size), _ptr(out)))
        return out

    def bary_weights(self, log2n, x, out=None):
        out = out or self.alloc(KIND_FR_MONT, 1 << log2n)
        self._check(self.lib.gzk_bary_weights(self.ctx, ctypes.c_uint(log2n), _ptr(_fr(x)), out.handle))
        return out

    def bary_weights_prefix(self, log2n, x, keep, out=None):
        """Whole-domain weights of which only the first `keep` and the last two are written."""
        out = out or self.alloc(KIND_FR_MONT, 1 << log2n)
        self._check(self.lib.gzk_bary_weights_prefix(self.ctx, ctypes.c_uint(log2n), _ptr(_fr(x)), ctypes.c_uint64(keep), out.handle))
        return out

    def bary_weights_multi(self, log2n, xs, outs=None):
        """Weights of one domain at several points (one launch for up to four points of a small domain)."""
        outs = outs or [self.alloc(KIND_FR_MONT, 1 << log2n) for _ in xs]
        points = np.ascontiguousarray(np.stack([_fr(x) for x in xs]))
        handles = (ctypes.c_void_p * len(outs))(*[o.handle for o in outs])
        self._check(self.lib.gzk_bary_weights_multi(self.ctx, ctypes.c_uint(log2n), _ptr(points), _sz(len(outs)), handles))
        return outs

    def logup_accumulator(self, table, query, mult, q_table, q_query, n, beta, active_count, out=None):
        out = out or self.alloc(KIND_FR_MONT, n)
        self._check(self.lib.gzk_logup_accumulator(self.ctx, table.handle, query.handle, mult.handle, q_table.handle, q_query.handle,
                                                   _sz(n), _ptr(_fr(beta)), _sz(active_count), out.handle))
        return out

    def logup_accumulator_indexed(self, table, mult, x, y, active_count, x_min, band, table_y, table_size, n, beta, out=None):
        """LogUp accumulator of a lookup into a banded static table with the inverses fetched per table row."""
        out = out or self.alloc(KIND_FR_MONT, n)
        self._check(self.lib.gzk_logup_accumulator_indexed(self.ctx, table.handle, mult.handle, x.handle, y.handle if y is not None else None,
                                                           _sz(active_count), ctypes.c_int64(x_min), _sz(band),
                                                           table_y.handle if table_y is not None else None, _sz(table_size), _sz(n), _ptr(_fr(beta)),
                                                           out.handle))
        return out

    def linear_combination(self, cols, coefficients, count, domain_size, out=None):
        """out[i] = sum_j coefficients[j] * cols[j][i] for i < count, zero tail (Montgomery buffer)."""
        handles = (ctypes.c_void_p * len(cols))(*[c.handle for c in cols])
        coeff = np.ascontiguousarray(coefficients, dtype=np.uint8).reshape(len(cols), 32)
        out = out or self.alloc(KIND_FR_MONT, domain_size)
        self._check(self.lib.gzk_linear_combination(self.ctx, handles, _ptr(coeff), _sz(len(cols)), _sz(count), _sz(domain_size), out.handle))
        return out

    def banded_lookup_multiplicity(self, x, y, count, x_min, band, table_y, table_size, domain_size, out=None):
        out = out or self.alloc(KIND_U32, domain_size)
        self._check(self.lib.gzk_banded_lookup_multiplicity(self.ctx, x.handle, y.handle if y is not None else None, _sz(count), ctypes.c_int64(x_min),
                                                            _sz(band), table_y.handle if table_y is not None else None, _sz(table_size),
                                                            _sz(domain_size), out.handle))
        return out

    def route_node_accumulator(self, table, mult, valid_length, domain_size, beta, out=None):
        out = out or self.alloc(KIND_FR_MONT, domain_size)
        self._check(self.lib.gzk_route_node_accumulator(self.ctx, table.handle, mult.handle, _sz(valid_length), _sz(domain_size),
                                                        _ptr(_fr(beta)), out.handle))
        return out

    def route_edge_accumulator(self, query, valid_length, domain_size, beta, out=None):
        out = out or self.alloc(KIND_FR_MONT, domain_size)
        self._check(self.lib.gzk_route_edge_accumulator(self.ctx, query.handle, _sz(valid_length), _sz(domain_size), _ptr(_fr(beta)), out.handle))
        return out

    def route_edge_accumulator_indexed(self, table, node_count, index, valid_length, domain_size, beta, out=None):
        """Edge side of a route whose query of edge e is table[index[e]]: the node-table inverses are fetched per edge."""
        out = out or self.alloc(KIND_FR_MONT, domain_size)
        self._check(self.lib.gzk_route_edge_accumulator_indexed(self.ctx, table.handle, _sz(node_count), index.handle, _sz(valid_length),
                                                                _sz(domain_size), _ptr(_fr(beta)), out.handle))
        return out

    def running_sums_batch(self, jobs):
        """jobs: list of (op, [input Buffers], count, domain_size, beta or None, out Buffer): gzk_running_sums_batch."""
        raw = (_ScanJob * len(jobs))()
        keep = []
        for r, (op, cols, count, domain_size, beta, out) in zip(raw, jobs):
            r.op = op
            handles = [c.handle for c in cols] + [None] * (5 - len(cols))
            r.c0, r.c1, r.c2, r.c3, r.c4 = handles
            r.count, r.domain_size = int(count), int(domain_size)
            if beta is not None:
                b = _fr(beta).copy()
                keep.append(b)
                r.beta = b.ctypes.data
            r.out = out.handle
        self._check(self.lib.gzk_running_sums_batch(self.ctx, raw, _sz(len(jobs))))

    def group_prefix_state(self, values, q_new, n, out=None):
        out = out or self.alloc(KIND_FR_MONT, n)
        self._check(self.lib.gzk_group_prefix_state(self.ctx, values.handle, q_new.handle, _sz(n), out.handle))
        return out

    def zkmap_accumulator(self, a, b, count, domain_size, out=None):
        out = out or self.alloc(KIND_FR_MONT, domain_size)
        mu = np.zeros(32, dtype=np.uint8)
        self._check(self.lib.gzk_zkmap_accumulator(self.ctx, a.handle, b.handle, _sz(count), _sz(domain_size), out.handle, _ptr(mu)))
        return out, mu

    def matrix_horner(self, matrix, rows, cols, x):
        out = np.zeros(32, dtype=np.uint8)
        self._check(self.lib.gzk_matrix_horner(self.ctx, matrix.handle, _sz(rows), _sz(cols), _ptr(_fr(x)), _ptr(out)))
        return out

    def fold_rows(self, matrix, rows, cols, weights, row_count, out=None):
        out = out or self.alloc(KIND_FR, cols)
        self._check(self.lib.gzk_fold_rows(self.ctx, matrix.handle, _sz(rows), _sz(cols), weights.handle, _sz(row_count), out.handle))
        return out

    def linear_form_rows(self, matrix, rows, cols, powers):
        out = self.alloc(KIND_FR_MONT, rows)
        self._check(self.lib.gzk_linear_form_rows(self.ctx, matrix.handle, _sz(rows), _sz(cols), powers.handle, out.handle))
        return out

    def powers(self, challenge, count):
        out = self.alloc(KIND_FR_MONT, count)
        self._check(self.lib.gzk_powers(self.ctx, _ptr(_fr(challenge)), _sz(count), out.handle))
        return out

    def weighted_sum(self, left, lam, right, count, domain_size, out=None):
        out = out or self.alloc(KIND_FR_MONT, domain_size)
        self._check(self.lib.gzk_weighted_sum(self.ctx, left.handle, _ptr(_fr(lam)), right.handle, _sz(count), _sz(domain_size), out.handle))
        return out

    def feature_lookup_rows(self, row_ids, feature_indices, features, rows, width, eta_index, eta_value):
        out = self.alloc(KIND_FR_MONT, rows * width)
        self._check(self.lib.gzk_feature_lookup_rows(self.ctx, row_ids.handle, feature_indices.handle, features.handle, _sz(rows), _sz(width),
                                                     _ptr(_fr(eta_index)), _ptr(_fr(eta_value)), out.handle))
        return out

    def broadcast_node_values(self, node_values, node_count, index, edge_count, domain_size, out=None):
        out = out or self.alloc(node_values.kind, domain_size)
        self._check(self.lib.gzk_broadcast_node_values(self.ctx, node_values.handle, _sz(node_count), index.handle, _sz(edge_count), _sz(domain_size), out.handle))
        return out

    def histogram(self, indices, count, domain_size, out=None):
        out = out or self.alloc(KIND_U32, domain_size)
        self._check(self.lib.gzk_histogram(self.ctx, indices.handle, _sz(count), _sz(domain_size), out.handle))
        return out

    def quantize(self, values, count):
        out = self.alloc(KIND_I64, count)
        self._check(self.lib.gzk_quantize(self.ctx, values.handle, _sz(count), out.handle))
        return out

    def quantize_guarded(self, values, count, guard):
        """(I64 buffer, number of values within `guard` of a rounding boundary)."""
        out = self.alloc(KIND_I64, count)
        counter = self.upload(np.zeros(1, dtype=np.uint32), KIND_U32)
        self._check(self.lib.gzk_quantize_guarded(self.ctx, values.handle, _sz(count), ctypes.c_double(guard), out.handle, counter.handle))
        return out, int(counter.download()[0])

    def gat_head_forward(self, features, seq_kernel, attn_src, bias_src, attn_dst, bias_dst, out_bias, apply_activation, edge_src, edge_dst,
                         node_count, input_width, output_width, incoming_ptr, incoming_src, out=None):
        """All arguments are Buffers (F64 matrices, U32 lists) except the scalars; returns the trace fields as a dict of F64 Buffers
        (`out`: such a dict from an earlier call, to be refilled)."""
        edges = edge_src.count if edge_src is not None else 0
        if out is None:
            out = {name: self.alloc(KIND_F64, node_count * output_width) for name in ("H_prime", "H_agg_pre_bias", "H_agg")}
            out.update({name: self.alloc(KIND_F64, node_count) for name in ("E_src", "E_dst", "M", "Sum", "inv")})
            out.update({name: self.alloc(KIND_F64, max(edges, 1)) for name in ("S", "Z", "Delta", "U", "alpha")})
        head = _GatHead(features.handle, input_width, output_width, seq_kernel.handle, attn_src.handle, attn_dst.handle, bias_src, bias_dst,
                        out_bias.handle if out_bias is not None else None, out_bias.count if out_bias is not None else 0, int(bool(apply_activation)))
        graph = _GatGraph(node_count, edges, edge_src.handle if edges else None, edge_dst.handle if edges else None, incoming_src.count,
                          incoming_ptr.handle, incoming_src.handle)
        trace = _GatTrace(*[out[name].handle for name in ("H_prime", "E_src", "E_dst", "M", "Sum", "inv", "S", "Z", "Delta", "U", "alpha",
                                                          "H_agg_pre_bias", "H_agg")])
        self._check(self.lib.gzk_gat_head_forward(self.ctx, ctypes.byref(head), ctypes.byref(graph), ctypes.byref(trace)))
        return out

    def first_zero_marker(self, delta, group_begin, group_end, groups, domain_size):
        out = self.alloc(KIND_U32, domain_size)
        self._check(self.lib.gzk_first_zero_marker(self.ctx, delta.handle, group_begin.handle, group_end.handle, _sz(groups), _sz(domain_size), out.handle))
        return out

    def g1_mul_same_base(self, base, scalars):
        base = np.ascontiguousarray(base, dtype=np.uint8).reshape(-1)
        sc = np.ascontiguousarray(scalars, dtype=np.uint8).reshape(-1, 32)
        out = np.zeros((sc.shape[0], 96), dtype=np.uint8)
        self._check(self.lib.gzk_g1_mul_same_base(self.ctx, _ptr(base), _ptr(sc), _sz(sc.shape[0]), _ptr(out)))
        return out

    def g1_fixed_base_mul(self, base, scalars, count):
        base = np.ascontiguousarray(base, dtype=np.uint8).reshape(-1)
        out = self.alloc(KIND_G1, count)
        self._check(self.lib.gzk_g1_fixed_base_mul(self.ctx, _ptr(base), scalars.handle, _sz(count), out.handle))
        return out

    def commit_batch(self, cols, length, log2n, weights_tau, base):
        base = np.ascontiguousarray(base, dtype=np.uint8).reshape(-1)
        handles = (ctypes.c_void_p * len(cols))(*[c.handle for c in cols])
        evals = np.zeros((len(cols), 32), dtype=np.uint8)
        points = np.zeros((len(cols), 96), dtype=np.uint8)
        self._check(self.lib.gzk_commit_batch(self.ctx, handles, _sz(len(cols)), _sz(length), ctypes.c_uint(log2n), weights_tau.handle,
                                              _ptr(base), _ptr(evals), _ptr(points)))
        return evals, points

    def msm(self, scalars, points, n):
        out = np.zeros(96, dtype=np.uint8)
        self._check(self.lib.gzk_msm(self.ctx, scalars.handle, points.handle, _sz(n), _ptr(out)))
        return out

    def msm_window_bits(self, n):
        return int(self.lib.gzk_msm_window_bits(_sz(n)))

    def msm_precompute(self, points, n, window_bits=None):
        """(table Buffer, window_bits): the shifted copies of a resident point set for msm_precomputed."""
        window_bits = window_bits or self.msm_window_bits(n)
        table = self.alloc(KIND_G1, int(self.lib.gzk_msm_table_points(_sz(n), ctypes.c_uint(window_bits))))
        self._check(self.lib.gzk_msm_precompute(self.ctx, points.handle, _sz(n), ctypes.c_uint(window_bits), table.handle))
        return table, window_bits

    def msm_precomputed(self, scalars, table, n, window_bits):
        out = np.zeros(96, dtype=np.uint8)
        self._check(self.lib.gzk_msm_precomputed(self.ctx, scalars.handle, table.handle, _sz(n), ctypes.c_uint(window_bits), _ptr(out)))
        return out

    def srs_lagrange(self, log2n, base, tau):
        base = np.ascontiguousarray(base, dtype=np.uint8).reshape(-1)
        out = self.alloc(KIND_G1, 1 << log2n)
        self._check(self.lib.gzk_srs_lagrange(self.ctx, ctypes.c_uint(log2n), _ptr(base), _ptr(_fr(tau)), out.handle))
        return out

    def ntt(self, inp, log2n, batch=1, inverse=False, coset_shift=None, out=None):
        out = out or self.alloc(KIND_FR_MONT, (1 << log2n) * batch)
        shift = None if coset_shift is None else _ptr(_fr(coset_shift))
        self._check(self.lib.gzk_ntt(self.ctx, inp.handle, out.handle, ctypes.c_uint(log2n), _sz(batch), int(bool(inverse)), shift))
        return out

    def wrap(self, kind, count, device_ptr):
        """A Buffer over device memory owned by the caller (e.g. a torch tensor)."""
        h = ctypes.c_void_p()
        self._check(self.lib.gzk_buf_wrap(self.ctx, int(kind), _sz(count), ctypes.c_void_p(device_ptr), ctypes.byref(h)))
        return Buffer(self, h, kind, count)

    def swap_outer(self, inp, d0, d1, d2, out=None):
        out = out or self.alloc(inp.kind, d0 * d1 * d2)
        self._check(self.lib.gzk_swap_outer(self.ctx, inp.handle, _sz(d0), _sz(d1), _sz(d2), out.handle))
        return out

    def transpose(self, inp, rows, cols, out=None):
        out = out or self.alloc(inp.kind, rows * cols)
        self._check(self.lib.gzk_transpose(self.ctx, inp.handle, _sz(rows), _sz(cols), out.handle))
        return out

    def ntt_twiddle(self, buf, log2n, row_first, rows, cols, inverse=False):
        self._check(self.lib.gzk_ntt_twiddle(self.ctx, buf.handle, ctypes.c_uint(log2n), ctypes.c_uint64(row_first), _sz(rows), _sz(cols),
                                             int(bool(inverse))))
        return buf

    def coset_lde(self, inp, log2n, log2_blowup, shift, out=None):
        out = out or self.alloc(KIND_FR_MONT, 1 << (log2n + log2_blowup))
        self._check(self.lib.gzk_coset_lde(self.ctx, inp.handle, ctypes.c_uint(log2n), ctypes.c_uint(log2_blowup), _ptr(_fr(shift)), out.handle))
        return out

    def fold(self, table, n, challenge, out=None):
        out = out or self.alloc(KIND_FR_MONT, n // 2)
        self._check(self.lib.gzk_fold(self.ctx, table.handle, _sz(n), _ptr(_fr(challenge)), out.handle))
        return out

    def fh_public_eval(self, features, rows, feature_count, abs_ids, weights):
        out = np.zeros((5, 32), dtype=np.uint8)
        self._check(self.lib.gzk_fh_public_eval(self.ctx, features.handle if features is not None else None, _sz(rows), _sz(feature_count),
                                                abs_ids.handle if abs_ids is not None else None, weights.handle, _ptr(out)))
        return out

    def bary_weights_range(self, log2n, x, first, count, out=None):
        out = out or self.alloc(KIND_FR_MONT, max(count, 1))
        self._check(self.lib.gzk_bary_weights_range(self.ctx, ctypes.c_uint(log2n), _ptr(_fr(x)), ctypes.c_uint64(first), ctypes.c_uint64(count), out.handle))
        return out

    def eval_batch_range(self, cols, length, row_offset, log2n, weights, weights_first, rotations=(0,)):
        handles = (ctypes.c_void_p * len(cols))(*[c.handle for c in cols])
        rot = np.ascontiguousarray(rotations, dtype=np.uint64)
        out = np.zeros((rot.size, len(cols), 32), dtype=np.uint8)
        self._check(self.lib.gzk_eval_batch_range(self.ctx, handles, _sz(len(cols)), _sz(length), ctypes.c_uint64(row_offset), ctypes.c_uint(log2n),
                                                  weights.handle, ctypes.c_uint64(weights_first), _ptr(rot), _sz(rot.size), _ptr(out)))
        return out

    def generated_column(self, what, valid, width, domain_size, kind=KIND_U32):
        out = self.alloc(kind, domain_size)
        self._check(self.lib.gzk_generated_column(self.ctx, int(what), _sz(valid), _sz(width), _sz(domain_size), out.handle))
        return out

    def fr_add_scalar(self, buf, offset, count, scalar):
        self._check(self.lib.gzk_fr_add_scalar(self.ctx, buf.handle, _sz(offset), _sz(count), _ptr(_fr(scalar))))

    def sumcheck_round_sums(self, table, n):
        out = np.zeros((3, 32), dtype=np.uint8)
        self._check(self.lib.gzk_sumcheck_round_sums(self.ctx, table.handle, _sz(n), _ptr(out)))
        return out

    def eval_batch_range_device(self, cols, length, row_offset, log2n, weights, weights_first, rotations, out, out_offset=0):
        handles = (ctypes.c_void_p * len(cols))(*[c.handle for c in cols])
        rot = np.ascontiguousarray(rotations, dtype=np.uint64)
        self._check(self.lib.gzk_eval_batch_range_device(self.ctx, handles, _sz(len(cols)), _sz(length), ctypes.c_uint64(row_offset), ctypes.c_uint(log2n),
                                                         weights.handle, ctypes.c_uint64(weights_first), _ptr(rot), _sz(rot.size), out.handle,
                                                         _sz(out_offset)))
        return out

    def eval_batch(self, cols, length, log2n, weights, rotations=(0,)):
        handles = (ctypes.c_void_p * len(cols))(*[c.handle for c in cols])
        rot = np.ascontiguousarray(rotations, dtype=np.uint64)
        out = np.zeros((rot.size, len(cols), 32), dtype=np.uint8)
        self._check(self.lib.gzk_eval_batch(self.ctx, handles, _sz(len(cols)), _sz(length), ctypes.c_uint(log2n), weights.handle, _ptr(rot), _sz(rot.size), _ptr(out)))
        return out


def eval_batch_static(device, stream, col_ptrs, col_kinds, length, log2n, weights_ptr, rotations, out_ptr):
    """gzk_eval_batch_static: the allocation-free variant of packed evaluation.  All
    pointers are raw device addresses (ints); results land in `out_ptr` once the
    caller has synchronised `stream`.  Raises GzkError with the library's message."""
    lib = load_library()
    k = len(col_ptrs)
    ptrs = (ctypes.c_void_p * k)(*col_ptrs)
    kinds = (ctypes.c_int * k)(*col_kinds)
    rot = np.ascontiguousarray(rotations, dtype=np.uint64)
    err = ctypes.create_string_buffer(256)
    rc = lib.gzk_eval_batch_static(int(device), ctypes.c_void_p(stream), ptrs, kinds, _sz(k), _sz(length), ctypes.c_uint(log2n),
                                   ctypes.c_void_p(weights_ptr), _ptr(rot), _sz(rot.size), ctypes.c_void_p(out_ptr), err, _sz(256))
    if rc != 0:
        raise GzkError(rc, err.value.decode())


class Comm:
    """gzk_comm: the NCCL communicator of one rank, bound to a Backend (its stream orders the collectives)."""

    def __init__(self, backend, nranks, rank, unique_id):
        self.be = backend
        uid = np.ascontiguousarray(unique_id, dtype=np.uint8).reshape(-1)
        assert uid.size == 128
        h = ctypes.c_void_p()
        backend._check(backend.lib.gzk_comm_create(backend.ctx, int(nranks), int(rank), _ptr(uid), ctypes.byref(h)))
        self.handle, self.nranks, self.rank = h, nranks, rank

    @staticmethod
    def unique_id():
        out = np.zeros(128, dtype=np.uint8)
        if load_library().gzk_comm_unique_id(_ptr(out)) != 0:
            raise GzkError(2, "gzk_comm_unique_id: NCCL is not available")
        return out

    def set_timeout(self, seconds):
        self.be._check(self.be.lib.gzk_comm_set_timeout(self.handle, ctypes.c_double(seconds)))

    def wait(self):
        self.be._check(self.be.lib.gzk_comm_wait(self.handle))

    def allgather(self, inp, count, out):
        self.be._check(self.be.lib.gzk_comm_allgather(self.handle, inp.handle, _sz(count), out.handle))
        return out

    def allgather_fr_sum(self, inp, count, out):
        self.be._check(self.be.lib.gzk_comm_allgather_fr_sum(self.handle, inp.handle, _sz(count), out.handle))
        return out

    def alltoall(self, inp, count_per_rank, out):
        self.be._check(self.be.lib.gzk_comm_alltoall(self.handle, inp.handle, _sz(count_per_rank), out.handle))
        return out

    def ntt_sharded(self, rows, log2n, work, out):
        self.be._check(self.be.lib.gzk_ntt_sharded(self.handle, rows.handle, ctypes.c_uint(log2n), work.handle, out.handle))
        return out

    def close(self):
        if self.handle:
            fn = self.be.lib.gzk_comm_destroy
            fn.restype = None
            fn.argtypes = [ctypes.c_void_p]
            fn(self.handle)
            self.handle = None


def inject_eval_stall(on):
    """gzk_debug_inject_eval_stall: makes the bounded waits of the packed-evaluation kernel run out (tests only)."""
    load_library().gzk_debug_inject_eval_stall(int(bool(on)))


TUNING_LIB_PATH = os.path.join(HERE, "libgatzk_b200_tuning.so")


def measure_mac_peak(device=0, chains=1, iters=20000):
    """Integer-pipe ceiling (8x8-limb multiply-accumulates per second) from the separate tuning library."""
    if not os.path.exists(TUNING_LIB_PATH):
        raise RuntimeError(f"{TUNING_LIB_PATH} is missing: build it with `python -m project_b200.build`")
    lib = ctypes.CDLL(TUNING_LIB_PATH)
    out = ctypes.c_double()
    rc = lib.gzk_tuning_mac_peak(int(device), int(chains), ctypes.c_uint32(iters), ctypes.byref(out))
    if rc != 0:
        raise GzkError(2, f"gzk_tuning_mac_peak: CUDA error {rc}")
    return out.value


def fr_sum(values):
    """Host combine of per-GPU partial results: values [groups, ..., 32] -> [..., 32]."""
    lib = load_library()
    v = np.ascontiguousarray(values, dtype=np.uint8)
    groups = v.shape[0]
    count = v[0].size // 32
    out = np.zeros(v.shape[1:], dtype=np.uint8)
    rc = lib.gzk_fr_sum(_ptr(v), _sz(groups), _sz(count), _ptr(out))
    if rc != 0:
        raise GzkError(rc, "gzk_fr_sum: non-canonical input")
    return out


def g1_sum(points):
    lib = load_library()
    v = np.ascontiguousarray(points, dtype=np.uint8).reshape(-1, 96)
    out = np.zeros(96, dtype=np.uint8)
    rc = lib.gzk_g1_sum(_ptr(v), _sz(v.shape[0]), _ptr(out))
    if rc != 0:
        raise GzkError(rc, "gzk_g1_sum: non-canonical input")
    return out


def shard_rows(n_rows, world, rank, align=1):
    """Contiguous row range [begin, end) of `rank` when n_rows rows are split over `world` GPUs."""
    per = -(-n_rows // world)
    per = -(-per // align) * align
    begin = min(n_rows, rank * per)
    return begin, min(n_rows, begin + per)

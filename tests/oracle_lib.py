"""ctypes loader for the CPU oracle (test infrastructure only)."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_DIR = os.path.join(os.path.dirname(_HERE), "oracle")
_LIB = None


def build():
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.ora_last_error.restype = ctypes.c_char_p
        _LIB.ora_active_transition_count.restype = ctypes.c_uint64
        _LIB.ora_fnv1a.restype = ctypes.c_uint64
    return _LIB


def _p(a):
    if a is None:
        return None
    return a.ctypes.data_as(ctypes.c_void_p)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _check(rc):
    if rc != 0:
        raise RuntimeError(lib().ora_last_error().decode())


def _sz(v):
    return ctypes.c_size_t(int(v))


def fr_binop(op, a, b):
    a, b = _u8(a), _u8(b)
    out = np.zeros_like(a)
    _check(lib().ora_fr_binop(op, _p(a), _p(b), _sz(a.size // 32), _p(out)))
    return out


def fp_binop(op, a, b):
    a, b = _u8(a), _u8(b)
    out = np.zeros_like(a)
    _check(lib().ora_fp_binop(op, _p(a), _p(b), _sz(a.size // 48), _p(out)))
    return out


def fr_inv(a):
    a = _u8(a)
    out = np.zeros_like(a)
    _check(lib().ora_fr_inv(_p(a), _sz(a.size // 32), _p(out)))
    return out


def fr_from_i64(v):
    v = np.ascontiguousarray(v, dtype=np.int64)
    out = np.zeros((v.size, 32), dtype=np.uint8)
    _check(lib().ora_fr_from_i64(_p(v), _sz(v.size), _p(out)))
    return out


def fr_to_decimal(a):
    buf = ctypes.create_string_buffer(100)
    a = _u8(a)
    _check(lib().ora_fr_to_decimal(_p(a), buf, _sz(100)))
    return buf.value.decode()


def root_of_unity(n):
    out = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_root_of_unity(ctypes.c_uint64(n), _p(out)))
    return out


def batch_invert(a):
    a = _u8(a)
    out = np.zeros_like(a)
    _check(lib().ora_batch_invert(_p(a), _sz(a.size // 32), _p(out)))
    return out


def bary_weights(x, n):
    x = _u8(x)
    out = np.zeros((n, 32), dtype=np.uint8)
    _check(lib().ora_bary_weights(_p(x), ctypes.c_uint64(n), _p(out)))
    return out


def eval_rotations(columns, weights, rotations, threads=1):
    """columns: [K][n][32] uint8 -> out [P][K][32]."""
    columns, weights = _u8(columns), _u8(weights)
    k, n = columns.shape[0], columns.shape[1]
    rot = np.ascontiguousarray(rotations, dtype=np.uint64)
    out = np.zeros((rot.size, k, 32), dtype=np.uint8)
    _check(lib().ora_eval_rotations(_p(columns), _sz(k), _sz(n), _p(weights), _p(rot), _sz(rot.size), _sz(threads), _p(out)))
    return out


def commit_tau_eval(columns, weights, threads=1):
    columns, weights = _u8(columns), _u8(weights)
    k, valid = columns.shape[0], columns.shape[1]
    out = np.zeros((k, 32), dtype=np.uint8)
    _check(lib().ora_commit_tau_eval(_p(columns), _sz(k), _sz(valid), _p(weights), _sz(threads), _p(out)))
    return out


def commit_tau_eval_i64(columns, weights):
    columns = np.ascontiguousarray(columns, dtype=np.int64)
    weights = _u8(weights)
    k, valid = columns.shape
    out = np.zeros((k, 32), dtype=np.uint8)
    _check(lib().ora_commit_tau_eval_i64(_p(columns), _sz(k), _sz(valid), _p(weights), _p(out)))
    return out


def horner(coeffs, x):
    coeffs, x = _u8(coeffs), _u8(x)
    out = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_horner(_p(coeffs), _sz(coeffs.size // 32), _p(x), _p(out)))
    return out


def poly_evaluate_barycentric(values, size, x):
    values, x = _u8(values), _u8(x)
    out = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_poly_evaluate_barycentric(_p(values), _sz(values.size // 32), ctypes.c_uint64(size), _p(x), _p(out)))
    return out


def matrix_row_major_eval(matrix, x):
    matrix, x = _u8(matrix), _u8(x)
    rows, cols = matrix.shape[0], matrix.shape[1]
    out = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_matrix_row_major_eval(_p(matrix), _sz(rows), _sz(cols), _p(x), _p(out)))
    return out


def weighted_column_sum(matrix, row_weights, row_count):
    matrix, row_weights = _u8(matrix), _u8(row_weights)
    rows, cols = matrix.shape[0], matrix.shape[1]
    out = np.zeros((cols, 32), dtype=np.uint8)
    _check(lib().ora_weighted_column_sum(_p(matrix), _sz(rows), _sz(cols), _p(row_weights), _sz(row_count), _p(out)))
    return out


def linear_form_by_powers(matrix, powers):
    matrix, powers = _u8(matrix), _u8(powers)
    rows, cols = matrix.shape[0], matrix.shape[1]
    out = np.zeros((rows, 32), dtype=np.uint8)
    _check(lib().ora_linear_form_by_powers(_p(matrix), _sz(rows), _sz(cols), _p(powers), _p(out)))
    return out


def powers(challenge, count):
    challenge = _u8(challenge)
    out = np.zeros((count, 32), dtype=np.uint8)
    _check(lib().ora_powers(_p(challenge), _sz(count), _p(out)))
    return out


def zkmap_accumulator(a, b, domain_size):
    a, b = _u8(a), _u8(b)
    count = a.size // 32
    acc = np.zeros((domain_size, 32), dtype=np.uint8)
    mu = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_zkmap_accumulator(_p(a), _p(b), _sz(count), _sz(domain_size), _p(acc), _p(mu)))
    return acc, mu


def logup_accumulator(table, query, mult, q_table, q_query, beta, active_count):
    arrs = [_u8(x) for x in (table, query, mult, q_table, q_query)]
    n = arrs[0].size // 32
    beta = _u8(beta)
    out = np.zeros((n, 32), dtype=np.uint8)
    _check(lib().ora_logup_accumulator(*[_p(x) for x in arrs], _sz(n), _p(beta), _sz(active_count), _p(out)))
    return out


def active_transition_count(q_table, q_query):
    q_table, q_query = _u8(q_table), _u8(q_query)
    return int(lib().ora_active_transition_count(_p(q_table), _p(q_query), _sz(q_table.size // 32)))


def route_node_accumulator(table, mult, valid_length, beta):
    table, mult, beta = _u8(table), _u8(mult), _u8(beta)
    n = table.size // 32
    out = np.zeros((n, 32), dtype=np.uint8)
    _check(lib().ora_route_node_accumulator(_p(table), _p(mult), _sz(valid_length), _sz(n), _p(beta), _p(out)))
    return out


def route_edge_accumulator(query, valid_length, beta):
    query, beta = _u8(query), _u8(beta)
    n = query.size // 32
    out = np.zeros((n, 32), dtype=np.uint8)
    _check(lib().ora_route_edge_accumulator(_p(query), _sz(valid_length), _sz(n), _p(beta), _p(out)))
    return out


def group_prefix_state(values, q_new):
    values, q_new = _u8(values), _u8(q_new)
    n = values.size // 32
    out = np.zeros((n, 32), dtype=np.uint8)
    _check(lib().ora_group_prefix_state(_p(values), _p(q_new), _sz(n), _p(out)))
    return out


def first_zero_marker(delta, group_begin, group_end, domain_size):
    delta = _u8(delta)
    gb = np.ascontiguousarray(group_begin, dtype=np.uint64)
    ge = np.ascontiguousarray(group_end, dtype=np.uint64)
    out = np.zeros((domain_size, 32), dtype=np.uint8)
    _check(lib().ora_first_zero_marker(_p(delta), _p(gb), _p(ge), _sz(gb.size), _sz(domain_size), _p(out)))
    return out


def quantize(values):
    values = np.ascontiguousarray(values, dtype=np.float64)
    out = np.zeros(values.shape, dtype=np.int64)
    _check(lib().ora_quantize(_p(values), _sz(values.size), _p(out)))
    return out


def broadcast_node_values(node_values, index, domain_size):
    node_values = _u8(node_values)
    index = np.ascontiguousarray(index, dtype=np.uint64)
    out = np.zeros((domain_size, 32), dtype=np.uint8)
    _check(lib().ora_broadcast_node_values(_p(node_values), _sz(node_values.size // 32), _p(index), _sz(index.size), _sz(domain_size), _p(out)))
    return out


def multiplicity_from_indices(indices, domain_size):
    indices = np.ascontiguousarray(indices, dtype=np.uint64)
    out = np.zeros((domain_size, 32), dtype=np.uint8)
    _check(lib().ora_multiplicity_from_indices(_p(indices), _sz(indices.size), _sz(domain_size), _p(out)))
    return out


def weighted_sum(left, lam, right, domain_size):
    left, lam, right = _u8(left), _u8(lam), _u8(right)
    out = np.zeros((domain_size, 32), dtype=np.uint8)
    _check(lib().ora_weighted_sum(_p(left), _p(lam), _p(right), _sz(left.size // 32), _sz(domain_size), _p(out)))
    return out


def feature_lookup_rows(row_ids, feature_indices, features, eta_index, eta_value):
    row_ids, feature_indices, features = _u8(row_ids), _u8(feature_indices), _u8(features)
    rows, width = features.shape[0], features.shape[1]
    out = np.zeros((rows * width, 32), dtype=np.uint8)
    ei, ev = _u8(eta_index), _u8(eta_value)
    _check(lib().ora_feature_lookup_rows(_p(row_ids), _p(feature_indices), _p(features), _sz(rows), _sz(width), _p(ei), _p(ev), _p(out)))
    return out


def g1_mul_same_base(base, scalars):
    base, scalars = _u8(base), _u8(scalars)
    count = scalars.size // 32
    out = np.zeros((count, 96), dtype=np.uint8)
    _check(lib().ora_g1_mul_same_base(_p(base), _p(scalars), _sz(count), _p(out)))
    return out


def g1_add(a, b):
    a, b = _u8(a), _u8(b)
    out = np.zeros(96, dtype=np.uint8)
    _check(lib().ora_g1_add(_p(a), _p(b), _p(out)))
    return out


def g1_on_curve(a):
    a = _u8(a)
    return lib().ora_g1_on_curve(_p(a)) == 1


def g1_msm_naive(points, scalars):
    points, scalars = _u8(points), _u8(scalars)
    out = np.zeros(96, dtype=np.uint8)
    _check(lib().ora_g1_msm_naive(_p(points), _p(scalars), _sz(scalars.size // 32), _p(out)))
    return out


def ntt(data, inverse=False, coset_shift=None):
    data = _u8(data).copy()
    n = data.size // 32
    cs = _u8(coset_shift) if coset_shift is not None else None
    _check(lib().ora_ntt(_p(data), ctypes.c_uint64(n), int(bool(inverse)), _p(cs)))
    return data


def dft_naive(data):
    data = _u8(data)
    out = np.zeros_like(data)
    _check(lib().ora_dft_naive(_p(data), ctypes.c_uint64(data.size // 32), _p(out)))
    return out


def fold(table, challenge):
    table, challenge = _u8(table), _u8(challenge)
    n = table.size // 32
    out = np.zeros((n // 2, 32), dtype=np.uint8)
    _check(lib().ora_fold(_p(table), _sz(n), _p(challenge), _p(out)))
    return out


def fnv1a(data: bytes):
    return int(lib().ora_fnv1a(data, _sz(len(data))))


def bench_eval(k, n, p_count, threads, seed=1):
    """Seconds the reference's packed-evaluation loop takes on native-form values."""
    sec = ctypes.c_double()
    chk = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_bench_eval(_sz(k), _sz(n), _sz(p_count), _sz(threads), ctypes.c_uint64(seed), ctypes.byref(sec), _p(chk)))
    return sec.value, chk


def bench_bary(n, threads, seed=1):
    sec = ctypes.c_double()
    chk = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_bench_bary(_sz(n), _sz(threads), ctypes.c_uint64(seed), ctypes.byref(sec), _p(chk)))
    return sec.value, chk


def fh_public_eval(features, rows, feature_count, abs_ids, weights):
    features = _u8(features) if features is not None else None
    ids = np.ascontiguousarray(abs_ids, dtype=np.uint64) if abs_ids is not None else None
    weights = _u8(weights)
    out = np.zeros((5, 32), dtype=np.uint8)
    _check(lib().ora_fh_public_eval(_p(features), _sz(rows), _sz(feature_count), _p(ids), _p(weights), _p(out)))
    return out


def bench_builders(n, valid, seed=1):
    """Seconds per column for [logup, route_node, route_edge, group_prefix, zkmap, fold_rows(valid/8 x 8)]."""
    sec = (ctypes.c_double * 6)()
    chk = np.zeros(32, dtype=np.uint8)
    _check(lib().ora_bench_builders(_sz(n), _sz(valid), ctypes.c_uint64(seed), sec, _p(chk)))
    return list(sec)


def gat_head_forward(features, seq_kernel, attn_src, bias_src, attn_dst, bias_dst, out_bias, apply_activation, edge_src, edge_dst):
    """gat.cpp:474-615 on row-major float64 arrays; returns the HeadForwardTrace fields as a dict."""
    features = np.ascontiguousarray(features, dtype=np.float64)
    seq_kernel = np.ascontiguousarray(seq_kernel, dtype=np.float64)
    nodes, inner = features.shape
    width = seq_kernel.shape[1]
    attn_src = np.ascontiguousarray(attn_src, dtype=np.float64)
    attn_dst = np.ascontiguousarray(attn_dst, dtype=np.float64)
    bias = np.ascontiguousarray(out_bias if out_bias is not None else np.zeros(0), dtype=np.float64)
    es = np.ascontiguousarray(edge_src, dtype=np.uint32)
    ed = np.ascontiguousarray(edge_dst, dtype=np.uint32)
    edges = es.size
    out = {name: np.zeros((nodes, width)) for name in ("H_prime", "H_agg_pre_bias", "H_agg")}
    out.update({name: np.zeros(nodes) for name in ("E_src", "E_dst", "M", "Sum", "inv")})
    out.update({name: np.zeros(edges) for name in ("S", "Z", "Delta", "U", "alpha")})
    dp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    _check(lib().ora_gat_head_forward(dp(features), _sz(nodes), _sz(inner), dp(seq_kernel), _sz(width), dp(attn_src), ctypes.c_double(bias_src),
                                      dp(attn_dst), ctypes.c_double(bias_dst), dp(bias), _sz(bias.size), int(out_bias is not None),
                                      int(bool(apply_activation)), dp(es), dp(ed), _sz(edges), dp(out["H_prime"]), dp(out["E_src"]),
                                      dp(out["E_dst"]), dp(out["S"]), dp(out["Z"]), dp(out["M"]), dp(out["Delta"]), dp(out["U"]), dp(out["Sum"]),
                                      dp(out["inv"]), dp(out["alpha"]), dp(out["H_agg_pre_bias"]), dp(out["H_agg"])))
    return out

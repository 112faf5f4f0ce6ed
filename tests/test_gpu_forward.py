"""fp64 forward pass of an attention head on the GPU against the CPU oracle (which follows the
reference's loops and uses the host's exp / expm1).

Bar: every value that involves no transcendental function (H', E_src, E_dst, S, Z, M, Delta) is
bit-identical; values downstream of exp / expm1 (U, Sum, inv, alpha, H_agg_pre_bias, H_agg)
agree to a relative 4e-15 (a few units in the last place: the CUDA and host math libraries may
round the last bit of exp differently), the signed sums H_agg_pre_bias / H_agg to 4e-15 of the
largest summand magnitude (max |H'|), since their terms can cancel; the quantised witness (round half away at scale 16)
is identical wherever 16*v is further than 1e-9 from a rounding boundary."""
import numpy as np
import pytest

import oracle_lib as ora

pytestmark = pytest.mark.gpu

EXACT = ("H_prime", "E_src", "E_dst", "S", "Z", "M", "Delta")
CLOSE = ("U", "Sum", "inv", "alpha", "H_agg_pre_bias", "H_agg")
REL_TOL = 4e-15


@pytest.fixture(scope="module")
def be():
    from project_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


def random_graph(rng, nodes, edges, self_loops):
    src = rng.integers(0, nodes, size=edges, dtype=np.uint32)
    dst = np.sort(rng.integers(0, nodes, size=edges, dtype=np.uint32))  # grouped by destination like the prover's edge list
    if self_loops:
        src = np.concatenate([src, np.arange(nodes, dtype=np.uint32)])
        dst = np.concatenate([dst, np.arange(nodes, dtype=np.uint32)])
        order = np.argsort(dst, kind="stable")
        src, dst = src[order], dst[order]
    return src, dst


def run_case(be, rng, nodes, inner, width, edges, self_loops, bias, activation, shuffle=False, hubs=()):
    from project_b200 import KIND_F64, KIND_U32, incoming_lists

    x = rng.normal(size=(nodes, inner)) * (rng.random((nodes, inner)) < 0.3)
    w = rng.uniform(-0.4, 0.4, size=(inner, width))
    a_src, a_dst = rng.uniform(-1, 1, size=width), rng.uniform(-1, 1, size=width)
    b_src, b_dst = float(rng.uniform(-0.1, 0.1)), float(rng.uniform(-0.1, 0.1))
    out_bias = rng.uniform(-0.2, 0.2, size=width) if bias else None
    src, dst = random_graph(rng, nodes, edges, self_loops)
    for node, degree in hubs:  # nodes with long incoming lists (the hubs of a power-law graph)
        src = np.concatenate([src, rng.integers(0, nodes, size=degree, dtype=np.uint32)])
        dst = np.concatenate([dst, np.full(degree, node, dtype=np.uint32)])
    if hubs:
        order = np.argsort(dst, kind="stable")
        src, dst = src[order], dst[order]
    if shuffle:  # the reference accepts any edge order; the incoming lists then follow that order
        perm = rng.permutation(src.size)
        src, dst = src[perm], dst[perm]
    want = ora.gat_head_forward(x, w, a_src, b_src, a_dst, b_dst, out_bias, activation, src, dst)
    ptr, inc = incoming_lists(src, dst, nodes)
    up = lambda a, kind: be.upload(np.ascontiguousarray(a).reshape(-1), kind)
    got = be.gat_head_forward(up(x, KIND_F64), up(w, KIND_F64), up(a_src, KIND_F64), b_src, up(a_dst, KIND_F64), b_dst,
                              up(out_bias, KIND_F64) if bias else None, activation, up(src, KIND_U32) if src.size else None,
                              up(dst, KIND_U32) if src.size else None, nodes, inner, width, up(ptr, KIND_U32), up(inc, KIND_U32))
    for name in EXACT:
        g = got[name].download()[:want[name].size].reshape(want[name].shape)
        assert np.array_equal(g.view(np.uint64), want[name].view(np.uint64)), name
    for name in CLOSE:
        g = got[name].download()[:want[name].size].reshape(want[name].shape)
        scale = np.maximum(np.abs(want[name]), 1e-300)
        if name.startswith("H_agg"):
            scale = np.maximum(scale, np.abs(want["H_prime"]).max())
        assert np.all(np.abs(g - want[name]) <= REL_TOL * scale + 1e-300), name
    # the quantised witness
    for name in ("H_agg", "alpha", "U"):
        g = got[name]
        count = want[name].size
        if count == 0:
            continue
        # guarded quantisation: when no value is flagged as close to a rounding boundary, EVERY quantised value
        # equals the oracle's (no mask); flagged values are the ones the prover flow re-computes on the host
        q_buf, flagged = be.quantize_guarded(g, count, 2.0 ** -30)
        q = q_buf.download()
        wq = ora.quantize(want[name].reshape(-1))
        if flagged == 0:
            assert np.array_equal(q, wq), name
        else:
            scaled = np.abs(want[name].reshape(-1) * 16.0) + 0.5
            near = np.abs(scaled - np.rint(scaled)) < 2.0 ** -29
            assert np.array_equal(q[~near], wq[~near]), name
            assert flagged <= int(near.sum()) + 1


@pytest.mark.parametrize("nodes,inner,width,edges,self_loops,bias,activation", [
    (1, 3, 2, 0, False, True, True),
    (40, 17, 8, 150, True, True, True),
    (300, 50, 8, 2000, True, False, True),
    (300, 64, 7, 1500, False, True, False),
    (2000, 33, 64, 15000, True, True, True),
    # width a multiple of 64 and inner a multiple of 8: the 128 x 64 projection tiles (ragged last row tile; one slice; many)
    (333, 8, 64, 2500, True, True, True),
    (1100, 72, 128, 9000, True, True, True),
    # an even width that is not a multiple of 64 (the 40 classes of the large model's output layer): ragged column tile
    (700, 48, 40, 5000, True, True, True),
    (260, 16, 98, 1500, True, True, True),
])
def test_head_forward_matches_oracle(be, nodes, inner, width, edges, self_loops, bias, activation):
    run_case(be, np.random.default_rng(nodes * 7 + width), nodes, inner, width, edges, self_loops, bias, activation)


def test_head_forward_with_hub_nodes(be):
    """Incoming lists of 1500 and 700 entries take the kernels for long lists (one warp per node for the softmax
    statistics, a CTA per node with asynchronous gathers for the aggregation); 300 output columns need two column
    passes there and a ragged last tile in the projection."""
    run_case(be, np.random.default_rng(4242), 600, 20, 300, 5000, True, True, True, hubs=((3, 1500), (5, 700), (599, 513)))


def test_head_forward_unsorted_edges(be):
    run_case(be, np.random.default_rng(99), 120, 20, 8, 700, False, True, True, shuffle=True)


def test_head_forward_rejects_bad_endpoint(be):
    from project_b200 import KIND_F64, KIND_U32, GzkError

    nodes, inner, width = 10, 4, 2
    up = lambda a, kind: be.upload(np.ascontiguousarray(a).reshape(-1), kind)
    ptr = np.arange(nodes + 1, dtype=np.uint32)
    inc = np.arange(nodes, dtype=np.uint32)
    inc[3] = 77  # beyond the node count
    with pytest.raises(GzkError) as e:
        be.gat_head_forward(up(np.ones((nodes, inner)), KIND_F64), up(np.ones((inner, width)), KIND_F64), up(np.ones(width), KIND_F64), 0.0,
                            up(np.ones(width), KIND_F64), 0.0, None, True, None, None, nodes, inner, width, up(ptr, KIND_U32), up(inc, KIND_U32))
    assert e.value.code == 1

"""Row-range sharding of the packed evaluation and point-range sharding of the MSM:
the per-shard partial results, combined by the host helpers, must equal the
single-GPU result bit for bit.  The shards run one after the other on one GPU here
(ranks that wait on each other never share a GPU; these do not wait)."""
import numpy as np
import pytest

import oracle_lib as ora
import pyref
from pyref import fr_array

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from project_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sharded_eval_equals_whole(be, world):
    from project_b200 import KIND_FR, fr_sum, shard_rows

    rng = np.random.default_rng(world)
    log2n, n, k, length = 12, 4096, 6, 3900
    cols = rng.integers(0, 256, size=(k, n, 32), dtype=np.uint8)
    cols[:, :, 31] &= 0x3F
    cols[:, length:] = 0
    x = fr_array([int(rng.integers(2, 1 << 62))])
    rots = (0, 1, 7)
    w_full = be.bary_weights(log2n, x)
    whole = be.eval_batch([be.upload(cols[i, :length], KIND_FR) for i in range(k)], length, log2n, w_full, rots)
    partials = []
    for rank in range(world):
        begin, end = shard_rows(length, world, rank, align=32)
        halo = max(rots)
        first = (begin - halo) % n
        w_slice = be.bary_weights_range(log2n, x, first, (end - begin) + halo)
        assert np.array_equal(w_slice.download()[: (end - begin) + halo], np.roll(w_full.download(), -first, axis=0)[: (end - begin) + halo])
        bufs = [be.upload(cols[i, begin:end] if end > begin else np.zeros((1, 32), np.uint8), KIND_FR) for i in range(k)]
        partials.append(be.eval_batch_range(bufs, end - begin, begin % n, log2n, w_slice, first, rots))
    assert np.array_equal(fr_sum(np.stack(partials)), whole)
    assert np.array_equal(whole, ora.eval_rotations(cols, w_full.download(), rots))


def test_sharded_msm_equals_whole(be):
    from project_b200 import KIND_FR, g1_sum, shard_rows

    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()
    rng = np.random.default_rng(9)
    n, world = 5000, 4
    kb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    sb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    kb[:, 31] &= 0x3F
    sb[:, 31] &= 0x3F
    pts = be.g1_fixed_base_mul(G, be.upload(kb, KIND_FR), n)
    whole = be.msm(be.upload(sb, KIND_FR), pts, n)
    host_pts = pts.download()
    from project_b200 import KIND_G1

    parts = []
    for rank in range(world):
        begin, end = shard_rows(n, world, rank)
        parts.append(be.msm(be.upload(sb[begin:end], KIND_FR), be.upload(host_pts[begin:end], KIND_G1), end - begin))
    assert np.array_equal(g1_sum(np.stack(parts)), whole)


def test_sharded_running_sum_with_carry(be):
    """A route accumulator whose rows are split over 3 'ranks': each computes its local
    running sum, the totals are exchanged, and the carry is added on the device."""
    from project_b200 import KIND_FR, fr_sum, shard_rows

    rng = np.random.default_rng(21)
    n, valid, world = 8192, 7000, 3
    query = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    query[:, 31] &= 0x3F
    beta = fr_array([424242424242])
    whole = be.route_edge_accumulator(be.upload(query, KIND_FR), valid, n, beta).download()
    pieces, totals = [], []
    for rank in range(world):
        begin, end = shard_rows(valid, world, rank, align=32)
        rows = end - begin
        local = be.route_edge_accumulator(be.upload(query[begin:end], KIND_FR), rows, rows + 1, beta)  # out[0..rows]
        pieces.append((begin, rows, local))
        totals.append(local.download(offset=rows, count=1)[0])
    got = np.zeros((n, 32), dtype=np.uint8)
    for rank, (begin, rows, local) in enumerate(pieces):
        if rank > 0:
            carry = fr_sum(np.stack(totals[:rank])) if rank > 1 else totals[0]
            be.fr_add_scalar(local, 0, rows + 1, carry)
        got[begin + 1:begin + rows + 1] = local.download(offset=1, count=rows)
    got[valid + 1:] = got[valid]
    assert np.array_equal(got, whole)


def test_generated_columns(be):
    from project_b200 import KIND_I64, KIND_U32

    n, valid, width = 5000, 4321, 37
    sel = be.generated_column(0, valid, 0, n).download()
    assert sel[:valid].all() and not sel[valid:].any()
    idx = np.arange(n)
    assert np.array_equal(be.generated_column(1, valid, 0, n, KIND_I64).download(), np.where(idx < valid, idx, 0))
    assert np.array_equal(be.generated_column(2, valid, width, n).download(), np.where(idx < valid, idx // width, 0))
    assert np.array_equal(be.generated_column(3, valid, width, n).download(), np.where(idx < valid, idx % width, 0))


def test_sharded_segmented_state_with_carry(be):
    """A segmented running sum (restarts where q_new = 1) whose rows are cut at arbitrary
    places over 4 'ranks': the carry of a rank is the state at the end of the rank before it
    and reaches only the rows ahead of the rank's first restart."""
    from project_b200 import KIND_FR, KIND_U32, fr_sum

    rng = np.random.default_rng(31)
    n = 9000
    values = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    values[:, 31] &= 0x3F
    q_new = (rng.random(n) < 0.002).astype(np.uint32)  # long segments, some ranks see no restart
    q_new[0] = 1
    q_new[2500:5200] = 0                               # rank 2 of the cut below sees none
    whole = be.group_prefix_state(be.upload(values, KIND_FR), be.upload(q_new, KIND_U32), n).download()
    cuts = [0, 1111, 2600, 5100, n]
    carry = None
    got = np.zeros_like(whole)
    for rank in range(4):
        begin, end = cuts[rank], cuts[rank + 1]
        rows = end - begin
        local = be.group_prefix_state(be.upload(values[begin:end], KIND_FR), be.upload(q_new[begin:end], KIND_U32), rows)
        restarts = np.flatnonzero(q_new[begin:end])
        reach = int(restarts[0]) if restarts.size else rows  # rows that continue the segment of the rank before
        if carry is not None and reach > 0:
            be.fr_add_scalar(local, 0, reach, carry)
        out = local.download()
        got[begin:end] = out
        carry = out[-1]  # the state at the end of this rank (already carries what came before)
    assert np.array_equal(got, whole)

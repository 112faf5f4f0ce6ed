"""Full-size runs (the domain sizes of the large configurations) checked through identities that
do not need a CPU pass over the data: partition of unity of the weights, the LogUp identity
(the accumulator of a permuted lookup ends at zero), transform round trips, and the scalar
identity of an MSM over multiples of the generator."""
import numpy as np
import pytest

import oracle_lib as ora
import pyref
from pyref import R, fr_array

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from project_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


def test_weights_sum_to_one_at_2p26(be):
    """sum_i w_i(x) = 1 at every rotation, through the quartet weights kernel and the packed evaluation of a
    generated all-ones column over 2^26 rows."""
    log2n = 26
    n = 1 << log2n
    x = fr_array([0x1234567890ABCDEF])
    w = be.bary_weights(log2n, x)
    ones = be.generated_column(0, n, 1, n)  # selector: 1 for every row
    index = be.generated_column(1, n, 1, n)  # the row index
    got = be.eval_batch([ones, index], n, log2n, w, (0, 1, 5))
    one = fr_array([1])[0]
    for p in range(3):
        assert np.array_equal(got[p, 0], one)
    # the row-index column rotated by r differs from the unrotated one by r on all but the last r rows:
    # sum_i w_i * ((i + r) mod n) = sum_i w_i * i + r - n * (sum of the last r weights)
    tail = w.download(offset=n - 5, count=5)
    value = lambda b: int.from_bytes(b.tobytes(), "little")
    base = value(got[0, 1])
    assert value(got[1, 1]) == (base + 1 - n * value(tail[4])) % R
    assert value(got[2, 1]) == (base + 5 - n * sum(value(t) for t in tail)) % R
    for b in (w, ones, index):
        b.free()


def test_logup_of_a_permuted_lookup_ends_at_zero_at_2p24(be):
    """Query = a permutation of the table, multiplicity 1: the running sum of 1/(T+b) - 1/(Q+b) returns to zero
    after the last active row (2^24 rows: the several-launch path with a global batch inversion)."""
    from project_b200 import KIND_I64, KIND_U32

    rng = np.random.default_rng(2024)
    n = 1 << 24
    active = n - 1
    table = rng.integers(-(1 << 40), 1 << 40, size=n, dtype=np.int64)
    query = table.copy()
    query[:active] = table[:active][rng.permutation(active)]
    mult = np.ones(n, dtype=np.uint32)
    sel = np.ones(n, dtype=np.uint32)
    beta = fr_array([0x0123456789ABCDEF0123])
    out = be.logup_accumulator(be.upload(table, KIND_I64), be.upload(query, KIND_I64), be.upload(mult, KIND_U32), be.upload(sel, KIND_U32),
                               be.upload(sel, KIND_U32), n, beta, active)
    head = out.download(count=3)
    last = out.download(offset=n - 1, count=1)
    assert not head[0].any()
    assert not last[0].any()
    # rows 1 and 2 against the oracle's field arithmetic
    tb = ora.fr_binop(0, ora.fr_from_i64(table[:2]), np.repeat(beta, 2, axis=0))
    qb = ora.fr_binop(0, ora.fr_from_i64(query[:2]), np.repeat(beta, 2, axis=0))
    terms = ora.fr_binop(1, ora.fr_inv(tb), ora.fr_inv(qb))
    assert np.array_equal(head[1], terms[0])
    assert np.array_equal(head[2], ora.fr_binop(0, terms[:1], terms[1:2])[0])
    out.free()


def test_ntt_round_trip_at_2p24(be):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(24)
    log2n = 24
    n = 1 << log2n
    a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    a[:, 31] &= 0x3F
    src = be.upload(a, KIND_FR)
    fwd = be.ntt(src, log2n)
    back = be.ntt(fwd, log2n, inverse=True)
    assert np.array_equal(back.download(), a)
    # X[0] = sum of the inputs, X[n/2] = alternating sum (omega^(n/2) = -1), by 64-bit limb sums on the host
    limbs = a.view(np.uint64).reshape(n, 4)
    total = sum(int(limbs[:, k].astype(object).sum()) << (64 * k) for k in range(4)) % R
    even = sum(int(limbs[0::2, k].astype(object).sum()) << (64 * k) for k in range(4))
    odd = sum(int(limbs[1::2, k].astype(object).sum()) << (64 * k) for k in range(4))
    value = lambda b: int.from_bytes(b.tobytes(), "little")
    assert value(fwd.download(count=1)[0]) == total
    assert value(fwd.download(offset=n // 2, count=1)[0]) == (even - odd) % R
    for b in (src, fwd, back):
        b.free()


def test_msm_resident_table_scalar_identity_at_2p20(be):
    """MSM(s, [k_i]G) = [sum s_i k_i]G over 2^20 points with the window the library chooses."""
    from project_b200 import KIND_FR

    rng = np.random.default_rng(20)
    n = 1 << 20
    kb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    sb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    kb[:, 31] &= 0x3F
    sb[:, 31] &= 0x3F
    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()
    pts = be.g1_fixed_base_mul(G, be.upload(kb, KIND_FR), n)
    table, wb = be.msm_precompute(pts, n)
    scalars = be.upload(sb, KIND_FR)
    got = be.msm_precomputed(scalars, table, n, wb)
    ks = [int.from_bytes(row.tobytes(), "little") for row in kb]
    ss = [int.from_bytes(row.tobytes(), "little") for row in sb]
    want = pyref.g1_bytes(pyref.g1_mul(sum(k * s for k, s in zip(ks, ss)) % R, (pyref.GX, pyref.GY)))
    assert bytes(got) == want
    assert bytes(be.msm(scalars, pts, n)) == want
    for b in (pts, table, scalars):
        b.free()

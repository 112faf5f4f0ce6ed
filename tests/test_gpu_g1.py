"""GPU parity of the G1 work (same-base batch, commitment, MSM, SRS) against the CPU
oracle and Python big-integer arithmetic, through the C ABI, byte-exact on affine
coordinates."""
import random

import numpy as np
import pytest

import oracle_lib as ora
import pyref
from pyref import R, fr_array, fr_ints

pytestmark = pytest.mark.gpu
G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()


@pytest.fixture(scope="module")
def be():
    from project_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


def test_same_base_batch_matches_oracle(be):
    rng = random.Random(1)
    scalars = [0, 1, 2, 255, 256, R - 1, 28, (1 << 254) + 12345] + pyref.rand_fr(rng, 40)
    got = be.g1_mul_same_base(G, fr_array(scalars))
    want = ora.g1_mul_same_base(G, fr_array(scalars))
    assert np.array_equal(got, want)
    assert not got[0].any()  # [0]G is the point at infinity
    # another base: 7G
    base7 = ora.g1_mul_same_base(G, fr_array([7]))[0]
    got = be.g1_mul_same_base(base7, fr_array(scalars[:10]))
    assert np.array_equal(got, ora.g1_mul_same_base(base7, fr_array(scalars[:10])))


def test_same_base_rejects_bad_base(be):
    from project_b200 import GzkError

    bad = G.copy()
    bad[0] ^= 1
    with pytest.raises(GzkError, match="not on the curve"):
        be.g1_mul_same_base(bad, fr_array([5]))
    with pytest.raises(GzkError):
        be.g1_mul_same_base(np.zeros(96, dtype=np.uint8), fr_array([5]))


def test_point_buffer_round_trip_and_fixed_base(be):
    from project_b200 import KIND_FR, KIND_G1

    rng = random.Random(2)
    ks = pyref.rand_fr(rng, 33) + [0]
    pts = be.g1_fixed_base_mul(G, be.upload(fr_array(ks), KIND_FR), len(ks))
    host = pts.download()
    assert np.array_equal(host, ora.g1_mul_same_base(G, fr_array(ks)))
    again = be.upload(host, KIND_G1).download()
    assert np.array_equal(again, host)


@pytest.mark.parametrize("n", [1, 2, 37, 300, 3000])
def test_msm_matches_naive_oracle(be, n):
    from project_b200 import KIND_FR, KIND_FR_MONT

    rng = random.Random(100 + n)
    ks = pyref.rand_fr(rng, n)
    scalars = pyref.rand_fr(rng, n)
    if n >= 37:
        scalars[0], scalars[1], scalars[2], scalars[3] = 0, 1, R - 1, (1 << 255) % R
        ks[5] = 0           # a point at infinity among the bases
        ks[7] = ks[6]       # repeated base
        scalars[7] = (R - scalars[6]) % R  # and opposite scalars: the two terms cancel
    pts = be.g1_fixed_base_mul(G, be.upload(fr_array(ks), KIND_FR), n)
    want_scalar = sum(k * s for k, s in zip(ks, scalars)) % R
    want = pyref.g1_bytes(pyref.g1_mul(want_scalar, (pyref.GX, pyref.GY)))
    got = be.msm(be.upload(fr_array(scalars), KIND_FR), pts, n)
    assert bytes(got) == want
    got = be.msm(be.upload(fr_array(scalars), KIND_FR_MONT), pts, n)
    assert bytes(got) == want
    if n <= 300:
        assert np.array_equal(got, ora.g1_msm_naive(pts.download(), fr_array(scalars)))


def test_msm_large_against_scalar_identity(be):
    """2^16 points: MSM(s, [k_i]G) must equal [sum s_i k_i]G (size-independent identity)."""
    from project_b200 import KIND_FR

    n = 1 << 16
    rng = np.random.default_rng(5)
    kb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    sb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    kb[:, 31] &= 0x3F
    sb[:, 31] &= 0x3F
    pts = be.g1_fixed_base_mul(G, be.upload(kb, KIND_FR), n)
    got = be.msm(be.upload(sb, KIND_FR), pts, n)
    ks, ss = fr_ints(kb), fr_ints(sb)
    want_scalar = sum(k * s for k, s in zip(ks, ss)) % R
    assert bytes(got) == pyref.g1_bytes(pyref.g1_mul(want_scalar, (pyref.GX, pyref.GY)))
    assert not be.msm(be.upload(sb, KIND_FR), pts, 0).any()


def test_commit_batch_and_msm_against_lagrange_srs_agree(be):
    """KZG::commit_batch semantics, and the self-check the honest-prover path offers:
    MSM(column, [L_i(tau)]G) == [column(tau)]G."""
    from project_b200 import KIND_FR

    rng = np.random.default_rng(6)
    log2n, n, k, valid = 10, 1024, 5, 900
    tau = fr_array([11 + 17])
    cols = rng.integers(0, 256, size=(k, n, 32), dtype=np.uint8)
    cols[:, :, 31] &= 0x3F
    cols[:, valid:] = 0
    w = be.bary_weights(log2n, tau)
    bufs = [be.upload(cols[i, :valid], KIND_FR) for i in range(k)]
    evals, points = be.commit_batch(bufs, valid, log2n, w, G)
    want_evals = ora.commit_tau_eval(cols[:, :valid].copy(), w.download()[:valid])
    assert np.array_equal(evals, want_evals)
    assert np.array_equal(points, ora.g1_mul_same_base(G, want_evals))
    srs = be.srs_lagrange(log2n, G, tau)
    for i in range(k):
        assert np.array_equal(be.msm(bufs[i], srs, valid), points[i])


def test_msm_skewed_scalars(be):
    """Small-integer and constant scalars put thousands of points into one bucket: the
    cooperative big-bucket path must give the same point."""
    from project_b200 import KIND_FR

    n = 1 << 15
    rng = np.random.default_rng(8)
    kb = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    kb[:, 31] &= 0x3F
    pts = be.g1_fixed_base_mul(G, be.upload(kb, KIND_FR), n)
    ks = fr_ints(kb)
    G0 = (pyref.GX, pyref.GY)
    for name, scalars in (("ones", [1] * n), ("bits", [int(v) for v in rng.integers(0, 2, size=n)]),
                          ("small signed", [int(v) % R for v in rng.integers(-40, 40, size=n)])):
        got = be.msm(be.upload(fr_array(scalars), KIND_FR), pts, n)
        want = sum(k * s for k, s in zip(ks, scalars)) % R
        assert bytes(got) == pyref.g1_bytes(pyref.g1_mul(want, G0)), name


@pytest.mark.parametrize("n,window_bits", [(1, 8), (37, 9), (300, 13), (5000, 16), (1 << 15, None)])
def test_msm_precomputed_table_equals_plain_msm(be, n, window_bits):
    """The shared-bucket MSM over the table of shifted points gives the point of gzk_msm (and of the
    scalar identity) for uniform and for skewed scalars, canonical and Montgomery."""
    from project_b200 import KIND_FR, KIND_FR_MONT

    rng = random.Random(900 + n)
    ks = pyref.rand_fr(rng, n)
    if n >= 37:
        ks[5] = 0           # a point at infinity among the bases
        ks[7] = ks[6]
    pts = be.g1_fixed_base_mul(G, be.upload(fr_array(ks), KIND_FR), n)
    table, wb = be.msm_precompute(pts, n, window_bits)
    assert table.count % n == 0 and table.count // n >= (255 + wb - 1) // wb
    G0 = (pyref.GX, pyref.GY)
    cases = {"uniform": pyref.rand_fr(rng, n), "ones": [1] * n, "minus one": [R - 1] * n,
             "small signed": [rng.randrange(-40, 40) % R for _ in range(n)], "top": [(R - 1 - i) % R for i in range(n)]}
    if n >= 37:
        cases["uniform"][0:4] = [0, 1, R - 1, (1 << 254) % R]
        cases["uniform"][7] = (R - cases["uniform"][6]) % R
    for name, scalars in cases.items():
        want = pyref.g1_bytes(pyref.g1_mul(sum(k * s for k, s in zip(ks, scalars)) % R, G0))
        buf = be.upload(fr_array(scalars), KIND_FR)
        assert bytes(be.msm_precomputed(buf, table, n, wb)) == want, name
        assert bytes(be.msm(buf, pts, n)) == want, name
    mont = be.upload(fr_array(cases["uniform"]), KIND_FR_MONT)
    assert bytes(be.msm_precomputed(mont, table, n, wb)) == bytes(be.msm(mont, pts, n))
    assert not be.msm_precomputed(mont, table, 0, wb).any()


def test_msm_precomputed_rejects_short_table(be):
    from project_b200 import KIND_FR, KIND_G1, GzkError

    n = 64
    pts = be.g1_fixed_base_mul(G, be.upload(fr_array(list(range(1, n + 1))), KIND_FR), n)
    with pytest.raises(GzkError):
        be.msm_precomputed(be.upload(fr_array([1] * n), KIND_FR), pts, n, 16)  # a plain point buffer is not a table

"""GPU parity of the stand-alone NTT / coset LDE / fold kernels against the CPU oracle
(textbook radix-2 transform over the reference's domain), bit-exact."""
import numpy as np
import pytest

import oracle_lib as ora
from pyref import fr_array

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from project_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


def rand_fr(rng, n):
    a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    a[:, 31] &= 0x3F
    return a


@pytest.mark.parametrize("log2n", [0, 1, 2, 5, 9, 10, 11, 12, 13, 14, 16, 18, 19, 21])
def test_ntt_matches_oracle(be, log2n):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(log2n)
    n = 1 << log2n
    a = rand_fr(rng, n)
    buf = be.upload(a, KIND_FR)
    fwd = be.ntt(buf, log2n)
    assert np.array_equal(fwd.download(), ora.ntt(a))
    assert np.array_equal(be.ntt(fwd, log2n, inverse=True).download(), a)
    shift = fr_array([5])
    cos = be.ntt(buf, log2n, coset_shift=shift)
    assert np.array_equal(cos.download(), ora.ntt(a, coset_shift=shift))
    assert np.array_equal(be.ntt(cos, log2n, inverse=True, coset_shift=shift).download(), a)


def test_ntt_batch_and_definition(be):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(77)
    log2n, n, batch = 8, 256, 5
    a = rand_fr(rng, n * batch)
    out = be.ntt(be.upload(a, KIND_FR), log2n, batch=batch).download().reshape(batch, n, 32)
    for b in range(batch):
        assert np.array_equal(out[b], ora.dft_naive(a.reshape(batch, n, 32)[b]))


def test_ntt_round_trip_large(be):
    """2^20: inverse(forward(x)) == x, and the transform of a delta is all ones."""
    from project_b200 import KIND_FR

    rng = np.random.default_rng(78)
    log2n, n = 20, 1 << 20
    a = rand_fr(rng, n)
    fwd = be.ntt(be.upload(a, KIND_FR), log2n)
    assert np.array_equal(be.ntt(fwd, log2n, inverse=True).download(), a)
    delta = np.zeros((n, 32), dtype=np.uint8)
    delta[0, 0] = 1
    out = be.ntt(be.upload(delta, KIND_FR), log2n).download()
    assert np.array_equal(out, np.tile(fr_array([1]), (n, 1)))


def test_coset_lde_matches_oracle_composition(be):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(79)
    log2n, n, blow = 9, 512, 2
    evals = rand_fr(rng, n)
    shift = fr_array([5])
    got = be.coset_lde(be.upload(evals, KIND_FR), log2n, blow, shift).download()
    coeffs = ora.ntt(evals, inverse=True)
    padded = np.zeros((n << blow, 32), dtype=np.uint8)
    padded[:n] = coeffs
    assert np.array_equal(got, ora.ntt(padded, coset_shift=shift))


@pytest.mark.parametrize("n", [2, 16, 4096, 100000])
def test_fold(be, n):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(n)
    t = rand_fr(rng, n)
    r = rand_fr(rng, 1)[0]
    want = ora.fold(t, r)
    assert np.array_equal(be.fold(be.upload(t, KIND_FR), n, r).download(), want)
    # every pairing of table form and output form
    from project_b200 import KIND_FR_MONT

    for table_kind in (KIND_FR, KIND_FR_MONT):
        for out_kind in (KIND_FR, KIND_FR_MONT):
            out = be.alloc(out_kind, n // 2)
            be.fold(be.upload(t, table_kind), n, r, out=out)
            assert np.array_equal(out.download(), want), (table_kind, out_kind)


def test_sumcheck_rounds_fold_to_the_multilinear_evaluation(be):
    """Run all rounds of a sumcheck-style fold on a 2^12 table, sharded over 2 'ranks' per
    round: the round sums must satisfy s(0)+s(1) = previous claim, s(2) = 2 s(1) - s(0), and
    the final value must equal the table folded by the oracle."""
    from project_b200 import KIND_FR, fr_sum
    import pyref
    from pyref import R, fr_ints

    rng = np.random.default_rng(55)
    n = 1 << 12
    t = rand_fr(rng, n)
    claim = sum(fr_ints(t)) % R
    cur_host = t
    cur = be.upload(t, KIND_FR)
    while n > 1:
        half = n // 2
        if n >= 4:
            # two ranks, each owning half of the table (an even number of entries)
            parts = [be.sumcheck_round_sums(be.upload(cur_host[:half], KIND_FR), half), be.sumcheck_round_sums(be.upload(cur_host[half:], KIND_FR), half)]
            sums = fr_sum(np.stack(parts))
        else:
            sums = be.sumcheck_round_sums(cur, n)
        s0, s1, s2 = fr_ints(sums)
        assert (s0 + s1) % R == claim
        assert s2 == (2 * s1 - s0) % R
        r = rand_fr(rng, 1)[0]
        r_int = fr_ints(r)[0]
        claim = (s0 + r_int * (s1 - s0)) % R
        nxt = be.fold(cur, n, r)
        cur_host = nxt.download()
        assert np.array_equal(cur_host, ora.fold(ora.fr_binop(0, cur.download() if cur.kind == 0 else cur.download(), np.zeros((n, 32), np.uint8)), r))
        cur, n = nxt, half
    assert fr_ints(cur_host)[0] == claim

"""GPU parity of the column builders (running sums, segmented states, bindings)
against the CPU oracle, through the C ABI, bit-exact."""
import numpy as np
import pytest

import oracle_lib as ora
from pyref import R, fr_array

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


def selector(valid, n):
    s = np.zeros((n, 32), dtype=np.uint8)
    s[:valid, 0] = 1
    return s


@pytest.mark.parametrize("n,t_valid,q_valid", [(16, 9, 13), (1024, 1000, 700), (5000, 4999, 4999), (40000, 12345, 33333), (1, 0, 0), (2, 1, 1)])
def test_logup_accumulator(be, n, t_valid, q_valid):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(n)
    table, query, mult = rand_fr(rng, n), rand_fr(rng, n), rand_fr(rng, n)
    qt, qq = selector(t_valid, n), selector(q_valid, n)
    beta = fr_array([int(rng.integers(1, 1 << 62))])
    active = ora.active_transition_count(qt, qq)
    want = ora.logup_accumulator(table, query, mult, qt, qq, beta, active)
    bufs = [be.upload(x, KIND_FR) for x in (table, query, mult, qt, qq)]
    got = be.logup_accumulator(*bufs, n, beta, active).download()
    assert np.array_equal(got, want)


def test_logup_small_integer_inputs_and_zero_denominator(be):
    from project_b200 import KIND_FR, KIND_I64, KIND_U32, GzkError

    rng = np.random.default_rng(5)
    n = 3000
    table_i = rng.integers(-500, 500, size=n, dtype=np.int64)
    query_i = rng.integers(-500, 500, size=n, dtype=np.int64)
    mult_u = rng.integers(0, 50, size=n, dtype=np.uint32)
    qt, qq = selector(2500, n), selector(2999, n)
    beta = fr_array([987654321987])
    want = ora.logup_accumulator(ora.fr_from_i64(table_i), ora.fr_from_i64(query_i), ora.fr_from_i64(mult_u.astype(np.int64)), qt, qq, beta, 2999)
    got = be.logup_accumulator(be.upload(table_i, KIND_I64), be.upload(query_i, KIND_I64), be.upload(mult_u, KIND_U32),
                               be.upload(qt, KIND_FR), be.upload(qq, KIND_FR), n, beta, 2999).download()
    assert np.array_equal(got, want)
    # beta = -table[7] makes a denominator vanish: the reference throws, the library reports GZK_E_DOMAIN
    bad_beta = fr_array([(-int(table_i[7])) % R])
    with pytest.raises(GzkError) as e:
        be.logup_accumulator(be.upload(table_i, KIND_I64), be.upload(query_i, KIND_I64), be.upload(mult_u, KIND_U32),
                             be.upload(qt, KIND_FR), be.upload(qq, KIND_FR), n, bad_beta, 2999)
    assert e.value.code == 3


@pytest.mark.parametrize("n,valid", [(16, 9), (2048, 2047), (2048, 0), (70000, 45678)])
def test_route_accumulators(be, n, valid):
    from project_b200 import KIND_FR, GzkError

    rng = np.random.default_rng(n + valid)
    table, mult = rand_fr(rng, n), rand_fr(rng, n)
    beta = fr_array([int(rng.integers(1, 1 << 62))])
    got = be.route_node_accumulator(be.upload(table, KIND_FR), be.upload(mult, KIND_FR), valid, n, beta).download()
    assert np.array_equal(got, ora.route_node_accumulator(table, mult, valid, beta))
    got = be.route_edge_accumulator(be.upload(table, KIND_FR), valid, n, beta).download()
    assert np.array_equal(got, ora.route_edge_accumulator(table, valid, beta))
    with pytest.raises(GzkError):
        be.route_edge_accumulator(be.upload(table, KIND_FR), n, n, beta)


@pytest.mark.parametrize("n", [1, 5, 1024, 1025, 50000])
def test_group_prefix_state(be, n):
    from project_b200 import KIND_FR, KIND_U32, GzkError

    rng = np.random.default_rng(n)
    values = rand_fr(rng, n)
    q = (rng.random(n) < 0.15).astype(np.uint32)
    if n > 3000:
        q[1500:4200] = 0  # one segment spanning several CTAs
    want = ora.group_prefix_state(values, fr_array([int(v) for v in q]))
    got = be.group_prefix_state(be.upload(values, KIND_FR), be.upload(q, KIND_U32), n).download()
    assert np.array_equal(got, want)
    if n >= 5:
        q2 = q.copy()
        q2[3] = 2
        with pytest.raises(GzkError):
            be.group_prefix_state(be.upload(values, KIND_FR), be.upload(q2, KIND_U32), n)


@pytest.mark.parametrize("count,domain", [(0, 8), (6, 16), (1023, 1024), (5000, 8192)])
def test_zkmap_accumulator(be, count, domain):
    from project_b200 import KIND_FR, GzkError

    rng = np.random.default_rng(count)
    a, b = rand_fr(rng, max(count, 1)), rand_fr(rng, max(count, 1))
    want_acc, want_mu = ora.zkmap_accumulator(a[:count], b[:count], domain)
    acc, mu = be.zkmap_accumulator(be.upload(a, KIND_FR), be.upload(b, KIND_FR), count, domain)
    assert np.array_equal(acc.download(), want_acc)
    assert np.array_equal(mu, want_mu)
    with pytest.raises(GzkError):
        be.zkmap_accumulator(be.upload(a, KIND_FR), be.upload(b, KIND_FR), domain, domain)

"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle.

Bit-exact comparison of 32-byte canonical field elements on seeded inputs."""
import random

import numpy as np
import pytest

import oracle_lib as ora
import pyref
from pyref import R, fr_array, fr_ints

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from project_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


def rand_fr_bytes(rng, n):
    """n uniform field elements as [n,32] uint8 (numpy-generated, rejection sampled)."""
    a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    a[:, 31] &= 0x3F  # < 2^254 < r
    return a


def test_root_of_unity(be):
    for log2n in (0, 1, 10, 22, 32):
        assert np.array_equal(be.root_of_unity(1 << log2n), ora.root_of_unity(1 << log2n))
    from project_b200 import GzkError

    with pytest.raises(GzkError):
        be.root_of_unity(12)


def test_buffer_round_trip(be):
    from project_b200 import KIND_FR, KIND_FR_MONT

    rng = np.random.default_rng(1)
    a = rand_fr_bytes(rng, 1000)
    a[0] = 0
    a[1] = fr_array([R - 1])[0]
    for kind in (KIND_FR, KIND_FR_MONT):
        buf = be.upload(a, kind)
        assert np.array_equal(buf.download(), a)
        buf.free()


@pytest.mark.parametrize("log2n", [0, 1, 4, 10, 11, 15, 18])
def test_bary_weights(be, log2n):
    rng = random.Random(100 + log2n)
    x = fr_array([rng.randrange(1 << 64)])
    n = 1 << log2n
    w = be.bary_weights(log2n, x)
    got = w.download()
    want = ora.bary_weights(x, n)
    assert np.array_equal(got, want)
    w.free()


@pytest.mark.parametrize("log2n,keeps", [(12, (0, 1, 255, 256, 257, 1023, 1024, 3000, 4096)),
                                         (20, (0, 1, 1000, 1024, 1025, 70000, (1 << 18) - 1024, (1 << 18) - 1, 1 << 18, 600000, 1 << 20))])
def test_bary_weights_prefix(be, log2n, keeps):
    """Only the quartets below the kept prefix and the ones holding the last two weights run: the first `keep` weights
    and the last two are the whole vector's; nothing else of the output is relied on."""
    from project_b200 import KIND_FR, KIND_FR_MONT

    rng = random.Random(300 + log2n)
    x = fr_array([rng.randrange(1 << 64)])
    n = 1 << log2n
    want = ora.bary_weights(x, n)
    for keep in keeps:
        out = be.upload(np.full((n, 32), 0x11, dtype=np.uint8), KIND_FR)
        out.retag(KIND_FR_MONT)
        got = be.bary_weights_prefix(log2n, x, keep, out).download()
        assert np.array_equal(got[:keep], want[:keep]), keep
        assert np.array_equal(got[n - 2:], want[n - 2:]), keep
        out.free()


def test_bary_weights_multi(be):
    rng = random.Random(77)
    for log2n, count in ((10, 3), (15, 4), (18, 2), (12, 6), (19, 2)):
        xs = [fr_array([rng.randrange(1 << 64)]) for _ in range(count)]
        outs = be.bary_weights_multi(log2n, xs)
        for x, w in zip(xs, outs):
            assert np.array_equal(w.download(), ora.bary_weights(x, 1 << log2n)), (log2n, count)
            w.free()


def test_bary_weights_point_on_domain(be):
    from project_b200 import GzkError

    om = ora.root_of_unity(16)
    with pytest.raises(GzkError) as e:
        be.bary_weights(4, om)
    assert e.value.code == 3


@pytest.mark.parametrize("k,log2n,length,rots", [
    (1, 4, 16, (0,)),
    (5, 6, 64, (0, 1)),
    (3, 10, 1000, (0,)),
    (43, 12, 4096, (0, 1)),
    (7, 15, 32768, (0, 1, 5)),
    (380, 10, 1024, (0, 1)),
    (2, 18, 200001, (0, 1)),
])
def test_eval_batch_matches_oracle(be, k, log2n, length, rots):
    from project_b200 import KIND_FR

    rng = np.random.default_rng(k * 1000 + log2n)
    n = 1 << log2n
    cols = np.zeros((k, n, 32), dtype=np.uint8)
    cols[:, :length] = rand_fr_bytes(rng, k * length).reshape(k, length, 32)
    x = fr_array([int(rng.integers(1, 1 << 62))])
    w = be.bary_weights(log2n, x)
    w_host = w.download()
    bufs = [be.upload(cols[i, :length], KIND_FR) for i in range(k)]
    got = be.eval_batch(bufs, length, log2n, w, rots)
    want = ora.eval_rotations(cols, w_host, rots, threads=8)
    assert np.array_equal(got, want)
    for b in bufs:
        b.free()
    w.free()


def test_eval_small_integer_and_montgomery_columns(be):
    from project_b200 import KIND_FR_MONT, KIND_I64, KIND_U32

    rng = np.random.default_rng(7)
    log2n, n = 9, 512
    x = fr_array([123456789])
    w = be.bary_weights(log2n, x)
    w_host = w.download()
    i64 = rng.integers(-(1 << 40), 1 << 40, size=n, dtype=np.int64)
    i64[:3] = [0, -1, np.iinfo(np.int64).min + 1]
    u32 = rng.integers(0, 1 << 32, size=n, dtype=np.uint64).astype(np.uint32)
    fr = rand_fr_bytes(rng, n)
    bufs = [be.upload(i64, KIND_I64), be.upload(u32, KIND_U32), be.upload(fr, KIND_FR_MONT)]
    got = be.eval_batch(bufs, n, log2n, w, (0, 1))
    cols = np.stack([ora.fr_from_i64(i64), fr_array([int(v) for v in u32]), fr])
    want = ora.eval_rotations(cols, w_host, (0, 1))
    assert np.array_equal(got, want)


def test_eval_empty_and_errors(be):
    from project_b200 import GzkError, KIND_FR

    w = be.bary_weights(4, fr_array([99]))
    col = be.upload(np.zeros((16, 32), dtype=np.uint8), KIND_FR)
    out = be.eval_batch([col], 0, 4, w, (0,))
    assert not out.any()
    with pytest.raises(GzkError):
        be.eval_batch([col], 17, 4, w, (0,))  # len beyond the domain
    with pytest.raises(GzkError):
        be.eval_batch([col], 16, 4, w, (16,))  # rotation out of range
    with pytest.raises(GzkError):
        be.eval_batch([col], 16, 4, col, (0,))  # weights not Montgomery


def test_commit_equals_barycentric_evaluation(be):
    """Size-independent property at a large size: the weight vector sums to one, and a
    column that is the evaluation of a known low-degree polynomial evaluates to
    that polynomial at x."""
    from project_b200 import KIND_FR

    log2n, n = 20, 1 << 20
    x = 0x1234567890ABCDEF
    w = be.bary_weights(log2n, fr_array([x]))
    om = pyref.root_of_unity(n)
    # f(X) = 3 + 5 X  evaluated on the domain: f(omega^i)
    ones = np.tile(fr_array([1]), (n, 1))
    c1 = be.upload(ones, KIND_FR)
    got = fr_ints(be.eval_batch([c1], n, log2n, w, (0,))[0])
    assert got == [1]
    # linear column via numpy-free big ints would be slow at 2^20; use the
    # rotation identity instead: sum_c w[c] * col[(c+1) mod n] for col = w-independent constant
    got = fr_ints(be.eval_batch([c1], n, log2n, w, (0, 1, 12345))[:, 0])
    assert got == [1, 1, 1]


def test_golden_fixtures_through_the_c_abi(be):
    """The committed fixtures (tests/golden/hotpath_small.json, produced from Python
    integers) reproduced by the CUDA library."""
    import json
    import os

    from project_b200 import KIND_FR

    with open(os.path.join(os.path.dirname(__file__), "golden", "hotpath_small.json")) as f:
        g = json.load(f)
    hx = lambda s: np.frombuffer(bytes.fromhex(s), dtype=np.uint8)
    assert bytes(be.root_of_unity(g["omega"]["n"])).hex() == g["omega"]["value"]
    bw = g["bary"]
    log2n = bw["n"].bit_length() - 1
    assert be.bary_weights(log2n, hx(bw["x"])).download().tobytes().hex() == bw["weights"]
    ev = g["eval"]
    cols = hx(ev["columns"]).reshape(ev["k"], ev["n"], 32)
    w = be.upload(hx(ev["weights"]).reshape(-1, 32), 1)  # KIND_FR_MONT: converted on upload
    out = be.eval_batch([be.upload(cols[i], KIND_FR) for i in range(ev["k"])], ev["n"], ev["n"].bit_length() - 1, w, ev["rotations"])
    assert out.tobytes().hex() == ev["out"]
    g1 = g["g1_same_base"]
    assert be.g1_mul_same_base(hx(g1["base"]), hx(g1["scalars"]).reshape(-1, 32)).tobytes().hex() == g1["points"]
    lg = g["logup"]
    bufs = [be.upload(hx(lg[k]).reshape(-1, 32), KIND_FR) for k in ("table", "query", "mult", "q_table", "q_query")]
    n = bufs[0].count
    assert be.logup_accumulator(*bufs, n, hx(lg["beta"]), lg["active"]).download().tobytes().hex() == lg["out"]


def test_bounded_wait_that_runs_out_returns_timeout():
    """Failure handling without a fault: with the stall injection on, the kernel's chunk barriers are armed
    but no copy is issued, every bounded wait gives up, and the call returns GZK_E_TIMEOUT (4); the context
    stays usable and the next call is correct."""
    from project_b200 import KIND_FR, Backend, GzkError
    from project_b200.lib import inject_eval_stall

    be = Backend(0)
    rng = np.random.default_rng(11)
    log2n, k = 11, 4
    n = 1 << log2n
    cols = rng.integers(0, 256, size=(k, n, 32), dtype=np.uint8)
    cols[:, :, 31] &= 0x3F
    x = np.zeros(32, dtype=np.uint8)
    x[0] = 9
    w = be.bary_weights(log2n, x)
    bufs = [be.upload(cols[i], KIND_FR) for i in range(k)]
    inject_eval_stall(True)
    try:
        with pytest.raises(GzkError) as info:
            be.eval_batch(bufs, n, log2n, w, (0, 1))
        assert info.value.code == 4
    finally:
        inject_eval_stall(False)
    got = be.eval_batch(bufs, n, log2n, w, (0, 1))
    assert np.array_equal(got, ora.eval_rotations(cols, w.download(), (0, 1)))
    be.close()


def test_small_deferred_uploads_are_staged_in_order(be):
    """Deferred mode queues uploads of at most 256 KiB through a ring of 16 pinned slots without waiting: forty
    uploads from one reused host array (more than the ring holds) must each arrive with the data they were given,
    a larger one (the waiting path) in between included."""
    from project_b200 import KIND_FR, KIND_FR_MONT, KIND_I64

    rng = np.random.default_rng(5)
    be.set_deferred(True)
    try:
        host = np.zeros(3000, dtype=np.int64)
        bufs, want = [], []
        for i in range(40):
            host[:] = rng.integers(-(1 << 40), 1 << 40, size=host.size)
            want.append(host.copy())
            bufs.append(be.upload(host, KIND_I64))
            if i == 20:
                big = rng.integers(0, 1 << 62, size=70000, dtype=np.int64)  # 560 KB: not staged
                big_buf = be.upload(big, KIND_I64)
        mont = rand_fr_local(rng, 500)
        mont_buf = be.upload(mont, KIND_FR_MONT)  # converted on the device behind the staged copy
        be.synchronize()
        for b, w in zip(bufs, want):
            assert np.array_equal(b.download(), w)
            b.free()
        assert np.array_equal(big_buf.download(), big)
        assert np.array_equal(mont_buf.download(), mont)
    finally:
        be.set_deferred(False)


def rand_fr_local(rng, n):
    a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    a[:, 31] &= 0x3F
    return a


def test_contexts_ordered_on_the_device(be):
    """gzk_ctx_wait_for: a second context (its own stream) consumes what the first one has only queued, and the first
    one then consumes the second one's result, with no host synchronisation in between."""
    from project_b200 import KIND_FR, KIND_I64, Backend

    rng = np.random.default_rng(11)
    side = Backend(0)
    n, log2n = 1 << 18, 18
    x = fr_array([int(rng.integers(2, 1 << 62))])
    one = np.frombuffer((1).to_bytes(32, "little"), dtype=np.uint8)
    a, b = rng.integers(-1000, 1000, size=n, dtype=np.int64), rng.integers(-1000, 1000, size=n, dtype=np.int64)
    be.set_deferred(True)
    side.set_deferred(True)
    try:
        ba, bb = be.upload(a, KIND_I64), be.upload(b, KIND_I64)
        w = be.bary_weights(log2n, x)                                        # queued on the main context
        col = be.linear_combination([ba, bb], np.concatenate([one, x.reshape(32)]), n, n)  # a + x b, queued behind it
        side.wait_for(be)
        out = side.alloc(KIND_FR, 2)
        side.eval_batch_range_device([col], n, 0, log2n, w, 0, (0, 1), out)  # reads both on the side stream
        be.wait_for(side)
        got = out.download()                                                  # a read through the main context
        side.synchronize()
    finally:
        be.set_deferred(False)
        side.set_deferred(False)
    xi = fr_ints(x)[0]
    col_host = fr_array([(int(u) + xi * int(v)) % R for u, v in zip(a, b)])
    want = ora.eval_rotations(col_host[None, :, :], ora.bary_weights(x, n), (0, 1))
    assert np.array_equal(got.reshape(2, 32), want.reshape(2, 32))
    side.close()


@pytest.mark.parametrize("length", [512, 389])
@pytest.mark.parametrize("rots", [(0, 1), (3, 500)])
def test_eval_groups_of_integer_columns_on_the_tensor_path(be, length, rots):
    """Seven and nine small-integer columns (I64 with negative and extreme values, U32 among them) beside two
    field-element columns at two evaluation points: whole groups of four integer columns, a group of three, and a
    column left over for the integer pipe, all against the oracle (eval_backend.cpp:191-444 semantics:
    FieldElement::from_signed for negative entries)."""
    from project_b200 import KIND_FR, KIND_FR_MONT, KIND_I64, KIND_U32

    rng = np.random.default_rng(41)
    log2n, n = 9, 512
    w = be.bary_weights(log2n, fr_array([987654321]))
    w_host = w.download()
    for integer_columns in (7, 9):
        cols, bufs = [], []
        for i in range(integer_columns):
            if i % 3 == 2:
                u32 = rng.integers(0, 1 << 32, size=n, dtype=np.uint64).astype(np.uint32)
                u32[:2] = [0, 0xFFFFFFFF]
                bufs.append(be.upload(u32, KIND_U32))
                cols.append(fr_array([int(v) for v in u32]))
            else:
                i64 = rng.integers(-(1 << 50), 1 << 50, size=n, dtype=np.int64)
                i64[:5] = [0, -1, 1, np.iinfo(np.int64).min + 1, np.iinfo(np.int64).max]
                bufs.append(be.upload(i64, KIND_I64))
                cols.append(ora.fr_from_i64(i64))
        for kind in (KIND_FR, KIND_FR_MONT):
            fr = rand_fr_bytes(rng, n)
            bufs.insert(1, be.upload(fr, kind))
            cols.insert(1, fr)
        got = be.eval_batch(bufs, length, log2n, w, rots)
        padded = np.stack(cols).copy()
        padded[:, length:] = 0  # the rows behind `length` are not part of the columns
        want = ora.eval_rotations(padded, w_host, rots)
        assert np.array_equal(got, want)
        for b in bufs:
            b.free()
    w.free()


def test_eval_long_units_fold_their_byte_products_in_time(be):
    """With many columns in one call the tile count is capped and a (tile, column) unit grows past 32768 rows, the
    most the s32 byte products of the tensor path can take before they are folded into the running sum.  600 aliases
    of one column of 2^25 rows at two points must all evaluate to what a single-column call gives (short units, and
    for the integer column the integer-pipe kernel): a size-independent check of the mid-unit fold of both tensor
    kernels."""
    from project_b200 import KIND_I64

    log2n, n = 25, 1 << 25
    w = be.bary_weights(log2n, fr_array([(1 << 200) + 12345]))
    field_column = be.bary_weights(log2n, fr_array([(1 << 100) + 7]))  # any 2^25 field elements will do
    rng = np.random.default_rng(3)
    values = rng.integers(-(1 << 45), 1 << 45, size=n, dtype=np.int64)
    integer_column = be.upload(values, KIND_I64)
    for column in (field_column, integer_column):
        single = be.eval_batch([column], n, log2n, w, (0, 1))
        many = be.eval_batch([column] * 600, n, log2n, w, (0, 1))
        assert many.shape == (2, 600, 32)
        assert np.array_equal(many, np.broadcast_to(single, many.shape))
    integer_column.free()
    field_column.free()
    w.free()

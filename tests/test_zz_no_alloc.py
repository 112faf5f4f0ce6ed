"""The allocation-free packed evaluation (gzk_eval_batch_static) against the regular
entry point (gzk_eval_batch), both through the C ABI.

Some callers of the library cannot allocate while they run (their own pool owns
the GPU's memory, or they cannot take the device-wide stall of a cudaMalloc), so
this variant works out of a fixed array inside the library.  The array is shared
by all calls and keeps the previous call's contents, hence two calls in a row of
different shapes: the second must not be disturbed by what the first left behind.
Results must be bit-identical to gzk_eval_batch.  Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _columns(rng, k, n):
    a = rng.integers(0, 256, size=(k, n, 32), dtype=np.uint8)
    a[:, :, 31] &= 0x3F
    return a


def test_static_entry_point_matches_regular_one_twice():
    from project_b200 import KIND_FR, KIND_I64, Backend, GzkError
    from project_b200.lib import eval_batch_static

    be = Backend(0)
    rng = np.random.default_rng(99)
    x = np.zeros(32, dtype=np.uint8)
    x[:8] = np.frombuffer((0xC0FFEE1234567).to_bytes(8, "little"), dtype=np.uint8)

    def run_case(log2n, k, length, rotations, with_i64):
        n = 1 << log2n
        w = be.bary_weights(log2n, x)
        host = _columns(rng, k, n)
        bufs = [be.upload(host[i, :length], KIND_FR) for i in range(k)]
        if with_i64:
            bufs.append(be.upload(rng.integers(-1000, 1000, size=length, dtype=np.int64), KIND_I64))
        want = be.eval_batch(bufs, length, log2n, w, rotations)
        out = be.alloc(KIND_FR, len(rotations) * len(bufs))
        be.synchronize()
        eval_batch_static(0, be.stream, [b.device_ptr for b in bufs], [b.kind for b in bufs], length, log2n,
                          w.device_ptr, rotations, out.device_ptr)
        be.synchronize()
        got = out.download().reshape(len(rotations), len(bufs), 32)
        assert np.array_equal(got, want)
        for b in bufs + [w, out]:
            b.free()

    # two calls in a row; the second is smaller and of another shape than the first
    run_case(14, 37, 16384, (0, 1), with_i64=True)
    run_case(10, 5, 777, (3,), with_i64=False)

    # sizes beyond the fixed work area are rejected with a message
    w = be.bary_weights(4, x)
    col = be.upload(np.zeros((16, 32), dtype=np.uint8), KIND_FR)
    out = be.alloc(KIND_FR, 1024)
    with pytest.raises(GzkError, match="256 columns"):
        eval_batch_static(0, be.stream, [col.device_ptr] * 257, [KIND_FR] * 257, 16, 4, w.device_ptr, (0,), out.device_ptr)
    with pytest.raises(GzkError, match="2 rotations"):
        eval_batch_static(0, be.stream, [col.device_ptr], [KIND_FR], 16, 4, w.device_ptr, (0, 1, 2), out.device_ptr)
    be.close()

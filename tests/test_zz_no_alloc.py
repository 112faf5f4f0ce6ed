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
    # a misaligned or non-device pointer is refused on the host, before anything is launched
    with pytest.raises(GzkError, match="misaligned"):
        eval_batch_static(0, be.stream, [col.device_ptr + 4], [KIND_FR], 15, 4, w.device_ptr, (0,), out.device_ptr)
    with pytest.raises(GzkError, match="misaligned"):
        eval_batch_static(0, be.stream, [col.device_ptr], [KIND_FR], 16, 4, w.device_ptr + 16, (0,), out.device_ptr)
    host_memory = np.zeros(16 * 32 + 64, dtype=np.uint8)
    host_ptr = (host_memory.ctypes.data + 31) & ~31
    with pytest.raises(GzkError, match="not memory of this GPU"):
        eval_batch_static(0, be.stream, [host_ptr], [KIND_FR], 16, 4, w.device_ptr, (0,), out.device_ptr)
    be.close()


def test_static_entry_point_poisons_outputs_when_a_wait_runs_out():
    """A bounded wait that gives up must not come back as a plausible result: with the stall
    injection on, the outputs of the call are 0xFF bytes; the next call (injection off)
    clears the status word itself and is correct again."""
    from project_b200 import KIND_FR, Backend
    from project_b200.lib import eval_batch_static, inject_eval_stall

    be = Backend(0)
    rng = np.random.default_rng(5)
    log2n, k = 10, 3
    n = 1 << log2n
    x = np.zeros(32, dtype=np.uint8)
    x[0] = 77
    w = be.bary_weights(log2n, x)
    host = _columns(rng, k, n)
    bufs = [be.upload(host[i], KIND_FR) for i in range(k)]
    want = be.eval_batch(bufs, n, log2n, w, (0, 1))
    out = be.alloc(KIND_FR, 2 * k)
    be.synchronize()
    args = (0, be.stream, [b.device_ptr for b in bufs], [b.kind for b in bufs], n, log2n, w.device_ptr, (0, 1), out.device_ptr)
    inject_eval_stall(True)
    try:
        eval_batch_static(*args)
        be.synchronize()
    finally:
        inject_eval_stall(False)
    assert np.all(out.download() == 0xFF)
    eval_batch_static(*args)
    be.synchronize()
    assert np.array_equal(out.download().reshape(2, k, 32), want)
    be.close()

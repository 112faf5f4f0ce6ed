"""Row-sharded transform: the ranks of a multi-GPU run emulated in one process on one GPU
(the exchange goes through the host), against the oracle's transform of the whole vector."""
import numpy as np
import pytest

import oracle_lib as ora

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


def test_transpose_swap_and_twiddle(be):
    from project_b200 import KIND_FR, KIND_FR_MONT
    from pyref import R, fr_array

    rng = np.random.default_rng(3)
    rows, cols = 37, 70
    m = rand_fr(rng, rows * cols)
    got = be.transpose(be.upload(m, KIND_FR), rows, cols).download()
    assert np.array_equal(got.reshape(cols, rows, 32), m.reshape(rows, cols, 32).transpose(1, 0, 2))
    d0, d1, d2 = 5, 3, 11
    t = rand_fr(rng, d0 * d1 * d2)
    got = be.swap_outer(be.upload(t, KIND_FR), d0, d1, d2).download()
    assert np.array_equal(got.reshape(d1, d0, d2, 32), t.reshape(d0, d1, d2, 32).transpose(1, 0, 2, 3))
    # twiddles: a block of ones becomes omega^((row_first + r) * c)
    log2n, row_first, r_count, c_count = 10, 13, 6, 32
    omega = int.from_bytes(ora.root_of_unity(1 << log2n).tobytes(), "little")
    for inverse in (False, True):
        block = be.powers(fr_array([1]), r_count * c_count)  # a Montgomery buffer of ones
        be.ntt_twiddle(block, log2n, row_first, r_count, c_count, inverse=inverse)
        got = block.download()
        base = pow(omega, R - 2, R) if inverse else omega
        want = fr_array([pow(base, ((row_first + r) * c) % (1 << log2n), R) for r in range(r_count) for c in range(c_count)])
        assert np.array_equal(got, want)


@pytest.mark.parametrize("log2n,world", [(4, 2), (9, 2), (12, 4), (15, 8), (16, 2)])
def test_sharded_forward_matches_oracle_and_inverse_round_trips(be, log2n, world):
    from project_b200 import KIND_FR
    from project_b200 import sharded_ntt as sn

    rng = np.random.default_rng(log2n * 10 + world)
    n = 1 << log2n
    x = rand_fr(rng, n)
    want = ora.ntt(x)
    l1, l2 = sn.split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1 = n1 // world
    inputs = [be.upload(x[g * rows1 * n2:(g + 1) * rows1 * n2], KIND_FR) for g in range(world)]
    outs = sn.run_emulated([be] * world, inputs, log2n, sn.forward)
    # rank g holds X[k1 + n1*k2] as [k1 local][k2]
    got = np.zeros_like(want)
    for g, o in enumerate(outs):
        block = o.download().reshape(rows1, n2, 32)
        k1 = g * rows1 + np.arange(rows1)
        for k2 in range(n2):
            got[k1 + n1 * k2] = block[:, k2]
    assert np.array_equal(got, want)
    back = sn.run_emulated([be] * world, outs, log2n, sn.inverse)
    for g, b in enumerate(back):
        assert np.array_equal(b.download(), x[g * rows1 * n2:(g + 1) * rows1 * n2])


def test_sharded_transform_with_preallocated_work_buffers(be):
    """The allocation-free form used under NCCL: two work buffers per rank, refilled and retagged in place."""
    from project_b200 import KIND_FR, KIND_FR_MONT
    from project_b200 import sharded_ntt as sn

    rng = np.random.default_rng(4242)
    log2n, world = 13, 4
    n = 1 << log2n
    x = rand_fr(rng, n)
    want = ora.ntt(x)
    l1, l2 = sn.split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1 = n1 // world
    local = rows1 * n2
    inputs = [be.upload(x[g * local:(g + 1) * local], KIND_FR) for g in range(world)]
    works = [(be.alloc(KIND_FR, local), be.alloc(KIND_FR_MONT, local)) for _ in range(world)]
    for _ in range(2):  # twice: the second run starts from work buffers left in the Montgomery kind
        outs = sn.run_emulated([be] * world, inputs, log2n, sn.forward, works=works)
        for g, o in enumerate(outs):
            assert o is works[g][1]
            block = o.download().reshape(rows1, n2, 32)
            k1 = g * rows1 + np.arange(rows1)
            for k2 in range(0, n2, 7):
                assert np.array_equal(block[:, k2], want[k1 + n1 * k2])
    # the inverse from a copy of the transposed output, through its own work buffers
    xt = [be.upload(o.download(), KIND_FR_MONT) for o in outs]
    works_inv = [(be.alloc(KIND_FR_MONT, local), be.alloc(KIND_FR_MONT, local)) for _ in range(world)]
    back = sn.run_emulated([be] * world, xt, log2n, sn.inverse, works=works_inv)
    for g, b in enumerate(back):
        assert np.array_equal(b.download(), x[g * local:(g + 1) * local])

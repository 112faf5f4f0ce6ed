"""World-size-2 gloo test of the exchange pattern of the row-sharded transform: the host
sequence of project_b200.sharded_ntt runs on a stand-in backend (numpy data movement, the
CPU oracle for the row transforms and twiddles) with a real all_to_all between two processes."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _HostBuf:
    def __init__(self, data, kind=0):
        self.data, self.kind = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1, 32), kind

    def retag(self, kind):
        self.kind = kind
        return self

    def free(self):
        self.data = None


class _HostBackend:
    """The calls the sequence makes, on host arrays of canonical field elements."""

    def __init__(self, ora, pyref):
        self.ora, self.pyref = ora, pyref

    def alloc(self, kind, count):
        return _HostBuf(np.zeros((count, 32), np.uint8), kind)

    def synchronize(self):
        pass

    def swap_outer(self, b, d0, d1, d2, out):
        out.data = np.ascontiguousarray(b.data.reshape(d0, d1, d2, 32).transpose(1, 0, 2, 3)).reshape(-1, 32)
        return out

    def transpose(self, b, rows, cols, out):
        out.data = np.ascontiguousarray(b.data.reshape(rows, cols, 32).transpose(1, 0, 2)).reshape(-1, 32)
        return out

    def ntt(self, b, log2n, batch=1, inverse=False, out=None):
        n = 1 << log2n
        rows = b.data.reshape(batch, n, 32)
        out.data = np.concatenate([self.ora.ntt(np.ascontiguousarray(rows[i]), inverse=inverse) for i in range(batch)])
        return out

    def ntt_twiddle(self, b, log2n, row_first, rows, cols, inverse=False):
        R = self.pyref.R
        omega = int.from_bytes(self.ora.root_of_unity(1 << log2n).tobytes(), "little")
        if inverse:
            omega = pow(omega, R - 2, R)
        tw = self.pyref.fr_array([pow(omega, ((row_first + r) * c) % (1 << log2n), R) for r in range(rows) for c in range(cols)])
        b.data = self.ora.fr_binop(2, b.data, tw)
        return b


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import oracle_lib as ora
    import pyref
    from project_b200 import sharded_ntt as sn

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    log2n = 8
    n = 1 << log2n
    rng = np.random.default_rng(77)  # same vector on every rank
    x = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    x[:, 31] &= 0x3F
    want = ora.ntt(x)
    l1, l2 = sn.split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1 = n1 // world
    be = _HostBackend(ora, pyref)

    def drive(gen):
        try:
            send = next(gen)
            while True:
                src = torch.from_numpy(send.data.copy())
                dst = torch.empty_like(src)
                dist.all_to_all_single(dst, src)
                send = gen.send(_HostBuf(dst.numpy()))
        except StopIteration as done:
            return done.value

    mine = _HostBuf(x[rank * rows1 * n2:(rank + 1) * rows1 * n2])
    out = drive(sn.forward(be, mine, log2n, rank, world))
    block = out.data.reshape(rows1, n2, 32)
    ok = True
    for a in range(rows1):
        k1 = rank * rows1 + a
        for k2 in range(n2):
            ok = ok and np.array_equal(block[a, k2], want[k1 + n1 * k2])
    back = drive(sn.inverse(be, out, log2n, rank, world))
    ok = ok and np.array_equal(back.data, x[rank * rows1 * n2:(rank + 1) * rows1 * n2])
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_rank_gloo_sharded_transform(tmp_path):
    import torch.multiprocessing as mp

    import __graft_entry__ as entry

    entry.build()
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"

"""Row-sharded transform over several GPUs: the host-side sequence around the library's kernels.

A vector of n = 2^log2n field elements is split by contiguous rows: with n = n1*n2 and element
i = i1*n2 + i2, rank g of `world` holds rows i1 in [g*n1/world, (g+1)*n1/world).  The forward
transform leaves rank g with X[k1 + n1*k2] for k1 in its block, stored as [k1][k2] ("transposed
out"); the inverse takes that layout back to contiguous rows.  Pointwise work between the two
needs no exchange.

Both directions are generators: they yield a Buffer whose `world` equal chunks go to ranks
0..world-1 and expect to be sent the Buffer of chunks received from ranks 0..world-1 (an
all-to-all).  `NcclExchange` drives one rank with torch.distributed; `run_emulated` drives all ranks
of a single process in lockstep (tests on one GPU)."""
from .lib import KIND_FR_MONT


def split(log2n, world):
    """(log2 n1, log2 n2): both at least log2(world) so that rows and columns split evenly."""
    lw = world.bit_length() - 1
    if world != 1 << lw:
        raise ValueError("world must be a power of two")
    l1 = log2n // 2
    l2 = log2n - l1
    if l1 < lw:
        raise ValueError("2^log2n is too small to split over this many ranks")
    return l1, l2


def forward(be, x, log2n, rank, world, work=None):
    """x: this rank's rows [n1/world][n2] (FR or FR_MONT).  Returns [n1/world][n2] FR_MONT = X[k1 + n1*k2].
    `work` = two Buffers of the local size (one of x's kind, one FR_MONT) to run without
    allocating; the result is then work[1].  Received Buffers stay the driver's."""
    l1, l2 = split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1, cols2 = n1 // world, n2 // world
    a, b = work if work is not None else (be.alloc(x.kind, rows1 * n2), be.alloc(KIND_FR_MONT, rows1 * n2))
    a.retag(x.kind)
    recv = yield be.swap_outer(x, rows1, world, cols2, out=a)   # [dest][i1 local][i2 local] -> [i1][i2 local]
    a.retag(recv.kind)
    be.transpose(recv, n1, cols2, out=a)                         # [i2 local][i1]
    be.ntt(a, l1, batch=cols2, out=b)                            # [i2 local][k1]
    be.ntt_twiddle(b, log2n, rank * cols2, cols2, n1)            # * omega_n^(i2*k1)
    a.retag(KIND_FR_MONT)
    recv = yield be.swap_outer(b, cols2, world, rows1, out=a)    # [dest][i2 local][k1 local] -> [i2][k1 local]
    be.transpose(recv, n2, rows1, out=a)                         # [k1 local][i2]
    be.ntt(a, l2, batch=rows1, out=b)                            # [k1 local][k2]
    if work is None:
        be.synchronize()
        a.free()
    return b


def inverse(be, xt, log2n, rank, world, work=None):
    """xt: [n1/world][n2] FR_MONT as left by `forward`.  Returns this rank's contiguous rows, FR_MONT
    (work[1] when `work`, two FR_MONT Buffers of the local size, is given)."""
    l1, l2 = split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1, cols2 = n1 // world, n2 // world
    a, b = work if work is not None else (be.alloc(KIND_FR_MONT, rows1 * n2), be.alloc(KIND_FR_MONT, rows1 * n2))
    be.ntt(xt, l2, batch=rows1, inverse=True, out=a)             # [k1 local][i2]
    recv = yield be.transpose(a, rows1, n2, out=b)               # [i2][k1 local]: chunk h = rows i2 of rank h
    be.swap_outer(recv, world, cols2, rows1, out=a)              # [i2 local][k1]
    be.ntt_twiddle(a, log2n, rank * cols2, cols2, n1, inverse=True)
    be.ntt(a, l1, batch=cols2, inverse=True, out=b)              # [i2 local][i1]
    recv = yield be.transpose(b, cols2, n1, out=a)               # [i1][i2 local]: chunk h = rows i1 of rank h
    be.swap_outer(recv, world, rows1, cols2, out=b)              # [i1 local][i2]
    if work is None:
        be.synchronize()
        a.free()
    return b


def run_emulated(backends, inputs, log2n, direction=forward, works=None):
    """All ranks in one process: backends[g] / inputs[g] (/ works[g]) per rank; the exchange goes through the host."""
    import numpy as np

    world = len(backends)
    gens = [direction(backends[g], inputs[g], log2n, g, world, work=None if works is None else works[g]) for g in range(world)]
    sends = [next(gen) for gen in gens]
    while True:
        host = [s.download().reshape(world, -1, 32) for s in sends]
        recvs = []
        for g in range(world):
            chunks = np.concatenate([host[h][g] for h in range(world)], axis=0)
            recvs.append(backends[g].upload(chunks, sends[g].kind))
        results, sends = [], []
        for g in range(world):
            try:
                sends.append(gens[g].send(recvs[g]))
            except StopIteration as done:
                results.append(done.value)
        for g in range(world):
            backends[g].synchronize()
            recvs[g].free()
        if results:
            if len(results) != world:
                raise RuntimeError("ranks finished at different exchange steps")
            return results


class NcclExchange:
    """The all-to-all of one rank under torch.distributed (NCCL), queued on the context's own
    stream: chunks land in a persistent tensor of this GPU's memory, which the next kernels read
    through a wrapped Buffer.  Nothing here waits on the host."""

    def __init__(self, be, count, device):
        import torch

        self.be, self.count = be, count
        self.device = torch.device("cuda", device)
        self.stream = torch.cuda.ExternalStream(be.stream, device=self.device)
        self.dst = torch.empty((count, 32), dtype=torch.uint8, device=self.device)
        self.recv = be.wrap(KIND_FR_MONT, count, self.dst.data_ptr())

    def run(self, gen):
        import torch
        import torch.distributed as dist

        try:
            send = next(gen)
            while True:
                with torch.cuda.stream(self.stream):
                    dist.all_to_all_single(self.dst, _as_tensor(send, self.count, self.device))
                self.recv.retag(send.kind)
                send = gen.send(self.recv)
        except StopIteration as done:
            return done.value

    def close(self):
        self.be.synchronize()
        self.recv.free()
        self.dst = None


def _as_tensor(buf, count, device):
    import torch

    class _Iface:
        pass

    holder = _Iface()
    holder.__cuda_array_interface__ = {"shape": (count, 32), "typestr": "|u1", "data": (buf.device_ptr, False), "version": 2}
    return torch.as_tensor(holder, device=device)


__all__ = ["forward", "inverse", "run_emulated", "NcclExchange", "split"]

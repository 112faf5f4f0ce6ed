"""Row-sharded transform over several GPUs: the host-side sequence around the library's kernels.

A vector of n = 2^log2n field elements is split by contiguous rows: with n = n1*n2 and element
i = i1*n2 + i2, rank g of `world` holds rows i1 in [g*n1/world, (g+1)*n1/world).  The forward
transform leaves rank g with X[k1 + n1*k2] for k1 in its block, stored as [k1][k2] ("transposed
out"); the inverse takes that layout back to contiguous rows.  Pointwise work between the two
needs no exchange.

Both directions are generators: they yield a Buffer whose `world` equal chunks go to ranks
0..world-1 and expect to be sent the Buffer of chunks received from ranks 0..world-1 (an
all-to-all).  `run_nccl` drives one rank with torch.distributed; `run_emulated` drives all ranks
of a single process in lockstep (tests on one GPU)."""

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


def forward(be, x, log2n, rank, world):
    """x: this rank's rows [n1/world][n2] (FR or FR_MONT).  Returns [n1/world][n2] FR_MONT = X[k1 + n1*k2].
    Intermediate buffers, the yielded ones and the received ones are freed here."""
    l1, l2 = split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1, cols2 = n1 // world, n2 // world
    send = be.swap_outer(x, rows1, world, cols2)                 # [dest][i1 local][i2 local]
    recv = yield send                                            # [src][i1 local][i2 local] = [i1][i2 local]
    send.free()
    t = be.transpose(recv, n1, cols2)                            # [i2 local][i1]
    recv.free()
    y = be.ntt(t, l1, batch=cols2)                               # [i2 local][k1]
    t.free()
    be.ntt_twiddle(y, log2n, rank * cols2, cols2, n1)            # * omega_n^(i2*k1)
    send = be.swap_outer(y, cols2, world, rows1)                 # [dest][i2 local][k1 local]
    y.free()
    recv = yield send                                            # [i2][k1 local]
    send.free()
    t = be.transpose(recv, n2, rows1)                            # [k1 local][i2]
    recv.free()
    out = be.ntt(t, l2, batch=rows1)                             # [k1 local][k2]
    t.free()
    return out


def inverse(be, xt, log2n, rank, world):
    """xt: [n1/world][n2] as left by `forward`.  Returns this rank's contiguous rows, FR_MONT."""
    l1, l2 = split(log2n, world)
    n1, n2 = 1 << l1, 1 << l2
    rows1, cols2 = n1 // world, n2 // world
    t = be.ntt(xt, l2, batch=rows1, inverse=True)                # [k1 local][i2]
    send = be.transpose(t, rows1, n2)                            # [i2][k1 local]: chunk h = rows i2 of rank h
    t.free()
    recv = yield send                                            # [src][i2 local][k1 local of src]
    send.free()
    y = be.swap_outer(recv, world, cols2, rows1)                 # [i2 local][k1]
    recv.free()
    be.ntt_twiddle(y, log2n, rank * cols2, cols2, n1, inverse=True)
    t = be.ntt(y, l1, batch=cols2, inverse=True)                 # [i2 local][i1]
    y.free()
    send = be.transpose(t, cols2, n1)                            # [i1][i2 local]: chunk h = rows i1 of rank h
    t.free()
    recv = yield send                                            # [src][i1 local][i2 local of src]
    send.free()
    out = be.swap_outer(recv, world, rows1, cols2)               # [i1 local][i2]
    recv.free()
    return out


def run_emulated(backends, inputs, log2n, direction=forward):
    """All ranks in one process: backends[g] / inputs[g] per rank; the exchange goes through the host."""
    import numpy as np

    world = len(backends)
    gens = [direction(backends[g], inputs[g], log2n, g, world) for g in range(world)]
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
        if results:
            if len(results) != world:
                raise RuntimeError("ranks finished at different exchange steps")
            return results


def run_nccl(be, gen, count, device):
    """One rank under torch.distributed (NCCL): every yielded Buffer is exchanged with
    all_to_all_single into a tensor of this GPU's own memory, which the next kernels read."""
    import torch
    import torch.distributed as dist

    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", device))
    keep = []
    try:
        send = next(gen)
        while True:
            be.synchronize()
            with torch.cuda.stream(stream):
                src = _as_tensor(send, count, device)
                dst = torch.empty_like(src)
                dist.all_to_all_single(dst, src)
            stream.synchronize()
            keep = [dst]  # the tensor backs the wrapped Buffer until the generator has consumed it
            send = gen.send(be.wrap(send.kind, count, dst.data_ptr()))
    except StopIteration as done:
        be.synchronize()
        del keep
        return done.value


def _as_tensor(buf, count, device):
    import torch

    class _Iface:
        pass

    holder = _Iface()
    holder.__cuda_array_interface__ = {"shape": (count, 32), "typestr": "|u1", "data": (buf.device_ptr, False), "version": 2}
    return torch.as_tensor(holder, device=torch.device("cuda", device))


__all__ = ["forward", "inverse", "run_emulated", "run_nccl", "split"]

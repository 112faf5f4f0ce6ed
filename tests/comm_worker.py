"""One rank of the 2-GPU exchange test (run by tests/test_gpu_comm.py as a child process per GPU)."""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main(rank, world, workdir):
    import oracle_lib as ora
    from project_b200 import KIND_FR, KIND_FR_MONT, Backend, shard_rows
    from project_b200.lib import Comm

    be = Backend(rank)
    id_path = os.path.join(workdir, "nccl_id.bin")
    if rank == 0:
        uid = Comm.unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid.tobytes())
        os.replace(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 60
        while not os.path.exists(id_path):
            if time.time() > deadline:
                raise RuntimeError("rank 0 never published the communicator id")
            time.sleep(0.05)
        uid = np.frombuffer(open(id_path, "rb").read(), dtype=np.uint8)
    comm = Comm(be, world, rank, uid)
    comm.set_timeout(20.0)
    rng = np.random.default_rng(77)  # the same stream on every rank: each rank can compute what the others hold

    def rand_fr(n):
        a = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
        a[:, 31] &= 0x3F
        return a

    # 1. sum of per-rank vectors on the device
    parts = [rand_fr(37) for _ in range(world)]
    mine = be.upload(parts[rank], KIND_FR)
    total = be.alloc(KIND_FR, 37)
    comm.allgather_fr_sum(mine, 37, total)
    comm.wait()
    want = parts[0]
    for p in parts[1:]:
        want = ora.fr_binop(0, want, p)
    assert np.array_equal(total.download(), want), "allgather_fr_sum"

    # 2. row-sharded packed evaluation: partial sums stay on the device, are summed over the ranks there
    log2n, k = 12, 5
    n = 1 << log2n
    cols = rand_fr(k * n).reshape(k, n, 32)
    x = np.zeros(32, dtype=np.uint8)
    x[:8] = np.frombuffer((0x1234567887654321).to_bytes(8, "little"), dtype=np.uint8)
    begin, end = shard_rows(n, world, rank, align=32)
    rows = end - begin
    w_first, w_count = (begin - 1) % n, rows + 1
    weights = be.bary_weights_range(log2n, x, w_first, w_count)
    local = [be.upload(cols[i, begin:end], KIND_FR) for i in range(k)]
    partial = be.alloc(KIND_FR_MONT, 2 * k)
    be.eval_batch_range_device(local, rows, begin, log2n, weights, w_first, (0, 1), partial)
    summed = be.alloc(KIND_FR_MONT, 2 * k)
    comm.allgather_fr_sum(partial, 2 * k, summed)
    comm.wait()
    want = ora.eval_rotations(cols, ora.bary_weights(x, n), (0, 1))
    assert np.array_equal(summed.download().reshape(2, k, 32), want), "sharded evaluation"

    # 3. all-to-all: chunk g of rank r is filled with the value 100 * r + g
    chunk = 8
    send = np.zeros((world * chunk, 32), dtype=np.uint8)
    for g in range(world):
        send[g * chunk:(g + 1) * chunk, 0] = 100 * rank + g
    recv = be.alloc(KIND_FR, world * chunk)
    comm.alltoall(be.upload(send, KIND_FR), chunk, recv)
    comm.wait()
    got = recv.download()
    for h in range(world):
        assert np.all(got[h * chunk:(h + 1) * chunk, 0] == 100 * h + rank), "alltoall"

    # 4. the row-sharded transform against the transform of the whole vector
    log2n = 12
    n = 1 << log2n
    vec = rand_fr(n)
    l1 = log2n // 2
    n1, n2 = 1 << l1, 1 << (log2n - l1)
    rows1 = n1 // world
    mine = be.upload(vec.reshape(n1, n2, 32)[rank * rows1:(rank + 1) * rows1].reshape(-1, 32), KIND_FR)
    work, out = be.alloc(KIND_FR, rows1 * n2), be.alloc(KIND_FR_MONT, rows1 * n2)
    comm.ntt_sharded(mine, log2n, work, out)
    comm.wait()
    whole = ora.ntt(vec).reshape(n2, n1, 32)  # X[k1 + n1 * k2] at [k2][k1]
    want = np.transpose(whole, (1, 0, 2))[rank * rows1:(rank + 1) * rows1].reshape(-1, 32)
    assert np.array_equal(out.download(), want), "sharded transform"

    comm.close()
    be.close()
    with open(os.path.join(workdir, f"rank{rank}.ok"), "w") as f:
        f.write("ok")


if __name__ == "__main__":
    main(int(sys.argv[1]), int(sys.argv[2]), sys.argv[3])

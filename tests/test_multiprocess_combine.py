"""World-size-2 gloo test of the host side of the multi-GPU path: row sharding,
all-gather of the partial sums, and the library's host combine (gzk_fr_sum /
gzk_g1_sum).  The per-shard partial sums come from the CPU oracle here (no GPU in
this test); on a GPU box the same flow runs with gzk_eval_batch_range."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import oracle_lib as ora
    from project_b200 import fr_sum, g1_sum, shard_rows
    from pyref import fr_array
    import pyref

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(123)  # same data on every rank
    n, k, length = 256, 4, 230
    cols = rng.integers(0, 256, size=(k, n, 32), dtype=np.uint8)
    cols[:, :, 31] &= 0x3F
    cols[:, length:] = 0
    w = ora.bary_weights(fr_array([987654321]), n)
    begin, end = shard_rows(length, world, rank, align=32)
    local = np.zeros_like(cols)
    local[:, begin:end] = cols[:, begin:end]  # this rank's rows only
    partial = ora.eval_rotations(local, w, (0, 1))
    gathered = [torch.zeros(partial.shape, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(partial))
    total = fr_sum(np.stack([g.numpy() for g in gathered]))
    want = ora.eval_rotations(cols, w, (0, 1))
    ok = np.array_equal(total, want)

    G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()
    ks = [3 + rank, 1000 * (rank + 1)]
    mine = ora.g1_mul_same_base(G, fr_array([sum(ks)]))[0]
    pts = [torch.zeros(96, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(pts, torch.from_numpy(mine.copy()))
    combined = g1_sum(np.stack([p.numpy() for p in pts]))
    expect = ora.g1_mul_same_base(G, fr_array([sum(3 + r + 1000 * (r + 1) for r in range(world))]))[0]
    ok = ok and np.array_equal(combined, expect)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_rank_gloo_combine(tmp_path):
    import torch.multiprocessing as mp

    import __graft_entry__ as entry

    entry.build()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"

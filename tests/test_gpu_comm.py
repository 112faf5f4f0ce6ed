"""Exchange between GPUs behind the C ABI (gzk_comm_*): device-side sum of gathered partial sums, the
row-sharded packed evaluation, all-to-all and the row-sharded transform, on two GPUs with one child
process per GPU.  Skipped on a box with a single GPU (the host-side logic of the sharding is covered
by the two-rank CPU tests, tests/test_multiprocess_*.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_two_ranks_exchange_through_the_c_abi(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(here, "comm_worker.py"), str(rank), "2", str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outputs.append(out)
    for rank, p in enumerate(procs):
        assert p.returncode == 0 and os.path.exists(tmp_path / f"rank{rank}.ok"), f"rank {rank}:\n{outputs[rank][-3000:]}"

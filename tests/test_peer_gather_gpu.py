"""Two or more GPUs: the column-sharded linear whose all-gather is the kernel's own peer
stores (iex_linear_f16_splitk_gather + iex_peer_barrier) against the CPU oracle."""
import os
import subprocess
import sys

import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_peer_gather_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs of one box")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(REPO, "tests", "peer_gather_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PEER_GATHER_OK" in res.stdout

"""Two GPUs: the column-sharded ReLU-sparse FFN down projection with both gather methods
against torch.sparse.mm on CPU (skipped on a one-GPU box; bench.py repeats the comparison
at every GPU count and reports it)."""
import os
import subprocess
import sys

import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_ffn_sharded_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs of one box")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29541",
           os.path.join(REPO, "tests", "ffn_sharded_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "FFN_SHARDED_OK" in res.stdout

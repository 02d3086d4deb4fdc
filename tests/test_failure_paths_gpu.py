"""GPU: failure paths that can be exercised without faulting or hanging the device.

* A bounded device-side wait that runs out: the cross-GPU barrier kernel is given, on ONE
  GPU, a "peer" whose signal word nobody writes and a limit of a thousand polls (about
  0.1 ms).  The kernel must return, leave IEX_ERR_TIMEOUT in the status word, and the next
  normal launch must work.
* The CSR validator: malformed matrices are reported, and with IEX_VALIDATE_CSR=1 the
  operators refuse them before any gather kernel reads through a bad index.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from intrasm_engine_b200 import _lib, synthetic as syn
from . import gpu_util as G

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_barrier_wait_runs_out_and_context_survives():
    torch.cuda.synchronize()
    assert _lib.lib.iex_last_device_status(1) == 0
    # world = 2 on one GPU: rank 0's array and a stand-in for rank 1's, both local, zeroed.
    # Rank 0 publishes its epoch into both and waits for word 1 of its own array, which only
    # a rank 1 would write.
    mine = torch.zeros(3, dtype=torch.int32, device=G.DEV)
    absent_peer = torch.zeros(3, dtype=torch.int32, device=G.DEV)
    sig = (ctypes.c_void_p * 2)(mine.data_ptr(), absent_peer.data_ptr())
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.call("iex_peer_barrier_bounded", sig, 2, 0, 1000, G.stream_ptr())
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 100.0  # ms: the wait gave up, it did not spin for long
    assert _lib.lib.iex_last_device_status(1) == -5  # IEX_ERR_TIMEOUT, then cleared
    assert _lib.lib.iex_last_device_status(0) == 0
    assert int(mine[2]) == 1 and int(absent_peer[0]) == 1 and int(mine[1]) == 0
    # world = 1 needs nobody else: completes, status stays clean
    solo = torch.zeros(2, dtype=torch.int32, device=G.DEV)
    sig1 = (ctypes.c_void_p * 1)(solo.data_ptr())
    _lib.call("iex_peer_barrier_bounded", sig1, 1, 0, 1000, G.stream_ptr())
    # and an ordinary kernel of the library still runs in this context
    x = torch.randn(64, 256, device=G.DEV).half()
    w = (torch.randn(128, 256, device=G.DEV) * 0.05).half()
    out = torch.empty(64, 128, dtype=torch.float16, device=G.DEV)
    _lib.call("iex_linear_f16", 64, 256, 128, x.data_ptr(), w.data_ptr(), out.data_ptr(), G.stream_ptr())
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), x.float() @ w.float().t(), rtol=2e-3, atol=2e-3)
    assert _lib.lib.iex_last_device_status(1) == 0


def _validate(a, k, ascending=True, row_indices=True):
    res = torch.full((1,), -1, dtype=torch.int32, device=G.DEV)
    bits = 16 if a.column_indices.dtype == torch.int16 else 32
    _lib.call("iex_csr_validate", a.m, k, a.nnz, a.row_offsets.data_ptr(), G.ptr(a.column_indices), bits,
              a.row_indices.data_ptr() if row_indices else None, int(ascending), res.data_ptr(), G.stream_ptr())
    return int(res.item())


@pytest.mark.parametrize("idx", [np.int16, np.int32])
def test_csr_validate_reports_each_rule(idx):
    rng = np.random.default_rng(5)
    a = syn.csr_from_mask(rng.random((300, 520)) < 0.2, rng=rng, dtype=np.float16, index_dtype=idx)
    assert _validate(G.DevCSR(a), 520) == 0
    empty = syn.csr_from_mask(np.zeros((7, 16), bool), rng=rng, dtype=np.float16, index_dtype=idx)
    assert _validate(G.DevCSR(empty), 16) == 0
    # two columns of one row swapped: still in range, no longer ascending
    d = G.DevCSR(a)
    p = int(a.row_offsets[5])
    d.column_indices[p], d.column_indices[p + 1] = d.column_indices[p + 1].clone(), d.column_indices[p].clone()
    assert _validate(d, 520) == 16
    assert _validate(d, 520, ascending=False) == 0
    # a repeated column is not strictly ascending either
    d = G.DevCSR(a)
    d.column_indices[p + 1] = d.column_indices[p]
    assert _validate(d, 520) == 16
    # a column past the matrix
    d = G.DevCSR(a)
    d.column_indices[a.nnz - 1] = 520
    assert _validate(d, 520) & 8
    # broken offsets
    d = G.DevCSR(a)
    d.row_offsets[0] = 1
    assert _validate(d, 520) & 1
    d = G.DevCSR(a)
    d.row_offsets[300] = a.nnz - 1
    assert _validate(d, 520) & 2
    d = G.DevCSR(a)
    d.row_offsets[10] = d.row_offsets[11] + 3
    assert _validate(d, 520) & 4
    d = G.DevCSR(a)
    d.row_indices[0] = 300
    assert _validate(d, 520) & 32
    assert _validate(d, 520, row_indices=False) == 0


def test_operators_refuse_unsorted_columns_when_validation_is_on():
    """IEX_VALIDATE_CSR is read once per process, so the check runs in a child process."""
    code = r"""
import numpy as np, torch, sys
sys.path.insert(0, %r)
import intrasm_engine_b200
from intrasm_engine_b200 import synthetic as syn
rng = np.random.default_rng(1)
a = syn.csr_from_mask(rng.random((128, 256)) < 0.3, rng=rng, dtype=np.float16, index_dtype=np.int16)
t = lambda z: torch.as_tensor(np.ascontiguousarray(z)).cuda()
ro, va, ci = t(a.row_offsets), t(a.values), t(a.column_indices)
x = t(rng.standard_normal((256, 64)).astype(np.float16))
ops = torch.ops.iex_ops
ops.spmm_tc_half(x, ro, va, ci, 128)                      # well formed: accepted
assert ops.validate_csr(ro, ci, 128, 256, True) == 0
p = int(a.row_offsets[3])
ci[p], ci[p + 1] = ci[p + 1].clone(), ci[p].clone()
assert ops.validate_csr(ro, ci, 128, 256, True) == 16
try:
    ops.spmm_tc_half(x, ro, va, ci, 128)
except RuntimeError as e:
    assert "malformed CSR" in str(e), e
    print("REFUSED")
""" % REPO
    env = dict(os.environ, IEX_VALIDATE_CSR="1")
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "REFUSED" in res.stdout

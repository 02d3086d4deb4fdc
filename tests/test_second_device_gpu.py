"""GPU: one process driving two GPUs.  The opt-in shared-memory size of a kernel and the SM count
belong to a device, so the library remembers them per device; a launch on cuda:1 after cuda:0
must configure the kernels there as well.  Skipped on a one-GPU box."""
import numpy as np
import pytest
import torch

from intrasm_engine_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def test_tensor_core_ops_on_a_second_device_after_the_first(oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ops = torch.ops.iex_ops
    rng = np.random.default_rng(2)
    m, k, n, md = 300, 1024, 64, 384
    a = syn.csr_from_mask(rng.random((m, k)) < 0.3, rng=rng, std=0.05, dtype=np.float16, index_dtype=np.int16)
    x = rng.standard_normal((k, n)).astype(np.float16)
    w = (rng.standard_normal((md, k)) * 0.05).astype(np.float16)
    mask, q, kk, _ = syn.sddmm_chain_case(1, 256, 4096, 64, 0.05)
    results = []
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        t = lambda z: torch.as_tensor(np.ascontiguousarray(z)).to(dev)
        ro, va, ci, dx, dw = t(a.row_offsets), t(a.values), t(a.column_indices), t(x), t(w)
        sp = ops.spmm_tc_half(dx, ro, va, ci, m)
        lin = ops.linear_fp16(dx.t().contiguous(), dw)
        fs, fd = ops.fused_spmm_linear_half(dx, ro, va, ci, m, dw)
        mro, mci = t(mask.row_offsets), t(mask.column_indices)
        plan = ops.sddmm_plan(mro, mci, 256, 4096)
        sd = ops.sddmm_tc_planned(t(q), t(kk), plan, mask.nnz)
        torch.cuda.synchronize(dev)
        results.append([z.cpu() for z in (sp, lin, fs, fd, sd)])
    for other in results[1:]:
        for r0, r1 in zip(results[0], other):
            assert torch.equal(r0, r1)  # same kernels, same order of operations on every device
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, x, m)[0]
    assert np.allclose(results[1][0].float().numpy(), ref, rtol=2e-3, atol=2e-3 * np.abs(ref).max())

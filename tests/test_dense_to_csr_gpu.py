"""GPU: dense -> CSR conversion kernels (iex_dense_to_csr_count / _fill) against the CPU
oracle, bit for bit (indices, order and values)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(m, k, density, dtype, seed, ties=False):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(dtype)
    a[rng.random((m, k)) >= density] = 0
    if ties and m >= 4:
        a[m // 2] = a[0]          # equal row lengths: order must follow the row number
        a[m - 1] = 0              # an empty row
    return a


@pytest.mark.parametrize("m,k,density", [(1, 1, 1.0), (7, 33, 0.5), (256, 11008, 0.1), (1031, 517, 0.03),
                                         (4096, 4096, 0.05), (3, 70000, 0.01)])
@pytest.mark.parametrize("dtype,idx", [(np.float16, torch.int16), (np.float16, torch.int32),
                                       (np.float32, torch.int32)])
@pytest.mark.parametrize("relu", [False, True])
def test_dense_to_csr_matches_oracle(m, k, density, dtype, idx, relu):
    from intrasm_engine_b200.pytorch.utils import dense_to_sparse_cuda
    from oracle import oracle
    if idx == torch.int16 and k > 65536:
        pytest.skip("16-bit indices cannot address this many columns")
    a = _case(m, k, density, dtype, seed=m * 31 + k, ties=True)
    d = torch.as_tensor(a).cuda()
    values, row_indices, row_offsets, cols = dense_to_sparse_cuda(d, index_dtype=idx, relu=relu)
    ev, eri, ero, eci = oracle.dense_to_csr(a, relu=relu)
    assert np.array_equal(row_offsets.cpu().numpy(), ero)
    assert np.array_equal(row_indices.cpu().numpy(), eri)
    got_cols = cols.cpu().numpy()
    if idx == torch.int16:
        got_cols = got_cols.view(np.uint16)
    assert np.array_equal(got_cols.astype(np.int64), eci.astype(np.int64))
    assert np.array_equal(values.cpu().numpy().view(np.uint16 if dtype == np.float16 else np.uint32),
                          ev.view(np.uint16 if dtype == np.float16 else np.uint32))


def test_dense_to_csr_empty_and_errors():
    from intrasm_engine_b200 import _lib
    from intrasm_engine_b200.pytorch.utils import dense_to_sparse_cuda
    z = torch.zeros((5, 16), dtype=torch.float16, device="cuda")
    values, row_indices, row_offsets, cols = dense_to_sparse_cuda(z)
    assert values.numel() == 0 and cols.numel() == 0
    assert row_offsets.cpu().tolist() == [0] * 6
    assert row_indices.cpu().tolist() == [0, 1, 2, 3, 4]
    with pytest.raises(RuntimeError):
        dense_to_sparse_cuda(torch.zeros((2, 2), dtype=torch.float64, device="cuda"))
    ro = torch.empty(3, dtype=torch.int32, device="cuda")
    assert _lib.lib.iex_dense_to_csr_count(2, 2, z.data_ptr(), 8, 0, ro.data_ptr(), ro.data_ptr(), None) == -1


def test_relu_csr_feeds_the_spmm():
    """relu(act) as CSR times a dense weight: the kernels' CSR drives the CUDA-core SpMM to the
    same bits as the oracle's CSR does."""
    from intrasm_engine_b200.pytorch.utils import dense_to_sparse_cuda
    from oracle import oracle
    rng = np.random.default_rng(5)
    act = rng.standard_normal((64, 512)).astype(np.float32)
    w = rng.standard_normal((512, 96)).astype(np.float32)
    values, row_indices, row_offsets, cols = dense_to_sparse_cuda(torch.as_tensor(act).cuda(), relu=True)
    out = torch.ops.iex_ops.spmm_sputnik_reuse_weight(torch.as_tensor(w).cuda()[None], row_indices, values,
                                                      row_offsets, cols, 64)
    ev, eri, ero, eci = oracle.dense_to_csr(act, relu=True)
    ref = oracle.spmm(eri, ev, ero, eci, w[None], 64)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), np.asarray(ref, dtype=np.float32).view(np.uint32))

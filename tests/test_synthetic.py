"""CPU: the seeded workload generators produce valid CSR with the stated statistics."""
import numpy as np

from intrasm_engine_b200 import synthetic as syn


def _valid(oracle, a):
    m, k = a.shape
    assert oracle.validate_csr(m, k, a.row_indices, a.row_offsets, a.column_indices.astype(np.int32)) == 0
    nnz_rows = np.diff(a.row_offsets)
    assert np.all(np.diff(nnz_rows[a.row_indices]) <= 0), "row_indices must be by decreasing nnz"
    for r in range(0, m, max(1, m // 16)):
        seg = a.column_indices[a.row_offsets[r]:a.row_offsets[r + 1]]
        assert np.all(np.diff(seg.astype(np.int64)) > 0)


def test_spmm_fp32_case(oracle):
    a, b = syn.spmm_fp32_case(0, 256, 256, 64, 0.1)
    _valid(oracle, a)
    assert a.values.dtype == np.float32 and b.shape == (256, 64)
    assert abs(a.nnz / (256 * 256) - 0.1) < 0.01
    a2, b2 = syn.spmm_fp32_case(0, 256, 256, 64, 0.1)
    np.testing.assert_array_equal(a.values, a2.values)
    np.testing.assert_array_equal(b, b2)


def test_sddmm_chain_case(oracle):
    mask, q, k, v = syn.sddmm_chain_case(1, 128, 192, 32, 0.05)
    _valid(oracle, mask)
    assert q.shape == (128, 32) and k.shape == (192, 32) and v.shape == (192, 32)


def test_pruned_sweep_case(oracle):
    a, b = syn.pruned_sweep_case(2, 512, 512, 0.9, 128)
    _valid(oracle, a)
    nnz_rows = np.diff(a.row_offsets)
    assert np.all(nnz_rows % 2 == 0)
    assert abs(nnz_rows.mean() - 51.2) < 4
    assert 0.2 < nnz_rows.std() / nnz_rows.mean() < 0.4
    assert a.values.dtype == np.float16 and a.column_indices.dtype == np.int16


def test_fused_layer_case_small(oracle):
    a, w, x = syn.fused_layer_case(3, m_sparse=96, k=128, tokens=16, m_dense=64)
    _valid(oracle, a)
    assert abs(a.nnz / (96 * 128) - 0.5) < 0.02
    assert w.shape == (64, 128) and x.shape == (128, 16)
    kept = np.abs(a.values.astype(np.float32)).min()
    dense = a.to_dense().astype(np.float32)
    assert kept > 0 and np.count_nonzero(dense) == a.nnz


def test_relu_ffn_case(oracle):
    a, w = syn.relu_ffn_layer_case(4, layer=2, tokens=32, k=256, n=64)
    _valid(oracle, a)
    assert np.all(a.values > 0) and w.shape == (256, 64)
    a2, _ = syn.relu_ffn_layer_case(4, layer=3, tokens=32, k=256, n=64, with_weight=False)
    assert a2.nnz != a.nnz or not np.array_equal(a2.column_indices, a.column_indices)


def test_dense_to_csr_roundtrip():
    rng = np.random.default_rng(0)
    d = rng.standard_normal((20, 30)).astype(np.float32) * (rng.random((20, 30)) < 0.3)
    a = syn.dense_to_csr(d)
    np.testing.assert_array_equal(a.to_dense(), d)


def test_traffic_formulas():
    assert syn.spmm_bytes(1024, 1024, 256, 104858, 4, 4) == 104858 * 8 + 4 * 1025 + 4 * 1024 + 1024 * 256 * 4 * 2
    assert syn.sddmm_flops(10, 64) == 1280

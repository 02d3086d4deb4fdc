"""GPU parity: CSR SpMM through the C ABI against the CPU oracle and the golden vectors.

Tolerances: the CUDA-core kernels add each output's terms in storage order with fused
multiply-adds, exactly like the oracle, so fp32 and fp16 results must be BIT-EXACT against
it; against the torch CPU golden vectors (different summation order) fp32 must agree to
1e-5 relative (plus 1e-5 of the tensor's max magnitude for cancelled sums), fp16 to 1e-2.
"""
import glob
import os

import numpy as np
import pytest
import torch

from intrasm_engine_b200 import _lib, synthetic as syn
from . import gpu_util as G

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "spmm_*.npz")))


def _csr_from_golden(g):
    return syn.CSR(g["values"], g["row_indices"], g["row_offsets"], g["column_indices"],
                   (int(g["m"]), int(g["k"])))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_spmm_golden(oracle, path):
    g = np.load(path)
    a = _csr_from_golden(g)
    da = G.DevCSR(a)
    dense = G.dev(g["dense"])[None]
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, g["dense"], a.shape[0])[0]
    if a.values.dtype == np.float32:
        got = G.spmm_f32(da, dense)[0].cpu().numpy()
        np.testing.assert_array_equal(got, ref)
        assert G.close(got, g["out"], 1e-5, 1e-5)
    else:
        got = G.spmm_f16(da, dense)[0].cpu().numpy()
        np.testing.assert_array_equal(got, ref.astype(np.float16))
        assert G.close(got, g["out"], 1e-2, 1e-2)
        da.column_indices = da.column_indices.to(torch.int16)
        got16 = G.spmm_f16(da, dense)[0].cpu().numpy()
        np.testing.assert_array_equal(got16, got)


SHAPES = [  # m, k, n, density
    (1, 1, 1, 1.0), (5, 3, 2, 0.7), (37, 50, 7, 0.3), (64, 64, 4, 0.2), (64, 80, 8, 0.2),
    (100, 96, 20, 0.15), (130, 128, 36, 0.1), (257, 300, 64, 0.1), (128, 128, 128, 0.1),
    (96, 512, 132, 0.05), (64, 256, 256, 0.2), (40, 200, 260, 0.2), (32, 128, 512, 0.1),
    (33, 1000, 1024, 0.02), (50, 64, 96, 0.0),
]


@pytest.mark.parametrize("m,k,n,density", SHAPES)
def test_spmm_f32_shapes(oracle, m, k, n, density):
    a, b = syn.spmm_fp32_case(m * 1000 + n, m, k, n, density)
    got = G.spmm_f32(G.DevCSR(a), G.dev(b)[None])[0].cpu().numpy()
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, m)[0]
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("m,k,n,density", SHAPES)
@pytest.mark.parametrize("idx", [np.int16, np.int32])
def test_spmm_f16_shapes(oracle, m, k, n, density, idx):
    rng = np.random.default_rng(m * 77 + n)
    a = syn.csr_from_mask(rng.random((m, k)) < density, rng=rng, std=0.5, dtype=np.float16,
                          index_dtype=idx)
    b = rng.standard_normal((k, n)).astype(np.float16)
    got = G.spmm_f16(G.DevCSR(a), G.dev(b)[None])[0].cpu().numpy()
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, m)[0]
    np.testing.assert_array_equal(got, ref.astype(np.float16))


def test_spmm_empty_inputs():
    a, b = syn.spmm_fp32_case(0, 8, 8, 4, 0.5)
    da = G.DevCSR(a)
    # n == 0 and batch == 0 and m == 0 are accepted and launch nothing
    out = torch.full((1, 8, 4), 7.0, device=G.DEV)
    from intrasm_engine_b200 import _lib
    _lib.call("iex_spmm_f32", 0, 8, 4, 0, None, None, 0, None, None, None, None, None, 1, 0, None)
    _lib.call("iex_spmm_f32", 8, 8, 0, da.nnz, G.ptr(da.row_indices), G.ptr(da.values), 0,
              G.ptr(da.row_offsets), G.ptr(da.column_indices), G.ptr(out), None, G.ptr(out), 1, 0, None)
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0
    with pytest.raises(_lib.IexError):
        _lib.call("iex_spmm_f32", 8, 8, 4, da.nnz, None, None, 0, None, None, None, None, None, 1, 0, None)
    with pytest.raises(_lib.IexError):
        _lib.call("iex_spmm_f32", -1, 8, 4, 0, None, None, 0, None, None, None, None, None, 1, 0, None)


def test_spmm_f32_unaligned_pointers(oracle):
    """Bases off a 16-byte boundary select the scalar-load variants; results do not change."""
    a, b = syn.spmm_fp32_case(11, 70, 90, 24, 0.2)
    da = G.DevCSR(a)
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, 70)[0]
    pad_v = torch.zeros(da.nnz + 1, device=G.DEV)
    pad_v[1:] = da.values
    pad_c = torch.zeros(da.nnz + 1, dtype=torch.int32, device=G.DEV)
    pad_c[1:] = da.column_indices
    da.values, da.column_indices = pad_v[1:], pad_c[1:]
    pad_b = torch.zeros(b.size + 1, device=G.DEV)
    pad_b[1:] = G.dev(b).flatten()
    dense = pad_b[1:].view(1, 90, 24)
    got = G.spmm_f32(da, dense)[0].cpu().numpy()
    np.testing.assert_array_equal(got, ref)


def test_spmm_f32_bias_relu_accumulate_batch(oracle):
    a, _ = syn.spmm_fp32_case(5, 96, 128, 64, 0.1)
    rng = np.random.default_rng(5)
    dense = rng.standard_normal((3, 128, 64)).astype(np.float32)
    bias = rng.standard_normal(96).astype(np.float32)
    da = G.DevCSR(a)
    args = (a.row_indices, a.values, a.row_offsets, a.column_indices, dense, 96)
    got = G.spmm_f32(da, G.dev(dense)).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.spmm(*args))
    got = G.spmm_f32(da, G.dev(dense), bias=G.dev(bias)).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.spmm(*args, bias=bias))
    # per-batch values + accumulate onto ones (the "atomic" stamp)
    while a.nnz % 4:
        a, _ = syn.spmm_fp32_case(5 + a.nnz, 96, 128, 64, 0.1)
        da = G.DevCSR(a)
    vals = rng.standard_normal((3, a.nnz)).astype(np.float32)
    start = np.ones((3, 96, 64), np.float32)
    got = G.spmm_f32(da, G.dev(dense), out=G.dev(start), accumulate=True, values=G.dev(vals)).cpu().numpy()
    ref = oracle.spmm(a.row_indices, vals, a.row_offsets, a.column_indices, dense, 96, out=start)
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("seed", range(24))
def test_spmm_random_shapes(oracle, seed):
    """Seeded random shapes for the CUDA-core kernels: ragged rows, every n (odd ones too),
    batches, bias; fp32 and fp16 (both index widths) bit for bit against the oracle."""
    rng = np.random.default_rng(700 + seed)
    m, k = int(rng.integers(1, 500)), int(rng.integers(1, 900))
    n = int(rng.choice([1, 3, 8, 16, 24, 33, 64, 100, 128, 256, 264]))
    batch = int(rng.integers(1, 3))
    row_density = rng.choice([0.0, 0.02, 0.2, 1.0], size=m, p=[0.15, 0.4, 0.35, 0.1])
    mask = rng.random((m, k)) < row_density[:, None]
    a = syn.csr_from_mask(mask, rng=rng)
    dense = rng.standard_normal((batch, k, n)).astype(np.float32)
    bias = rng.standard_normal(m).astype(np.float32) if seed % 2 else None
    got = G.spmm_f32(G.DevCSR(a), G.dev(dense), bias=None if bias is None else G.dev(bias)).cpu().numpy()
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, dense, m, bias=bias)
    np.testing.assert_array_equal(got, ref)
    idx = np.int16 if seed % 3 else np.int32
    ah = syn.csr_from_mask(mask, rng=rng, std=0.05, dtype=np.float16, index_dtype=idx)
    dh = dense.astype(np.float16)
    goth = G.spmm_f16(G.DevCSR(ah), G.dev(dh), bias=None if bias is None else G.dev(bias)).cpu().numpy()
    refh = oracle.spmm(ah.row_indices, ah.values, ah.row_offsets, ah.column_indices, dh, m, bias=bias)
    np.testing.assert_array_equal(goth, refh.astype(np.float16))


def test_spmm_cfg1_full_size(oracle):
    """Benchmark configuration 1: 1024x1024 at 90 % sparsity times 1024x256, fp32."""
    for seed in (0, 1):
        a, b = syn.spmm_fp32_case(seed)
        got = G.spmm_f32(G.DevCSR(a), G.dev(b)[None])[0].cpu().numpy()
        ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, 1024)[0]
        np.testing.assert_array_equal(got, ref)
        tref = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, b, 1024)
        assert G.close(got, tref, 1e-5, 1e-5), G.max_violation(got, tref, 1e-5, 1e-5)


@pytest.mark.parametrize("rows,cols", [(512, 512), (2048, 512), (512, 2048)])
@pytest.mark.parametrize("sparsity", [0.5, 0.7, 0.8, 0.9, 0.95, 0.98])
@pytest.mark.parametrize("n", [128, 256])
@pytest.mark.parametrize("idx", [np.int16, np.int32])
def test_spmm_cfg3_sweep(oracle, rows, cols, sparsity, n, idx):
    """Benchmark configuration 3, the whole sweep (36 cases x 2 index widths): fp16 values,
    fp32 accumulate.  The CUDA-core kernel is bit-exact against the oracle and within 1e-2 of
    the torch CPU path; the tensor-core kernel within fp16 rounding of the oracle
    (gpu_util.tc_close, far inside the 1e-2 bar)."""
    a, b = syn.pruned_sweep_case(int(sparsity * 100) + rows, rows, cols, sparsity, n, index_dtype=idx)
    da = G.DevCSR(a)
    got = G.spmm_f16(da, G.dev(b)[None])[0].cpu().numpy()
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, rows)[0]
    np.testing.assert_array_equal(got, ref.astype(np.float16))
    tref = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, b, rows)
    assert G.close(got, tref, 1e-2, 1e-2)
    tc = torch.empty((rows, n), dtype=torch.float16, device=G.DEV)
    db = G.dev(b)  # kept alive: the call is asynchronous
    _lib.call("iex_spmm_f16_tc", rows, cols, n, a.nnz, da.row_offsets.data_ptr(), da.column_indices.data_ptr(),
              16 if idx == np.int16 else 32, da.values.data_ptr(), db.data_ptr(), tc.data_ptr(),
              G.stream_ptr())
    _ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, b, rows)
    assert G.tc_close(tc.cpu().numpy(), ref, sabs)
    assert _lib.lib.iex_last_device_status(1) == 0


@pytest.mark.parametrize("m,k,n,density", [(4096, 4096, 64, 0.05), (300, 2048, 128, 0.1), (777, 6000, 24, 0.02)])
def test_spmm_f32_large_operand(oracle, m, k, n, density):
    """Dense operands far larger than L1 (the gather-latency-bound regime): bit-exact against
    the oracle, with bias+ReLU and with accumulation."""
    a, b = syn.spmm_fp32_case(m + k, m, k, n, density)
    da = G.DevCSR(a)
    args = (a.row_indices, a.values, a.row_offsets, a.column_indices, b, m)
    got = G.spmm_f32(da, G.dev(b)[None])[0].cpu().numpy()
    np.testing.assert_array_equal(got, oracle.spmm(*args)[0])
    bias = np.linspace(-1, 1, m).astype(np.float32)
    got = G.spmm_f32(da, G.dev(b)[None], bias=G.dev(bias))[0].cpu().numpy()
    np.testing.assert_array_equal(got, oracle.spmm(*args, bias=bias)[0])
    start = np.full((1, m, n), 0.5, np.float32)
    got = G.spmm_f32(da, G.dev(b)[None], out=G.dev(start), accumulate=True).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.spmm(*args, out=start))


def test_spmm_linearity_and_determinism():
    """Size-independent properties at a size the oracle is not run on."""
    a, b = syn.spmm_fp32_case(3, 4096, 4096, 128, 0.02)
    da = G.DevCSR(a)
    d1 = G.dev(b)[None]
    o1 = G.spmm_f32(da, d1)
    o2 = G.spmm_f32(da, d1)
    assert torch.equal(o1, o2)
    o3 = G.spmm_f32(da, 2 * d1)
    assert torch.equal(o3, 2 * o1)  # scaling by a power of two is exact
    ident = syn.dense_to_csr(np.eye(128, dtype=np.float32))
    x = torch.randn(1, 128, 72, device=G.DEV)
    assert torch.equal(G.spmm_f32(G.DevCSR(ident), x), x)


def test_torch_ops_spmm(oracle):
    import intrasm_engine_b200  # noqa: F401
    a, b = syn.spmm_fp32_case(9, 128, 96, 64, 0.1)
    da = G.DevCSR(a)
    out = torch.ops.iex_ops.spmm_sputnik_reuse_weight(G.dev(b)[None], da.row_indices, da.values,
                                                      da.row_offsets, da.column_indices, 128)
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, 128)
    np.testing.assert_array_equal(out.cpu().numpy(), ref)
    with pytest.raises(RuntimeError):
        torch.ops.iex_ops.spmm_sputnik_reuse_weight(G.dev(b), da.row_indices, da.values,
                                                    da.row_offsets, da.column_indices, 128)
    # atomic stamp: per-batch values, output starts from zero
    while a.nnz % 4:
        a, b = syn.spmm_fp32_case(9 + a.nnz, 128, 96, 64, 0.1)
        da = G.DevCSR(a)
    vals = torch.randn(2, a.nnz, device=G.DEV)
    dense = torch.randn(2, 96, 64, device=G.DEV)
    out = torch.ops.iex_ops.spmm_sputnik_atomic(dense, da.row_indices, vals, da.row_offsets,
                                                da.column_indices, 128)
    ref = oracle.spmm(a.row_indices, vals.cpu().numpy(), a.row_offsets, a.column_indices,
                      dense.cpu().numpy(), 128)
    np.testing.assert_array_equal(out.cpu().numpy(), ref)
    # fp16 op (registered here, defined but unregistered in the reference)
    ah, bh = syn.pruned_sweep_case(1, 64, 128, 0.8, 64)
    dh = G.DevCSR(ah)
    out = torch.ops.iex_ops.spmm_sputnik_reuse_weight_half(G.dev(bh)[None], dh.row_indices, dh.values,
                                                           dh.row_offsets, dh.column_indices, 64)
    ref = oracle.spmm(ah.row_indices, ah.values, ah.row_offsets, ah.column_indices, bh, 64)
    np.testing.assert_array_equal(out.cpu().numpy(), ref.astype(np.float16))


# ----------------------------------------------------------------------------------------
# Tensor-core fp32 SpMM (iex_tile_plan_build + iex_spmm_f32_tc): a band of the sparse matrix
# expanded into TF32 head/tail planes, multiplied with the dense rows on tcgen05.  The bar is
# the task's 1e-5 relative, measured against the double-precision product and the sum of the
# terms' magnitudes (the summation order differs from the oracle's); small integers are exact.
# ----------------------------------------------------------------------------------------

def _check_spmm_tc(oracle, a, b):
    got = G.spmm_f32_tc(G.DevCSR(a), G.dev(b)).cpu().numpy()
    torch.cuda.synchronize()
    assert _lib.lib.iex_last_device_status(1) == 0
    dense_a = a.to_dense().astype(np.float64)
    exact = dense_a @ b.astype(np.float64)
    sabs = np.abs(dense_a) @ np.abs(b.astype(np.float64))
    assert got.shape == exact.shape and not np.isnan(got).any()
    assert np.all(np.abs(got - exact) <= 1e-5 * np.abs(exact) + 2e-6 * sabs), \
        float(np.max(np.abs(got - exact) / (1e-5 * np.abs(exact) + 2e-6 * sabs + 1e-300)))
    return got


@pytest.mark.parametrize("m,k,n,density", [
    (128, 64, 64, 0.2), (128, 128, 32, 0.5), (1, 1, 32, 1.0), (130, 257, 64, 0.2), (300, 1000, 64, 0.05),
    (1000, 300, 32, 0.05), (256, 4096, 64, 0.02), (2048, 512, 64, 0.3), (129, 129, 64, 1.0),
    (640, 640, 64, 0.0), (20000, 256, 32, 0.03),
])
def test_spmm_tc_f32_shapes(oracle, m, k, n, density):
    rng = np.random.default_rng(m + 3 * k + 7 * n)
    a = syn.csr_from_mask(rng.random((m, k)) < density, rng=rng)
    b = rng.standard_normal((k, n)).astype(np.float32)
    _check_spmm_tc(oracle, a, b)


@pytest.mark.parametrize("seed", range(16))
def test_spmm_tc_f32_random_shapes(oracle, seed):
    rng = np.random.default_rng(1300 + seed)
    m, k = int(rng.integers(1, 1500)), int(rng.integers(1, 1500))
    n = int(rng.choice([32, 64]))
    row_density = rng.choice([0.0, 0.01, 0.05, 0.3, 1.0], size=m, p=[0.1, 0.2, 0.4, 0.2, 0.1])
    a = syn.csr_from_mask(rng.random((m, k)) < row_density[:, None], rng=rng)
    b = rng.standard_normal((k, n)).astype(np.float32)
    _check_spmm_tc(oracle, a, b)


def test_spmm_tc_f32_exact_on_small_integers_and_repeatable(oracle):
    rng = np.random.default_rng(17)
    m, k, n = 700, 900, 64
    a = syn.csr_from_mask(rng.random((m, k)) < 0.07, rng=rng)
    a.values[:] = rng.integers(-7, 8, size=a.nnz).astype(np.float32)
    b = rng.integers(-7, 8, size=(k, n)).astype(np.float32)
    da, db = G.DevCSR(a), G.dev(b)
    got = G.spmm_f32_tc(da, db)
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, m)[0]
    np.testing.assert_array_equal(got.cpu().numpy(), ref)
    # a second launch reuses stages whose entries were zeroed again: same bits
    assert torch.equal(G.spmm_f32_tc(da, db), got)


def test_spmm_tc_f32_cfg2_full_size(oracle):
    """Benchmark configuration 2's follow-on SpMM (scores CSR 4096x4096 at 5 % times V 4096x64)
    on the tensor-core kernel: against the double-precision product, the CUDA-core kernel and
    the torch operators."""
    mask, q, kk, v = syn.sddmm_chain_case(0)
    rng = np.random.default_rng(5)
    mask.values[:] = rng.standard_normal(mask.nnz).astype(np.float32)
    got = _check_spmm_tc(oracle, mask, v)
    dm = G.DevCSR(mask)
    simt = G.spmm_f32(dm, G.dev(v)[None])[0].cpu().numpy()
    assert G.close(got, simt, 1e-5, 1e-5)
    import intrasm_engine_b200  # noqa: F401
    ops = torch.ops.iex_ops
    plan = ops.spmm_plan(dm.row_offsets, dm.column_indices, 4096, 4096)
    assert torch.equal(ops.spmm_tc_planned(G.dev(v), dm.values, plan, 4096).cpu(), torch.as_tensor(got))
    assert _lib.lib.iex_spmm_f32_prefers_tc(4096, 4096, 64, mask.nnz) == 0      # 5 %: gather kernels win
    assert _lib.lib.iex_spmm_f32_prefers_tc(4096, 4096, 64, 3 * mask.nnz) == 1  # 15 %: dense tiles win
    assert _lib.lib.iex_spmm_f32_tc_supported(4096, 4096, 48) == 0

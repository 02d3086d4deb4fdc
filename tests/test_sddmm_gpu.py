"""GPU parity: SDDMM through the C ABI against the CPU oracle and the golden vectors.

The kernel splits each dot product over the lanes of a sub-warp, so the fp32 summation
order differs from the oracle's: values must agree to 1e-5 relative (plus 1e-5 of the
tensor's max magnitude for cancelled sums) with the double-precision oracle.  The output
ORDER (aligned with column_indices) is exact by construction and checked through the
position-dependent reference.
"""
import glob
import os

import numpy as np
import pytest
import torch

from intrasm_engine_b200 import synthetic as syn
from . import gpu_util as G

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "sddmm_*.npz")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_sddmm_golden(oracle, path):
    g = np.load(path)
    mask = syn.CSR(np.zeros(len(g["column_indices"]), np.float32), g["row_indices"], g["row_offsets"],
                   g["column_indices"], (int(g["m"]), int(g["n"])))
    got = G.sddmm_f32(G.DevCSR(mask), G.dev(g["lhs"])[None], G.dev(g["rhs"])[None]).cpu().numpy()
    assert G.close(got, g["out"], 1e-5, 1e-5)
    exact = oracle.sddmm(g["lhs"], g["rhs"], g["row_indices"], g["row_offsets"], g["column_indices"], f64=True)
    assert G.close(got, exact, 1e-5, 1e-5)


@pytest.mark.parametrize("m,n,k,density,batch", [
    (1, 1, 1, 1.0, 1), (9, 11, 3, 0.5, 1), (64, 64, 8, 0.3, 1), (70, 90, 16, 0.2, 2),
    (128, 128, 32, 0.1, 1), (100, 300, 36, 0.2, 1), (256, 256, 64, 0.05, 3), (60, 500, 100, 0.3, 1),
    (64, 64, 128, 0.5, 1), (48, 80, 260, 0.2, 2), (33, 47, 7, 0.6, 1), (128, 64, 64, 0.0, 1),
    (16, 2000, 64, 0.4, 1),
])
def test_sddmm_shapes(oracle, m, n, k, density, batch):
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    mask = syn.csr_from_mask(rng.random((m, n)) < density, rng=rng)
    lhs = rng.standard_normal((batch, m, k)).astype(np.float32)
    rhs = rng.standard_normal((batch, n, k)).astype(np.float32)
    got = G.sddmm_f32(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    exact = oracle.sddmm(lhs, rhs, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    assert got.shape == exact.shape
    assert G.close(got, exact, 1e-5, 1e-5), G.max_violation(got, exact, 1e-5, 1e-5)


@pytest.mark.parametrize("seed", range(24))
def test_sddmm_random_shapes(oracle, seed):
    """Seeded random shapes: ragged rows (empty to full), every k alignment class, batches."""
    rng = np.random.default_rng(500 + seed)
    m, n = int(rng.integers(1, 400)), int(rng.integers(1, 600))
    k = int(rng.choice([1, 3, 4, 8, 20, 32, 36, 64, 100, 128, 200, 260]))
    batch = int(rng.integers(1, 4))
    row_density = rng.choice([0.0, 0.02, 0.2, 1.0], size=m, p=[0.15, 0.4, 0.35, 0.1])
    mask = syn.csr_from_mask(rng.random((m, n)) < row_density[:, None], rng=rng)
    lhs = rng.standard_normal((batch, m, k)).astype(np.float32)
    rhs = rng.standard_normal((batch, n, k)).astype(np.float32)
    got = G.sddmm_f32(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    exact = oracle.sddmm(lhs, rhs, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    assert got.shape == exact.shape
    assert G.close(got, exact, 1e-5, 1e-5), (m, n, k, batch, G.max_violation(got, exact, 1e-5, 1e-5))


def test_sddmm_accumulate_and_determinism(oracle):
    mask, q, k, _ = syn.sddmm_chain_case(2, 128, 160, 64, 0.1)
    dm = G.DevCSR(mask)
    o1 = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    o2 = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    assert torch.equal(o1, o2)
    start = torch.ones_like(o1)
    o3 = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None], out=start.clone(), accumulate=True)
    assert torch.allclose(o3, o1 + 1, rtol=1e-6, atol=1e-6)


def test_sddmm_cfg2_chain_full_size(oracle):
    """Benchmark configuration 2: SDDMM over a 4096x4096 mask at 95 % sparsity (K=64), then SpMM with V."""
    mask, q, k, v = syn.sddmm_chain_case(0)
    dm = G.DevCSR(mask)
    scores = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    exact = oracle.sddmm(q, k, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    got = scores.cpu().numpy()
    assert G.close(got, exact, 1e-5, 1e-5), G.max_violation(got, exact, 1e-5, 1e-5)
    tref = oracle.torch_sddmm(q, k, mask.row_offsets, mask.column_indices)
    assert G.close(got, tref, 1e-5, 1e-5)
    dm.values = scores
    out = G.spmm_f32(dm, G.dev(v)[None])[0].cpu().numpy()
    ref = oracle.spmm(mask.row_indices, got, mask.row_offsets, mask.column_indices, v, 4096)[0]
    np.testing.assert_array_equal(out, ref)  # SpMM is bit-exact given the same values


def test_torch_ops_sddmm(oracle):
    import intrasm_engine_b200  # noqa: F401
    mask, q, k, _ = syn.sddmm_chain_case(4, 96, 80, 32, 0.2)
    dm = G.DevCSR(mask)
    out = torch.ops.iex_ops.sddmm_sputnik_atomic_upd_weight(G.dev(q)[None], G.dev(k)[None], dm.row_indices,
                                                            dm.row_offsets, dm.column_indices)
    exact = oracle.sddmm(q, k, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    assert G.close(out.cpu().numpy(), exact, 1e-5, 1e-5)
    with pytest.raises(RuntimeError):
        torch.ops.iex_ops.sddmm_sputnik_atomic_upd_weight(G.dev(q)[None], G.dev(k[:, :16])[None],
                                                          dm.row_indices, dm.row_offsets, dm.column_indices)


# ----------------------------------------------------------------------------------------
# Tensor-core SDDMM (iex_sddmm_plan_build + iex_sddmm_f32_tc): dense 128 x 128 tiles in TF32
# head/tail arithmetic, sampled at the stored positions through a plan of the pattern.  Same
# bar as the CUDA-core kernel (1e-5 against the double-precision oracle), plus a bound relative
# to the sum of the terms' magnitudes, the output order through a position-dependent
# reference, exact small-integer cases, and the plan itself against a host-side regrouping.
# ----------------------------------------------------------------------------------------

def _tc_case(rng, m, n, k, row_density):
    mask = syn.csr_from_mask(rng.random((m, n)) < np.asarray(row_density).reshape(-1, 1), rng=rng)
    lhs = rng.standard_normal((m, k)).astype(np.float32)
    rhs = rng.standard_normal((n, k)).astype(np.float32)
    return mask, lhs, rhs


def _check_tc(oracle, mask, lhs, rhs):
    from intrasm_engine_b200 import _lib
    got = G.sddmm_f32_tc(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    torch.cuda.synchronize()
    assert _lib.lib.iex_last_device_status(1) == 0
    exact = oracle.sddmm(lhs[None], rhs[None], mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    sabs = oracle.sddmm(np.abs(lhs)[None], np.abs(rhs)[None], mask.row_indices, mask.row_offsets,
                        mask.column_indices, f64=True)
    assert got.shape == exact.shape
    assert G.close(got, exact, 1e-5, 1e-5), G.max_violation(got, exact, 1e-5, 1e-5)
    assert G.sddmm_close(got, exact, sabs)
    return got


@pytest.mark.parametrize("m,n,k,density", [
    (128, 128, 64, 0.1), (128, 128, 32, 0.5), (1, 1, 32, 1.0), (130, 257, 64, 0.2), (300, 1000, 64, 0.05),
    (1000, 300, 32, 0.05), (256, 4096, 64, 0.02), (2048, 512, 64, 0.3), (129, 129, 64, 1.0),
    (640, 640, 64, 0.0), (20000, 256, 32, 0.03),
])
def test_sddmm_tc_shapes(oracle, m, n, k, density):
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    mask, lhs, rhs = _tc_case(rng, m, n, k, np.full(m, density))
    _check_tc(oracle, mask, lhs, rhs)


@pytest.mark.parametrize("seed", range(24))
def test_sddmm_tc_random_shapes(oracle, seed):
    """Ragged rows in one matrix -- empty, a few entries, completely full (tiles with more
    entries than the epilogue threads keep in registers) -- and sizes that are not multiples
    of the tile."""
    rng = np.random.default_rng(900 + seed)
    m, n = int(rng.integers(1, 1500)), int(rng.integers(1, 1500))
    k = int(rng.choice([32, 64]))
    row_density = rng.choice([0.0, 0.01, 0.05, 0.3, 1.0], size=m, p=[0.1, 0.2, 0.4, 0.2, 0.1])
    mask, lhs, rhs = _tc_case(rng, m, n, k, row_density)
    _check_tc(oracle, mask, lhs, rhs)


@pytest.mark.parametrize("m,n,density", [(300, 500, 0.1), (129, 1000, 0.6), (1, 1, 1.0), (700, 64, 0.02)])
def test_sddmm_plan_regroups_positions_by_tile(m, n, density):
    """The plan against the same regrouping done on the host: per 128 x 128 tile the stored
    positions in storage order, with their row / column inside the tile."""
    from intrasm_engine_b200 import _lib
    rng = np.random.default_rng(m + n)
    mask = syn.csr_from_mask(rng.random((m, n)) < density, rng=rng)
    dm = G.DevCSR(mask)
    plan = G.sddmm_plan(dm, n).cpu().numpy()
    bands, T = (m + 127) // 128, (n + 127) // 128
    ntiles, nnz = bands * T, mask.nnz
    up16 = lambda x: (x + 15) & ~15
    tile_ptr = plan[:4 * (ntiles + 1)].view(np.int32)
    o_dest = up16(4 * (ntiles + 1))
    dest = plan[o_dest:o_dest + 4 * nnz].view(np.int32)
    o_entry = o_dest + up16(4 * nnz)
    entry = plan[o_entry:o_entry + 2 * nnz].view(np.uint16)
    assert _lib.lib.iex_sddmm_plan_bytes(m, n, nnz) == o_entry + up16(2 * nnz) + up16(4 * ntiles * 128)
    rows = np.repeat(np.arange(m), np.diff(mask.row_offsets))
    cols = mask.column_indices.astype(np.int64)
    tile = (rows // 128) * T + cols // 128
    order = np.argsort(tile, kind="stable")  # storage order kept inside a tile
    np.testing.assert_array_equal(dest, order.astype(np.int32))
    np.testing.assert_array_equal(entry, (((rows % 128) << 7) | (cols % 128))[order].astype(np.uint16))
    np.testing.assert_array_equal(tile_ptr, np.concatenate([[0], np.cumsum(np.bincount(tile, minlength=ntiles))]))


def test_sddmm_tc_output_order_and_accumulate(oracle):
    """lhs = one-hot rows and rhs = small integers make out[p] a function of (row(p), col[p])
    alone, exactly: the output must be aligned with column_indices."""
    rng = np.random.default_rng(3)
    m, n, k = 300, 500, 64
    mask = syn.csr_from_mask(rng.random((m, n)) < 0.1, rng=rng)
    lhs = np.zeros((m, k), np.float32)
    lhs[np.arange(m), np.arange(m) % k] = 1.0 + np.arange(m) // k
    rhs = rng.integers(-8, 9, size=(n, k)).astype(np.float32)
    dm = G.DevCSR(mask)
    plan = G.sddmm_plan(dm, n)
    got = G.sddmm_f32_tc(dm, G.dev(lhs), G.dev(rhs), plan=plan).cpu().numpy()
    rows = np.repeat(np.arange(m), np.diff(mask.row_offsets))
    expect = (1.0 + rows // k) * rhs[mask.column_indices, rows % k]
    np.testing.assert_array_equal(got, expect.astype(np.float32))
    start = torch.full((mask.nnz,), 2.0, device=G.DEV)
    acc = G.sddmm_f32_tc(dm, G.dev(lhs), G.dev(rhs), out=start, accumulate=True, plan=plan).cpu().numpy()
    np.testing.assert_array_equal(acc, (expect + 2.0).astype(np.float32))


def test_sddmm_tc_exact_on_small_integers(oracle):
    """Integers of a few bits are exact in TF32 and their sums in fp32: bit-exact results."""
    rng = np.random.default_rng(8)
    m, n, k = 700, 900, 64
    mask = syn.csr_from_mask(rng.random((m, n)) < 0.07, rng=rng)
    lhs = rng.integers(-7, 8, size=(m, k)).astype(np.float32)
    rhs = rng.integers(-7, 8, size=(n, k)).astype(np.float32)
    got = G.sddmm_f32_tc(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    exact = oracle.sddmm(lhs[None], rhs[None], mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    np.testing.assert_array_equal(got, exact.astype(np.float32))


def test_sddmm_tc_cfg2_full_size_and_agreement_with_cuda_cores(oracle):
    """Benchmark configuration 2 on the tensor-core kernel: against the double-precision
    oracle, the torch CPU path, and the CUDA-core kernel; deterministic from run to run; the
    torch operators give the same bits."""
    mask, q, k, _v = syn.sddmm_chain_case(0)
    dm = G.DevCSR(mask)
    got = _check_tc(oracle, mask, q, k)
    tref = oracle.torch_sddmm(q, k, mask.row_offsets, mask.column_indices)
    assert G.close(got, tref, 1e-5, 1e-5)
    simt = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    tc2 = G.sddmm_f32_tc(dm, G.dev(q), G.dev(k))
    assert torch.equal(tc2.cpu(), torch.as_tensor(got))
    assert G.close(tc2.cpu().numpy(), simt.cpu().numpy(), 1e-5, 1e-5)
    import intrasm_engine_b200  # noqa: F401
    ops = torch.ops.iex_ops
    plan = ops.sddmm_plan(dm.row_offsets, dm.column_indices, 4096, 4096)
    assert torch.equal(ops.sddmm_tc_planned(G.dev(q), G.dev(k), plan, mask.nnz), tc2)


def test_sddmm_tc_takes_unsorted_columns_and_rejects_unsupported(oracle):
    """The plan keeps storage order whatever the order of the columns inside a row."""
    from intrasm_engine_b200 import _lib
    rng = np.random.default_rng(4)
    mask, lhs, rhs = _tc_case(rng, 256, 512, 64, np.full(256, 0.1))
    for r in range(256):  # shuffle every row's columns
        b, e = mask.row_offsets[r], mask.row_offsets[r + 1]
        mask.column_indices[b:e] = rng.permutation(mask.column_indices[b:e])
    _check_tc(oracle, mask, lhs, rhs)
    with pytest.raises(_lib.IexError) as e:
        G.sddmm_f32_tc(G.DevCSR(mask), G.dev(lhs[:, :48].copy()), G.dev(rhs[:, :48].copy()))
    assert e.value.status == -2
    assert _lib.lib.iex_sddmm_f32_tc_supported(256, 64, 512, 1) == 1
    assert _lib.lib.iex_sddmm_f32_tc_supported(256, 64, 512, 2) == 0
    assert _lib.lib.iex_sddmm_f32_prefers_tc(4096, 64, 4096, 838861, 1) == 1
    assert _lib.lib.iex_sddmm_f32_prefers_tc(4096, 64, 4096, 20000, 1) == 0


# ----------------------------------------------------------------------------- fp16
def _sddmm_f16(mask, lhs, rhs):
    from intrasm_engine_b200 import _lib
    batch, m, k = lhs.shape
    n = rhs.shape[1]
    out = torch.empty((mask.nnz,), dtype=torch.float16, device=G.DEV)
    bits = 16 if mask.column_indices.dtype == torch.int16 else 32
    _lib.call("iex_sddmm_f16", m, k, n, mask.nnz, G.ptr(mask.row_indices), G.ptr(mask.row_offsets),
              G.ptr(mask.column_indices), bits, G.ptr(lhs), G.ptr(rhs), G.ptr(out), batch, G.stream_ptr())
    return out


def _f16_bar(got, exact, sum_abs):
    """fp16 operands, fp32 accumulation, one rounding to fp16 at the end: the bar of the
    tensor-core fp16 kernels (2^-10 relative for the final rounding + 1e-5 of the sum of the
    terms' magnitudes for the accumulation order)."""
    return G.tc_close(got, exact, sum_abs)


@pytest.mark.parametrize("m,n,k,density,batch,idx", [
    (1, 1, 1, 1.0, 1, np.int32), (9, 11, 3, 0.5, 1, np.int16), (64, 64, 8, 0.3, 1, np.int16),
    (70, 90, 16, 0.2, 2, np.int32), (128, 128, 32, 0.1, 1, np.int16), (100, 300, 36, 0.2, 1, np.int32),
    (256, 256, 64, 0.05, 3, np.int16), (60, 500, 104, 0.3, 1, np.int16), (64, 64, 128, 0.5, 1, np.int32),
    (48, 80, 264, 0.2, 2, np.int16), (33, 47, 7, 0.6, 1, np.int32), (128, 64, 64, 0.0, 1, np.int16),
    (16, 2000, 64, 0.4, 1, np.int16), (512, 512, 256, 0.1, 1, np.int16),
])
def test_sddmm_half_shapes(oracle, m, n, k, density, batch, idx):
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    mask = syn.csr_from_mask(rng.random((m, n)) < density, rng=rng, index_dtype=idx)
    lhs = rng.standard_normal((batch, m, k)).astype(np.float16)
    rhs = rng.standard_normal((batch, n, k)).astype(np.float16)
    got = _sddmm_f16(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    ci = mask.column_indices.astype(np.int32)
    exact = oracle.sddmm(lhs.astype(np.float32), rhs.astype(np.float32), mask.row_indices, mask.row_offsets, ci,
                         f64=True)
    sabs = oracle.sddmm(np.abs(lhs).astype(np.float32), np.abs(rhs).astype(np.float32), mask.row_indices,
                        mask.row_offsets, ci, f64=True)
    assert got.shape == exact.shape
    assert _f16_bar(got, exact, sabs)


def test_sddmm_half_exact_on_small_integers(oracle):
    """Small-integer operands: every product and partial sum is exact, so is the fp16 result."""
    rng = np.random.default_rng(4)
    m, n, k = 300, 700, 64
    mask = syn.csr_from_mask(rng.random((m, n)) < 0.1, rng=rng, index_dtype=np.int16)
    lhs = rng.integers(-3, 4, size=(1, m, k)).astype(np.float16)
    rhs = rng.integers(-3, 4, size=(1, n, k)).astype(np.float16)
    got = _sddmm_f16(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy().astype(np.float64)
    exact = oracle.sddmm(lhs.astype(np.float32), rhs.astype(np.float32), mask.row_indices, mask.row_offsets,
                         mask.column_indices.astype(np.int32), f64=True)
    assert np.array_equal(got, exact)


def test_sddmm_half_torch_op_and_fp16_backward(oracle):
    """The op, and MySpMM's fp16 backward through it: d values = SDDMM(grad, b) without an fp32 detour."""
    from intrasm_engine_b200.pytorch.cpp_extensions.layers_and_funcs.sputnik import MySpMM
    from intrasm_engine_b200.pytorch.utils import get_transpose_info
    rng = np.random.default_rng(6)
    m, k, n = 256, 384, 64
    a = syn.csr_from_mask(rng.random((m, k)) < 0.2, rng=rng, std=0.1, dtype=np.float16, index_dtype=np.int16)
    da = G.DevCSR(a)
    b = torch.tensor(rng.standard_normal((k, n)).astype(np.float16), device=G.DEV, requires_grad=True)
    values = da.values.clone().requires_grad_(True)
    info = get_transpose_info(m, k, da.row_indices, da.row_offsets, da.column_indices)
    out = MySpMM.run(b, da.row_indices, values, da.row_offsets, da.column_indices, m, info)
    grad = torch.tensor(rng.standard_normal((m, n)).astype(np.float16), device=G.DEV)
    out.backward(grad)
    assert values.grad.dtype == torch.float16
    g32, b32 = grad.float().cpu().numpy()[None], b.detach().float().cpu().numpy()[None]
    ci = a.column_indices.astype(np.int32)
    exact = oracle.sddmm(g32, b32, a.row_indices, a.row_offsets, ci, f64=True)
    sabs = oracle.sddmm(np.abs(g32), np.abs(b32), a.row_indices, a.row_offsets, ci, f64=True)
    assert _f16_bar(values.grad.cpu().numpy(), exact, sabs)
    direct = torch.ops.iex_ops.sddmm_sputnik_half(grad[None], b.detach()[None], da.row_indices, da.row_offsets,
                                                  da.column_indices)
    assert torch.equal(direct, values.grad)


def test_sddmm_tc_batched_equals_single_launches(oracle):
    """Several products of one shape in one launch (own operands, masks and plans; one of them
    with an empty mask): every result equals its single launch bit for bit, CTAs that take more
    than one unit included (6 problems x 32 units on 148 SMs)."""
    import ctypes
    from intrasm_engine_b200 import _lib
    m, n, k, count = 1024, 2048, 64, 6
    rng = np.random.default_rng(21)
    probs = []
    for i in range(count):
        dens = 0.0 if i == 2 else 0.03 + 0.02 * i
        mask = syn.csr_from_mask(rng.random((m, n)) < dens, rng=rng)
        dm = G.DevCSR(mask)
        lhs = G.dev(rng.standard_normal((m, k)).astype(np.float32))
        rhs = G.dev(rng.standard_normal((n, k)).astype(np.float32))
        plan = G.sddmm_plan(dm, n)
        single = G.sddmm_f32_tc(dm, lhs, rhs, plan=plan) if mask.nnz else torch.empty(0, device=G.DEV)
        probs.append((mask, dm, lhs, rhs, plan, single, torch.full((max(mask.nnz, 1),), 7.0, device=G.DEV)))
    P = ctypes.c_void_p * count
    nnz = (ctypes.c_int * count)(*[p[0].nnz for p in probs])
    _lib.call("iex_sddmm_f32_tc_batched", count, m, k, n, nnz, P(*[p[4].data_ptr() for p in probs]),
              P(*[p[2].data_ptr() for p in probs]), P(*[p[3].data_ptr() for p in probs]),
              P(*[p[6].data_ptr() for p in probs]), 0, G.stream_ptr())
    torch.cuda.synchronize()
    assert _lib.lib.iex_last_device_status(1) == 0
    for mask, dm, lhs, rhs, plan, single, out in probs:
        if mask.nnz == 0:
            assert float(out[0]) == 7.0  # untouched
            continue
        assert torch.equal(out, single)
        exact = oracle.sddmm(lhs.cpu().numpy()[None], rhs.cpu().numpy()[None], mask.row_indices, mask.row_offsets,
                             mask.column_indices, f64=True)
        sabs = oracle.sddmm(np.abs(lhs.cpu().numpy())[None], np.abs(rhs.cpu().numpy())[None], mask.row_indices,
                            mask.row_offsets, mask.column_indices, f64=True)
        assert G.sddmm_close(out.cpu().numpy(), exact, sabs)
    too_many = _lib.lib.iex_sddmm_f32_tc_max_batch() + 1
    big = (ctypes.c_void_p * too_many)()
    st = _lib.lib.iex_sddmm_f32_tc_batched(too_many, m, k, n, (ctypes.c_int * too_many)(), big, big, big, big, 0,
                                           G.stream_ptr())
    assert st == -1  # IEX_ERR_BAD_ARG

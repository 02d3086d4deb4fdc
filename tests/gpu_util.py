"""Helpers for the GPU parity tests: device copies of CSR inputs and raw C-ABI calls."""
import numpy as np
import torch

from intrasm_engine_b200 import _lib

DEV = "cuda:0"


def close(got, ref, rtol, scale_tol):
    """|got-ref| <= rtol*|ref| + scale_tol*max|ref| elementwise (float64 compare)."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    if ref.size == 0:
        return got.size == 0
    bound = rtol * np.abs(ref) + scale_tol * np.abs(ref).max()
    return bool(np.all(np.abs(got - ref) <= bound))


def tc_close(got, ref, sum_abs):
    """Bar for the fp16-in / fp32-accumulate tensor-core kernels, as tight as the arithmetic
    earns: |got - ref| <= 2^-10 * |ref| (the final rounding to fp16, with a factor two of
    slack) + 1e-5 * sum_abs, where sum_abs[i, j] = sum_k |a[i, k]| * |b[k, j]| bounds what the
    order of the fp32 accumulation can change.  A dropped or doubled term (one part in a few
    thousand of sum_abs at the benchmark sizes) fails it; the task's own bar of 1e-2 relative
    would not notice one."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    if ref.size == 0:
        return got.size == 0
    bound = 2.0 ** -10 * np.abs(ref) + 1e-5 * np.asarray(sum_abs, dtype=np.float64) + 1e-7
    return bool(np.all(np.abs(got - ref) <= bound))


def spmm_ref_and_sum_abs(oracle, a, b, m, bias=None):
    """fp32 oracle result of A @ b (optionally with bias + ReLU) and |A| @ |b|."""
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, m, bias=bias)[0]
    sabs = oracle.spmm(a.row_indices, np.abs(a.values), a.row_offsets, a.column_indices, np.abs(b), m)[0]
    return ref, sabs.astype(np.float64) + (0.0 if bias is None else np.abs(bias)[:, None])


def linear_ref_and_sum_abs(x, w):
    x32, w32 = np.asarray(x, np.float32), np.asarray(w, np.float32)
    return x32 @ w32.T, np.abs(x32) @ np.abs(w32).T


def max_violation(got, ref, rtol, scale_tol):
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    bound = rtol * np.abs(ref) + scale_tol * np.abs(ref).max() + 1e-300
    return float(np.max(np.abs(got - ref) / bound))


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV)


class DevCSR:
    def __init__(self, csr):
        self.m, self.k = csr.shape
        self.nnz = csr.nnz
        self.values = dev(csr.values)
        self.row_indices = dev(csr.row_indices.astype(np.int32))
        self.row_offsets = dev(csr.row_offsets.astype(np.int32))
        self.column_indices = dev(csr.column_indices)


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return None if t is None else t.data_ptr()


def spmm_f32(a: DevCSR, dense, bias=None, out=None, accumulate=False, values=None):
    """Raw iex_spmm_f32 call. dense [batch,k,n] device fp32; returns [batch,m,n]."""
    batch, k, n = dense.shape
    vals = a.values if values is None else values
    vstride = 0 if vals.dim() == 1 else vals.shape[1]
    if out is None:
        out = torch.empty((batch, a.m, n), dtype=torch.float32, device=DEV)
    _lib.call("iex_spmm_f32", a.m, k, n, a.nnz, ptr(a.row_indices), ptr(vals), vstride,
              ptr(a.row_offsets), ptr(a.column_indices), ptr(dense), ptr(bias), ptr(out),
              batch, int(accumulate), stream_ptr())
    return out


def spmm_f16(a: DevCSR, dense, bias=None):
    batch, k, n = dense.shape
    out = torch.empty((batch, a.m, n), dtype=torch.float16, device=DEV)
    name = "iex_spmm_f16_i16" if a.column_indices.dtype == torch.int16 else "iex_spmm_f16_i32"
    _lib.call(name, a.m, k, n, a.nnz, ptr(a.row_indices), ptr(a.values), ptr(a.row_offsets),
              ptr(a.column_indices), ptr(dense), ptr(bias), ptr(out), batch, stream_ptr())
    return out


def sddmm_f32(mask: DevCSR, lhs, rhs, out=None, accumulate=False):
    batch, m, k = lhs.shape
    n = rhs.shape[1]
    if out is None:
        out = torch.empty((mask.nnz,), dtype=torch.float32, device=DEV)
    _lib.call("iex_sddmm_f32", m, k, n, mask.nnz, ptr(mask.row_indices), ptr(mask.row_offsets),
              ptr(mask.column_indices), ptr(lhs), ptr(rhs), ptr(out), batch, int(accumulate),
              stream_ptr())
    return out


def sddmm_plan(mask: DevCSR, n):
    """Plan of the pattern for the tensor-core SDDMM (iex_sddmm_plan_build); an opaque buffer."""
    nbytes = _lib.lib.iex_sddmm_plan_bytes(mask.m, n, mask.nnz)
    plan = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=DEV)
    _lib.call("iex_sddmm_plan_build", mask.m, n, mask.nnz, ptr(mask.row_offsets), ptr(mask.column_indices),
              ptr(plan), nbytes, stream_ptr())
    return plan


def sddmm_f32_tc(mask: DevCSR, lhs2d, rhs2d, out=None, accumulate=False, plan=None):
    """Raw iex_sddmm_f32_tc call (tensor cores; batch 1): lhs [m, k], rhs [n, k] device fp32."""
    m, k = lhs2d.shape
    n = rhs2d.shape[0]
    if plan is None:
        plan = sddmm_plan(mask, n)
    if out is None:
        out = torch.empty((mask.nnz,), dtype=torch.float32, device=DEV)
    _lib.call("iex_sddmm_f32_tc", m, k, n, mask.nnz, ptr(plan), ptr(lhs2d), ptr(rhs2d), ptr(out),
              int(accumulate), stream_ptr())
    return out


def sddmm_close(got, exact, sum_abs):
    """The fp32 bar of the task (1e-5 relative) with the error measured against the sum of the
    terms' magnitudes, which is what a dot product's rounding error scales with:
    |got - exact| <= 1e-5 * |exact| + 2e-6 * sum_k |lhs||rhs|."""
    got = np.asarray(got, dtype=np.float64)
    exact = np.asarray(exact, dtype=np.float64)
    if exact.size == 0:
        return got.size == 0
    return bool(np.all(np.abs(got - exact) <= 1e-5 * np.abs(exact) + 2e-6 * np.asarray(sum_abs, np.float64)))


def spmm_f32_tc(a: DevCSR, dense2d, values=None):
    """iex_tile_plan_build (64-column tiles) + iex_spmm_f32_tc: dense [k, n] device fp32 -> [m, n]."""
    k, n = dense2d.shape
    nbytes = _lib.lib.iex_tile_plan_bytes(a.m, k, a.nnz, 64)
    plan = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=DEV)
    _lib.call("iex_tile_plan_build", a.m, k, a.nnz, 64, ptr(a.row_offsets), ptr(a.column_indices), ptr(plan),
              nbytes, stream_ptr())
    need = _lib.lib.iex_spmm_f32_tc_workspace_bytes(a.m, k, n)
    ws = torch.empty(max(int(need), 16), dtype=torch.uint8, device=DEV)
    out = torch.full((a.m, n), float("nan"), dtype=torch.float32, device=DEV)
    vals = a.values if values is None else values
    _lib.call("iex_spmm_f32_tc", a.m, k, n, a.nnz, ptr(plan), ptr(vals), ptr(dense2d), ptr(out), ptr(ws), need,
              stream_ptr())
    return out

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

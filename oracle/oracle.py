"""numpy front end of the CPU oracle (``iex_oracle.c``) plus the torch CPU path.

TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared against.  Nothing in
``intrasm_engine_b200`` imports this module; only the tests, the smoke check and the CPU
baseline leg of the benchmark do.

PARITY STATUS: "parity unpinned" by the reference's own tests (it has none that evaluate
SpMM or SDDMM, tests/test_torch_load_library.py:15-19).  The C restatement is pinned
against ``tests/golden/*.npz``, made with ``torch.sparse.mm``,
``torch.sparse.sampled_addmm`` and ``torch.matmul`` on CPU by
``tests/golden/make_golden.py``.

Two layers:
  * ``spmm`` / ``sddmm`` / ``linear`` — the C restatement (fp32 FMA in the reference's
    term order; ``*_f64`` for double accumulation).  Half inputs are widened to fp32
    exactly, as the reference's fp16 kernel does before accumulating
    (sputnik_spmm.cu.inc:187).
  * ``torch_spmm`` / ``torch_sddmm`` / ``torch_linear`` — the multi-threaded torch CPU
    kernels, the timed CPU baseline.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libiex_oracle.so")
_lib = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_u8p = ctypes.POINTER(ctypes.c_uint8)


def build(force: bool = False) -> str:
    """Compile ``iex_oracle.c`` with the Makefile beside it; returns the library path."""
    src = os.path.join(_HERE, "iex_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libiex_oracle.so"], check=True,
                       capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.int32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.float32)


def spmm(row_indices, values, row_offsets, column_indices, dense, m, bias=None,
         out=None, f64: bool = False) -> np.ndarray:
    """``out[z, r, :] = sum_p values[p] * dense[z, col[p], :]`` (+bias, ReLU).

    ``dense`` is ``[batch, k, n]`` (or ``[k, n]``); ``values`` is ``[nnz]`` (shared by the
    batch) or ``[batch, nnz]``.  ``out`` given => the result is added onto it (the
    atomic-store variant).  Returns fp32 (fp64 when ``f64``) ``[batch, m, n]``.
    """
    lib = _load()
    dense = _f32(dense)
    if dense.ndim == 2:
        dense = dense[None]
    batch, k, n = dense.shape
    values = _f32(values)
    ri, ro, ci = _i32(row_indices), _i32(row_offsets), _i32(column_indices)
    nnz = ci.shape[0]
    stride = 0 if values.ndim == 1 else nnz
    if values.ndim == 2:
        assert values.shape == (batch, nnz)
    if f64:
        res = np.zeros((batch, m, n), dtype=np.float64)
        lib.iex_oracle_spmm_f64(m, k, n, batch, _p(ri, _i32p), _p(values, _f32p),
                                ctypes.c_long(stride), _p(ro, _i32p), _p(ci, _i32p),
                                _p(dense, _f32p), _p(res, _f64p))
        return res
    accumulate = out is not None
    res = np.zeros((batch, m, n), dtype=np.float32) if out is None else _f32(out).copy()
    b = None if bias is None else _f32(bias)
    lib.iex_oracle_spmm_f32(m, k, n, nnz, batch, _p(ri, _i32p), _p(values, _f32p),
                            ctypes.c_long(stride), _p(ro, _i32p), _p(ci, _i32p),
                            _p(dense, _f32p), None if b is None else _p(b, _f32p),
                            _p(res, _f32p), int(accumulate))
    return res


def sddmm(lhs, rhs, row_indices, row_offsets, column_indices, out=None,
          f64: bool = False) -> np.ndarray:
    """``out[p] = sum_z dot(lhs[z, row(p)], rhs[z, col[p]])``; lhs ``[batch,m,k]``, rhs ``[batch,n,k]``."""
    lib = _load()
    lhs, rhs = _f32(lhs), _f32(rhs)
    if lhs.ndim == 2:
        lhs, rhs = lhs[None], rhs[None]
    batch, m, k = lhs.shape
    n = rhs.shape[1]
    ri, ro, ci = _i32(row_indices), _i32(row_offsets), _i32(column_indices)
    nnz = ci.shape[0]
    if f64:
        res = np.zeros(nnz, dtype=np.float64)
        lib.iex_oracle_sddmm_f64(m, k, n, batch, _p(ri, _i32p), _p(ro, _i32p),
                                 _p(ci, _i32p), _p(lhs, _f32p), _p(rhs, _f32p),
                                 _p(res, _f64p))
        return res
    accumulate = out is not None
    res = np.zeros(nnz, dtype=np.float32) if out is None else _f32(out).copy()
    lib.iex_oracle_sddmm_f32(m, k, n, nnz, batch, _p(ri, _i32p), _p(ro, _i32p),
                             _p(ci, _i32p), _p(lhs, _f32p), _p(rhs, _f32p),
                             _p(res, _f32p), int(accumulate))
    return res


def linear(inp, weight) -> np.ndarray:
    """``input @ weight.T`` with sequential fp32 FMA (small cases); fp32 result."""
    lib = _load()
    inp, weight = _f32(inp), _f32(weight)
    t, c = inp.shape
    f = weight.shape[0]
    res = np.zeros((t, f), dtype=np.float32)
    lib.iex_oracle_linear_f32(t, c, f, _p(inp, _f32p), _p(weight, _f32p), _p(res, _f32p))
    return res


def dense_to_csr(dense: np.ndarray, relu: bool = False, index_dtype=np.int32):
    """CSR of a dense matrix (of relu(dense) with ``relu``): ``(values, row_indices,
    row_offsets, column_indices)``; rows ordered by decreasing length (stable), columns
    ascending -- the layout intrasm_engine/pytorch/utils.py:143-153 obtains from xformers."""
    dense = np.asarray(dense)
    mask = dense > 0 if relu else dense != 0
    counts = mask.sum(axis=1)
    row_offsets = np.zeros(dense.shape[0] + 1, dtype=np.int32)
    row_offsets[1:] = np.cumsum(counts)
    column_indices = np.nonzero(mask)[1].astype(index_dtype)
    values = dense[mask]
    row_indices = np.argsort(-counts.astype(np.int64), kind="stable").astype(np.int32)
    return values, row_indices, row_offsets, column_indices


def validate_csr(m, k, row_indices, row_offsets, column_indices) -> int:
    """0 when the CSR triple satisfies every launcher precondition, else a rule code."""
    lib = _load()
    ri, ro, ci = _i32(row_indices), _i32(row_offsets), _i32(column_indices)
    if ri.shape[0] != m or ro.shape[0] != m + 1:
        return 6
    seen = np.zeros(max(m, 1), dtype=np.uint8)
    return int(lib.iex_oracle_validate_csr(m, k, ci.shape[0], _p(ri, _i32p), _p(ro, _i32p),
                                           _p(ci, _i32p), _p(seen, _u8p)))


# --------------------------------------------------------------------------------------
# torch CPU path: the oracle of record named by the task and the timed CPU baseline.
# CSR matmul is not implemented for Half on CPU, so half inputs are widened to fp32.
# int32 indices select the fast (MKL) CSR path; int64 indices do not.
# --------------------------------------------------------------------------------------

def torch_csr(row_offsets, column_indices, values, m, k):
    import torch
    return torch.sparse_csr_tensor(
        torch.as_tensor(np.asarray(row_offsets, dtype=np.int32)),
        torch.as_tensor(np.asarray(column_indices, dtype=np.int32)),
        torch.as_tensor(np.asarray(values, dtype=np.float32)),
        size=(m, k),
    )


def torch_spmm(row_offsets, column_indices, values, dense, m):
    """``torch.sparse.mm(A_csr, dense)`` on CPU in fp32; ``dense`` is ``[k, n]``."""
    import torch
    dense_t = torch.as_tensor(np.asarray(dense, dtype=np.float32))
    a = torch_csr(row_offsets, column_indices, values, m, dense_t.shape[0])
    return torch.sparse.mm(a, dense_t).numpy()


def torch_sddmm(lhs, rhs, row_offsets, column_indices):
    """``torch.sparse.sampled_addmm`` with a zero CSR input and ``beta=0``; returns ``[nnz]`` values."""
    import torch
    lhs_t = torch.as_tensor(np.asarray(lhs, dtype=np.float32))
    rhs_t = torch.as_tensor(np.asarray(rhs, dtype=np.float32))
    nnz = len(column_indices)
    mask = torch_csr(row_offsets, column_indices, np.zeros(nnz, np.float32),
                     lhs_t.shape[0], rhs_t.shape[0])
    res = torch.sparse.sampled_addmm(mask, lhs_t, rhs_t.t(), beta=0.0)
    return res.values().numpy()


def torch_linear(inp, weight):
    import torch
    return torch.matmul(torch.as_tensor(np.asarray(inp, dtype=np.float32)),
                        torch.as_tensor(np.asarray(weight, dtype=np.float32)).t()).numpy()

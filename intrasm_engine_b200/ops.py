"""``torch.ops.iex_ops.*`` — the reference's operator boundary, bound to the C ABI.

Schemas, argument checks, output shapes and stream choice follow
intrasm_engine/pytorch/csrc/extensions/sputnik_kernels.cpp:32-193.  Outputs come from the
torch caching allocator and kernels are enqueued on the current torch stream with no
synchronisation, so every op can be recorded by a stream capture, as the reference's
callers do (layers_and_funcs/sputnik.py:59-66).

Deliberate differences from the reference, all supersets:
  * ``spmm_sputnik_reuse_weight_half`` is registered (the reference defines it at
    sputnik_kernels.cpp:179-181 but leaves it out of the TORCH_LIBRARY block :189-193);
    it takes int16 or int32 column indices.
  * The atomic variants zero their output before accumulating; the reference accumulates
    onto an uninitialised ``at::empty`` tensor (sputnik_kernels.cpp:91, :21-24).
  * ``linear_fp16``, ``spmm_tc_half`` and ``fused_spmm_linear_half`` are new ops for the dense
    branch, the tensor-core SpMM and the fused sparse||dense layer; the reference has no
    kernel of its own for any of them.
"""
from __future__ import annotations

import torch

from . import _lib

_DEF = torch.library.Library("iex_ops", "DEF")


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _common_checks(named: dict) -> None:
    first = next(iter(named.values()))
    for name, t in named.items():
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
        _check(t.is_contiguous(), f"{name} must be a contiguous tensor")
        _check(not t.is_sparse, f"{name} must be a dense tensor")
        _check(t.device == first.device, f"{name} should be in the same device as {next(iter(named))}")


def _spmm_checks(b, row_indices, values, row_offsets, column_indices, m, per_batch_values):
    _check(b.dim() == 3, "b must be [batch, k, n]")
    if per_batch_values:
        _check(values.dim() == 2, "values must be [batch, nnz]")
        _check(b.size(0) == values.size(0), "values and b disagree on the batch size")
        _check(values.size(1) == column_indices.size(0), "values and column_indices disagree on nnz")
    else:
        _check(values.dim() == 1, "values must be [nnz]")
        _check(values.size(0) == column_indices.size(0), "values and column_indices disagree on nnz")
    _check(row_indices.dim() == 1 and row_offsets.dim() == 1 and column_indices.dim() == 1,
           "row_indices, row_offsets and column_indices must be 1-D")
    _common_checks({"b": b, "row_indices": row_indices, "values": values,
                    "row_offsets": row_offsets, "column_indices": column_indices})
    _check(row_indices.dtype == torch.int32 and row_offsets.dtype == torch.int32,
           "row_indices and row_offsets must be int32")
    _check(row_indices.size(0) == m and row_offsets.size(0) == m + 1,
           "row_indices must have m entries and row_offsets m + 1")
    batch, nnz = b.size(0), column_indices.size(0)
    _check(batch == 1 or nnz % 4 == 0,
           "If batch size > 1 then number of nonzeros should be a multiple of 4")


def _spmm_f32(b, row_indices, values, row_offsets, column_indices, m, per_batch_values):
    _spmm_checks(b, row_indices, values, row_offsets, column_indices, m, per_batch_values)
    _check(b.dtype == torch.float32 and values.dtype == torch.float32, "b and values must be float32")
    _check(column_indices.dtype == torch.int32, "column_indices must be int32")
    batch, k, n = b.shape
    nnz = column_indices.size(0)
    with torch.cuda.device(b.device):
        if per_batch_values:
            out = torch.zeros((batch, m, n), dtype=b.dtype, device=b.device)
        else:
            out = torch.empty((batch, m, n), dtype=b.dtype, device=b.device)
        _lib.call("iex_spmm_f32", m, k, n, nnz, row_indices.data_ptr(), values.data_ptr(),
                  nnz if per_batch_values else 0, row_offsets.data_ptr(),
                  column_indices.data_ptr(), b.data_ptr(), None, out.data_ptr(), batch,
                  1 if per_batch_values else 0, _stream_ptr(b.device))
    return out


def spmm_sputnik_reuse_weight(b, row_indices, values, row_offsets, column_indices, m):
    """fp32 CSR SpMM, one values vector shared by the batch (sputnik_kernels.cpp:173-175)."""
    return _spmm_f32(b, row_indices, values, row_offsets, column_indices, int(m), False)


def spmm_sputnik_atomic(b, row_indices, values, row_offsets, column_indices, m):
    """fp32 CSR SpMM with per-batch values, atomic accumulate (sputnik_kernels.cpp:170-172)."""
    return _spmm_f32(b, row_indices, values, row_offsets, column_indices, int(m), True)


def spmm_sputnik_reuse_weight_half(b, row_indices, values, row_offsets, column_indices, m):
    """fp16 CSR SpMM, fp32 accumulate, int16 or int32 column indices (sputnik_kernels.cpp:179-181)."""
    m = int(m)
    _spmm_checks(b, row_indices, values, row_offsets, column_indices, m, False)
    _check(b.dtype == torch.float16 and values.dtype == torch.float16, "b and values must be float16")
    _check(column_indices.dtype in (torch.int16, torch.int32), "column_indices must be int16 or int32")
    batch, k, n = b.shape
    nnz = column_indices.size(0)
    name = "iex_spmm_f16_i16" if column_indices.dtype == torch.int16 else "iex_spmm_f16_i32"
    with torch.cuda.device(b.device):
        out = torch.empty((batch, m, n), dtype=b.dtype, device=b.device)
        _lib.call(name, m, k, n, nnz, row_indices.data_ptr(), values.data_ptr(),
                  row_offsets.data_ptr(), column_indices.data_ptr(), b.data_ptr(), None,
                  out.data_ptr(), batch, _stream_ptr(b.device))
    return out


def sddmm_sputnik_atomic_upd_weight(a, b, row_indices, row_offsets, column_indices):
    """fp32 SDDMM, batch items summed into one ``[nnz]`` vector (sputnik_kernels.cpp:182-184)."""
    _check(a.dim() == b.dim() and a.dim() == 3, "a and b must be [batch, rows, k]")
    _check(a.size(0) == b.size(0), "a and b disagree on the batch size")
    _check(a.size(2) == b.size(2), "a and b disagree on k")
    _check(row_indices.dim() == 1 and row_offsets.dim() == 1 and column_indices.dim() == 1,
           "row_indices, row_offsets and column_indices must be 1-D")
    _common_checks({"a": a, "b": b, "row_indices": row_indices, "row_offsets": row_offsets,
                    "column_indices": column_indices})
    _check(a.dtype == torch.float32 and b.dtype == torch.float32, "a and b must be float32")
    _check(row_indices.dtype == torch.int32 and row_offsets.dtype == torch.int32
           and column_indices.dtype == torch.int32, "index tensors must be int32")
    batch, m, k = a.shape
    n = b.size(1)
    _check(row_indices.size(0) == m and row_offsets.size(0) == m + 1,
           "row_indices must have m entries and row_offsets m + 1")
    nnz = column_indices.size(0)
    with torch.cuda.device(a.device):
        out = torch.empty((nnz,), dtype=a.dtype, device=a.device)
        _lib.call("iex_sddmm_f32", m, k, n, nnz, row_indices.data_ptr(), row_offsets.data_ptr(),
                  column_indices.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), batch,
                  0, _stream_ptr(a.device))
    return out


def linear_fp16(input, weight):
    """Dense branch on tensor cores: ``input @ weight.T`` (fp16 in, fp32 accumulate, fp16 out).

    ``input`` ``[tokens, in_features]``, ``weight`` ``[out_features, in_features]`` — the
    computation of MyLinear.forward (layers_and_funcs/torch.py:17).  tokens must be a multiple
    of 16 and at most 256, in_features a multiple of 8.
    """
    _check(input.dim() == 2 and weight.dim() == 2, "input and weight must be 2-D")
    _check(input.size(1) == weight.size(1), "input and weight disagree on in_features")
    _common_checks({"input": input, "weight": weight})
    _check(input.dtype == torch.float16 and weight.dtype == torch.float16, "input and weight must be float16")
    tokens, cin = input.shape
    cout = weight.size(0)
    with torch.cuda.device(input.device):
        out = torch.empty((tokens, cout), dtype=input.dtype, device=input.device)
        _lib.call("iex_linear_f16", tokens, cin, cout, input.data_ptr(), weight.data_ptr(),
                  out.data_ptr(), _stream_ptr(input.device))
    return out


def _tc_sparse_checks(x, row_offsets, values, column_indices, m):
    _check(x.dim() == 2, "x must be [k, n]")
    _check(values.dim() == 1 and values.size(0) == column_indices.size(0),
           "values and column_indices must be 1-D with nnz entries")
    _check(row_offsets.dim() == 1 and row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries")
    _common_checks({"x": x, "row_offsets": row_offsets, "values": values, "column_indices": column_indices})
    _check(x.dtype == torch.float16 and values.dtype == torch.float16, "x and values must be float16")
    _check(row_offsets.dtype == torch.int32, "row_offsets must be int32")
    _check(column_indices.dtype in (torch.int16, torch.int32), "column_indices must be int16 or int32")
    return 16 if column_indices.dtype == torch.int16 else 32


def spmm_tc_half(x, row_offsets, values, column_indices, m):
    """CSR SpMM on tensor cores: ``A @ x`` with A ``[m, k]`` in CSR and x ``[k, n]`` fp16.

    Column indices must ascend inside each row (what every CSR converter produces); rows
    are taken in natural order, so there is no ``row_indices`` argument.  n must be 64 or
    128 and k a multiple of 8.  Returns ``[m, n]``.
    """
    m = int(m)
    bits = _tc_sparse_checks(x, row_offsets, values, column_indices, m)
    k, n = x.shape
    with torch.cuda.device(x.device):
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
        _lib.call("iex_spmm_f16_tc", m, k, n, column_indices.size(0), row_offsets.data_ptr(),
                  column_indices.data_ptr(), bits, values.data_ptr(), x.data_ptr(), out.data_ptr(),
                  _stream_ptr(x.device))
    return out


def fused_spmm_linear_half(x, row_offsets, values, column_indices, m, weight):
    """Fused sparse || dense layer in ONE launch, both branches reading ``x`` ``[k, n]``:

        out_sparse = A_csr @ x            ``[m, n]``
        out_dense  = (weight @ x).T       ``[n, out_features]``   (MyLinear's layout)

    The reference has no kernel for this; its pair function runs the two library calls
    on two captured streams (tests/test_interleaving.py:434-476).
    """
    m = int(m)
    bits = _tc_sparse_checks(x, row_offsets, values, column_indices, m)
    _check(weight.dim() == 2 and weight.size(1) == x.size(0), "weight must be [out_features, k]")
    _common_checks({"x": x, "weight": weight})
    _check(weight.dtype == torch.float16, "weight must be float16")
    k, n = x.shape
    md = weight.size(0)
    with torch.cuda.device(x.device):
        out_s = torch.empty((m, n), dtype=x.dtype, device=x.device)
        out_d = torch.empty((n, md), dtype=x.dtype, device=x.device)
        _lib.call("iex_fused_spmm_linear_f16", m, md, k, n, column_indices.size(0),
                  row_offsets.data_ptr(), column_indices.data_ptr(), bits, values.data_ptr(),
                  weight.data_ptr(), x.data_ptr(), out_s.data_ptr(), out_d.data_ptr(), 1,
                  _stream_ptr(x.device))
    return out_s, out_d


_SPMM_SCHEMA = ("(Tensor b, Tensor row_indices, Tensor values, Tensor row_offsets, "
                "Tensor column_indices, int m) -> Tensor")
_DEF.define("spmm_sputnik_reuse_weight" + _SPMM_SCHEMA)
_DEF.define("spmm_sputnik_atomic" + _SPMM_SCHEMA)
_DEF.define("spmm_sputnik_reuse_weight_half" + _SPMM_SCHEMA)
_DEF.define("sddmm_sputnik_atomic_upd_weight(Tensor a, Tensor b, Tensor row_indices, "
            "Tensor row_offsets, Tensor column_indices) -> Tensor")
_DEF.define("linear_fp16(Tensor input, Tensor weight) -> Tensor")
_DEF.define("spmm_tc_half(Tensor x, Tensor row_offsets, Tensor values, Tensor column_indices, int m) -> Tensor")
_DEF.define("fused_spmm_linear_half(Tensor x, Tensor row_offsets, Tensor values, Tensor column_indices, "
            "int m, Tensor weight) -> (Tensor, Tensor)")
_DEF.impl("linear_fp16", linear_fp16, "CUDA")
_DEF.impl("spmm_tc_half", spmm_tc_half, "CUDA")
_DEF.impl("fused_spmm_linear_half", fused_spmm_linear_half, "CUDA")
_DEF.impl("spmm_sputnik_reuse_weight", spmm_sputnik_reuse_weight, "CUDA")
_DEF.impl("spmm_sputnik_atomic", spmm_sputnik_atomic, "CUDA")
_DEF.impl("spmm_sputnik_reuse_weight_half", spmm_sputnik_reuse_weight_half, "CUDA")
_DEF.impl("sddmm_sputnik_atomic_upd_weight", sddmm_sputnik_atomic_upd_weight, "CUDA")

"""``MySpMM`` — CSR SpMM as an autograd operator (forward SpMM; backward SDDMM + SpMM on A^T).

Same inputs as intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/sputnik.py:19-149:
``(b, row_indices, values, row_offsets, column_indices, m, _transp_info)`` with ``b`` the
dense ``[k, n]`` operand, and the same derivative scheme (:77-149):
    d values = SDDMM(grad, b) sampled at A's pattern,   d b = A^T @ grad.
fp32 runs the CUDA-core kernels (bit-reproducible); fp16 runs the CUDA-core fp16 kernel or,
with ``use_tensor_cores=True`` in the forward kwargs, the tcgen05 kernel;
``use_tensor_cores="auto"`` lets the cost model of ``pytorch/tuning.py`` choose.
"""
from __future__ import annotations

import torch

from .... import ops  # noqa: F401  (registers torch.ops.iex_ops)
from ...tuning import choose_spmm_kernel
from ...utils import transpose_with_info
from .utils import MyAutogradFunc, captured


def _spmm(b2d, row_indices, values, row_offsets, column_indices, m, use_tc=False):
    if values.dtype == torch.float32:
        return torch.ops.iex_ops.spmm_sputnik_reuse_weight(b2d.unsqueeze(0), row_indices, values,
                                                           row_offsets, column_indices, m)[0]
    if use_tc == "auto":  # cost model fitted to measurements (pytorch/tuning.py)
        use_tc = choose_spmm_kernel(m, b2d.size(0), b2d.size(1), values.numel(), 16,
                                    16 if column_indices.dtype == torch.int16 else 32) == "tensor_core"
    if use_tc:
        return torch.ops.iex_ops.spmm_tc_half(b2d, row_offsets, values, column_indices, m)
    return torch.ops.iex_ops.spmm_sputnik_reuse_weight_half(b2d.unsqueeze(0), row_indices, values,
                                                            row_offsets, column_indices, m)[0]


def _sddmm(grad2d, b2d, row_indices, row_offsets, column_indices):
    if grad2d.dtype == torch.float16:  # fp16 operands as they are: fp32 accumulation, fp16 result
        return torch.ops.iex_ops.sddmm_sputnik_half(grad2d.unsqueeze(0), b2d.to(torch.float16).unsqueeze(0),
                                                    row_indices, row_offsets, column_indices)
    return torch.ops.iex_ops.sddmm_sputnik_atomic_upd_weight(
        grad2d.unsqueeze(0), b2d.unsqueeze(0), row_indices, row_offsets, column_indices.to(torch.int32))


class MySpMM(MyAutogradFunc):
    @staticmethod
    def num_inputs(**kwargs) -> int:
        return 7

    @staticmethod
    def num_input_tensors(**kwargs) -> int:
        return 5

    @staticmethod
    def num_outputs(**kwargs) -> int:
        return 1

    @staticmethod
    def num_saved_tensors(**ctx_kwargs) -> int:
        return 5 + int(ctx_kwargs.get("num_transp_info", 4))

    @staticmethod
    def _forward(b, row_indices, values, row_offsets, column_indices, m, _transp_info, **kwargs):
        assert kwargs.get("num_streams", 1) == 1
        b = b.contiguous()
        with captured(kwargs.get("constructor"), kwargs.get("stream_beg", 0),
                      kwargs.get("constructor_enabled", False)):
            out = _spmm(b, row_indices, values, row_offsets, column_indices, int(m),
                        kwargs.get("use_tensor_cores", False))
        ctx_dict = {
            "backward_constructor": kwargs.get("backward_constructor"),
            "constructor_enabled": kwargs.get("constructor_enabled", False),
            "stream_beg": kwargs.get("stream_beg", 0),
            "num_transp_info": len(_transp_info),
            "needs_input_grad": (b.requires_grad, values.requires_grad),
        }
        saved = (b, row_indices, values, row_offsets, column_indices, *_transp_info)
        return (out,), ctx_dict, saved

    @staticmethod
    def _backward(grad, b, row_indices, values, row_offsets, column_indices, *_transp_info, **ctx):
        k = b.shape[0]
        grad = grad.contiguous()
        need_b, need_values = ctx.get("needs_input_grad", (True, True))
        bc, enabled, sidx = ctx.get("backward_constructor"), ctx.get("constructor_enabled", False), \
            ctx.get("stream_beg", 0)
        grad_values = grad_b = None
        if need_values:
            with captured(bc, sidx, enabled):
                grad_values = _sddmm(grad, b, row_indices, row_offsets, column_indices)
        if need_b:
            # transposing the pattern is bookkeeping outside the recorded region (sputnik.py:96-99)
            ri_t, values_t, ro_t, ci_t = transpose_with_info(values, _transp_info)
            with captured(bc, sidx, enabled):
                grad_b = _spmm(grad, ri_t, values_t, ro_t, ci_t, k)
        return grad_b, None, grad_values, None, None, None, None


class MySpMMPartitioned(MyAutogradFunc):
    """Row-partitioned SpMM: the rows of A are cut into nnz-balanced contiguous ranges and
    each range is one independent SpMM (on one GPU: back-to-back launches; across GPUs: one
    range per rank, no communication).  The reference leaves this class empty
    (sputnik.py:152-154)."""

    @staticmethod
    def num_inputs(**kwargs) -> int:
        return 6

    @staticmethod
    def num_outputs(**kwargs) -> int:
        return 1

    @staticmethod
    def num_saved_tensors(**kwargs) -> int:
        return 0

    @staticmethod
    def _forward(b, values, row_offsets, column_indices, m, parts, **kwargs):
        from ...utils import nnz_balanced_row_split, slice_csr_rows
        outs = []
        for begin, end in nnz_balanced_row_split(row_offsets, int(parts)):
            v, ri, ro, ci = slice_csr_rows(values, row_offsets, column_indices, begin, end)
            outs.append(_spmm(b.contiguous(), ri, v, ro, ci, end - begin,
                              kwargs.get("use_tensor_cores", False)))
        return (torch.cat(outs, 0),), {}, ()

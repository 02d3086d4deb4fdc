"""Swapping the sparse operators into a model's linear layers.

The reference sketches a peft-style tuner that walks a LLaMA model's modules and replaces the
targets (intrasm_engine/pytorch/huggingface_rewriter.py:91-170, ``inject_adapter`` /
``_create_and_replace``); it needs ``peft`` and its replacement modules were never written.
This is the part of it that the hot path needs, without ``peft``: a drop-in for
``torch.nn.Linear`` whose weight is a pruned CSR matrix (``SparseLinear``, forward and backward
through ``MySpMM``), and ``inject_sparse_linears`` that walks ``named_modules`` and replaces
the matching linears -- e.g. ``up_proj`` / ``gate_proj`` of every ``LlamaMLP``.
"""
from __future__ import annotations

import torch
from torch import nn

from . import horizontal_rewriter as hr
from .cpp_extensions.layers_and_funcs.sputnik import MySpMM
from .cpp_extensions.layers_and_funcs.utils import default_fwd_kwargs
from .utils import dense_to_sparse_cuda, get_transpose_info

hr.make_single_kernel_autograd_function(MySpMM)


def magnitude_prune(weight: torch.Tensor, sparsity: float) -> torch.Tensor:
    """``weight`` with its ``sparsity`` fraction of smallest-magnitude entries set to zero."""
    if sparsity <= 0.0:
        return weight.clone()
    k = int(weight.numel() * sparsity)
    if k == 0:
        return weight.clone()
    threshold = weight.abs().flatten().float().kthvalue(k).values
    return torch.where(weight.abs().float() > threshold, weight, torch.zeros_like(weight))


class SparseLinear(nn.Module):
    """``y = x @ W.T (+ bias)`` with ``W`` ``[out_features, in_features]`` stored as CSR (fp16
    values, int16 column indices when they fit).  The product runs as ``W_csr @ x.T`` through
    ``MySpMM`` -- the tensor-core kernel for 64..256 tokens in multiples of 64, the CUDA-core
    kernel otherwise, chosen by the cost model -- so gradients reach ``x`` (and ``values``)."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        super().__init__()
        assert weight.is_cuda and weight.dtype == torch.float16 and weight.dim() == 2
        self.out_features, self.in_features = weight.shape
        # 16-bit indices when both dimensions fit (the transposed pattern of the backward pass
        # stores row numbers in the same index type)
        index_dtype = torch.int16 if max(self.in_features, self.out_features) <= 32767 else torch.int32
        values, row_indices, row_offsets, column_indices = dense_to_sparse_cuda(
            weight.contiguous(), index_dtype=index_dtype)
        self.values = nn.Parameter(values, requires_grad=False)
        self.register_buffer("row_indices", row_indices)
        self.register_buffer("row_offsets", row_offsets)
        self.register_buffer("column_indices", column_indices)
        self.transp_info = get_transpose_info(self.out_features, self.in_features, row_indices, row_offsets,
                                              column_indices)
        self.bias = None if bias is None else nn.Parameter(bias.detach().clone(), requires_grad=False)

    @classmethod
    def from_linear(cls, linear: nn.Linear, sparsity: float) -> "SparseLinear":
        return cls(magnitude_prune(linear.weight.detach(), sparsity), linear.bias)

    def density(self) -> float:
        return self.values.numel() / float(self.out_features * self.in_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        b = x.reshape(-1, self.in_features).t().contiguous()  # [in_features, tokens]
        out = MySpMM.run(b, self.row_indices, self.values, self.row_offsets, self.column_indices,
                         self.out_features, self.transp_info,
                         fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores="auto"))
        y = out.t()
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)


def inject_sparse_linears(model: nn.Module, target_modules=("up_proj", "gate_proj"), sparsity: float = 0.5) -> int:
    """Replaces every ``nn.Linear`` whose attribute name is in ``target_modules`` (at any depth)
    by a ``SparseLinear`` of its magnitude-pruned weight; returns how many were replaced."""
    replaced = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if name in target_modules and isinstance(child, nn.Linear):
                setattr(parent, name, SparseLinear.from_linear(child, sparsity))
                replaced += 1
    if replaced == 0:
        raise ValueError(f"Target modules {target_modules} not found in the base model.")
    return replaced

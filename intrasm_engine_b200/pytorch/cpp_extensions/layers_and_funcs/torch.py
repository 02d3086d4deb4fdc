"""``MyLinear`` — the dense branch as an autograd operator: ``input @ weight.T``.

Same arguments as intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/torch.py:6-31
(``weight`` is ``[out_features, in_features]`` as in ``torch.nn.Linear``).  fp16 inputs with
in_features a multiple of 8 run on the tcgen05 kernel, whatever the token count (blocks of
up to 256 tokens, a ragged tail padded); other dtypes (the reference's ``MyLinear`` is
dtype-agnostic, :17) are a plain library GEMM through ``torch.mm``.  The backward pass is
the reference's two matmuls (:20-31), for fp16 on the same tensor-core kernel
(``linear_fp16_dgrad`` / ``linear_fp16_wgrad``: the operands are read in their other
major-ness, no transposed copies), otherwise through ``torch.mm``.
"""
from __future__ import annotations

import torch

from .... import ops  # noqa: F401
from .utils import MyAutogradFunc, captured


def tc_linear_eligible(input: torch.Tensor, weight: torch.Tensor) -> bool:
    """fp16, any token count (the operator runs blocks of up to 256 tokens and pads a ragged
    tail), in_features a multiple of 8, 16-byte aligned contiguous operands."""
    return (input.is_cuda and input.dtype == torch.float16 and weight.dtype == torch.float16
            and input.dim() == 2 and input.size(0) > 0
            and input.size(1) % 8 == 0 and input.is_contiguous() and weight.is_contiguous()
            and input.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_forward(input, weight):
    if tc_linear_eligible(input, weight):
        return torch.ops.iex_ops.linear_fp16(input, weight)
    return input.mm(weight.t())


class MyLinear(MyAutogradFunc):
    @staticmethod
    def num_inputs(**kwargs) -> int:
        return 2

    @staticmethod
    def num_outputs(**kwargs) -> int:
        return 1

    @staticmethod
    def num_saved_tensors(**kwargs) -> int:
        return 2

    @staticmethod
    def _forward(input, weight, **kwargs):
        assert kwargs.get("num_streams", 1) == 1
        with captured(kwargs.get("constructor"), kwargs.get("stream_beg", 0),
                      kwargs.get("constructor_enabled", False)):
            output = linear_forward(input, weight)
        ctx_dict = {"backward_constructor": kwargs.get("backward_constructor"),
                    "constructor_enabled": kwargs.get("constructor_enabled", False),
                    "stream_beg": kwargs.get("stream_beg", 0),
                    "needs_input_grad": (input.requires_grad, weight.requires_grad)}
        return (output,), ctx_dict, (input, weight)

    @staticmethod
    def _backward(grad_output, input, weight, **ctx):
        need_input, need_weight = ctx.get("needs_input_grad", (True, True))
        grad_input = grad_weight = None
        with captured(ctx.get("backward_constructor"), ctx.get("stream_beg", 0),
                      ctx.get("constructor_enabled", False)):
            own = (grad_output.dtype == torch.float16 and grad_output.is_cuda and weight.dtype == torch.float16
                   and input.dtype == torch.float16 and weight.size(0) % 8 == 0 and weight.size(1) % 8 == 0)
            if own:  # both products on the tensor-core kernel, operands read as they lie
                g = grad_output.contiguous()
                if need_input:
                    grad_input = torch.ops.iex_ops.linear_fp16_dgrad(g, weight.contiguous())
                if need_weight:
                    grad_weight = torch.ops.iex_ops.linear_fp16_wgrad(g, input.contiguous())
            else:    # other dtypes: the library GEMMs, as in the reference
                if need_input:
                    grad_input = grad_output.mm(weight)
                if need_weight:
                    grad_weight = grad_output.t().mm(input)
        return grad_input, grad_weight


class MyLinearPartitioned(MyAutogradFunc):
    """Column-sharded linear: ``weight`` is cut along out_features into ``parts`` slabs, each an
    independent GEMM whose outputs are concatenated (across GPUs: one slab per rank and an
    all-gather).  Empty in the reference (torch.py:34-36)."""

    @staticmethod
    def num_inputs(**kwargs) -> int:
        return 3

    @staticmethod
    def num_outputs(**kwargs) -> int:
        return 1

    @staticmethod
    def num_saved_tensors(**kwargs) -> int:
        return 0

    @staticmethod
    def _forward(input, weight, parts, **kwargs):
        slabs = torch.chunk(weight, int(parts), dim=0)
        return (torch.cat([linear_forward(input, s.contiguous()) for s in slabs], 1),), {}, ()

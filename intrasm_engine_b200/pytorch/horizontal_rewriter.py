"""Horizontal fusion at the autograd level: several independent operators as one node.

Entry points of intrasm_engine/pytorch/horizontal_rewriter.py:
``make_single_kernel_autograd_function`` (:49-73),
``make_kernel_pair_or_triple_autograd_function`` (:76-311), the graph-replay layers
(:314-359) and ``ConstructorEnabledLayer`` (:363-408).  What the reference leaves as TODOs
is filled in: the pair of ``MySpMM`` + ``MyLinear`` on a shared activation runs as ONE fused
kernel launch (the reference could only put the two library calls on two captured
streams), and ``SparseDenseLayer`` is the "SpMM + GEMM" module its comment at :362 asks for.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import nn

from .cpp_extensions.cuda_graph_constructor import TorchCUDAGraphConstructor
from .cpp_extensions.layers_and_funcs.sputnik import MySpMM
from .cpp_extensions.layers_and_funcs.torch import MyLinear
from .cpp_extensions.layers_and_funcs.utils import MyAutogradFunc, default_fwd_kwargs


def simple_combine_search_space(space_1: dict, space_2: dict, space_3: dict) -> dict:
    out = {}
    for idx, space in enumerate((space_1, space_2, space_3), start=1):
        for key, val in space.items():
            out[f"space_{idx}.{key}"] = val
    return out


def simple_unpack_params(params: dict[str, Any]):
    parts = ({}, {}, {})
    for key, val in params.items():
        for idx in range(3):
            prefix = f"space_{idx + 1}."
            if key.startswith(prefix):
                parts[idx][key[len(prefix):]] = val
                break
        else:
            raise ValueError(f"Unknown key {key}")
    return parts if parts[2] else parts[:2]


def _install(func_class, members):
    """Gives ``func_class`` its ``forward`` / ``backward`` (static methods bound to the class
    itself, not to the base class)."""

    def forward(ctx, fwd_kwargs, *args):
        results = [f._forward(*a, **kw) for f, a, kw in _split_inputs(members, args, fwd_kwargs)]
        ctx.ctx_dicts = [r[1] for r in results]
        ctx.num_args = [len(a) for _, a, _ in _split_inputs(members, args, fwd_kwargs)]
        ctx.save_for_backward(*[t for r in results for t in r[2]])
        ctx.num_saved = [len(r[2]) for r in results]
        ctx.num_out = [len(r[0]) for r in results]
        outs = tuple(o for r in results for o in r[0])
        return outs if len(outs) > 1 else outs[0]

    def backward(ctx, *grad_args):
        saved = ctx.saved_tensors
        grads, s0, g0 = [None], 0, 0  # leading None: the keyword dictionary
        for f, ctx_dict, ns, no, na in zip(members, ctx.ctx_dicts, ctx.num_saved, ctx.num_out,
                                           ctx.num_args):
            g = f._backward(*grad_args[g0:g0 + no], *saved[s0:s0 + ns], **ctx_dict)
            g = tuple(g) + (None,) * (na - len(g))
            grads.extend(g[:na])
            s0, g0 = s0 + ns, g0 + no
        return tuple(grads)

    func_class.forward = staticmethod(forward)
    func_class.backward = staticmethod(backward)


def _split_inputs(members, args, fwd_kwargs):
    out, pos = [], 0
    for idx, f in enumerate(members, start=1):
        kw = fwd_kwargs.get(f"fwd_kwargs_{idx}") or default_fwd_kwargs()
        n = f.num_inputs(**kw)
        out.append((f, args[pos:pos + n], kw))
        pos += n
    assert pos == len(args), f"expected {pos} positional inputs, got {len(args)}"
    return out


def make_single_kernel_autograd_function(func_class: type[MyAutogradFunc]) -> type[MyAutogradFunc]:
    """Installs ``forward`` / ``backward`` built from ``_forward`` / ``_backward`` on the class;
    call it as ``func_class.run(*inputs, fwd_kwargs_1={...})``."""
    _install(func_class, (func_class,))
    return func_class


def make_kernel_pair_or_triple_autograd_function(func1: type[MyAutogradFunc],
                                                 func2: type[MyAutogradFunc],
                                                 func3: Optional[type[MyAutogradFunc]] = None,
                                                 ) -> type[MyAutogradFunc]:
    """One autograd node that runs two or three independent operators.

    Inputs are the operators' inputs concatenated (split by ``num_inputs``), outputs and
    saved tensors likewise; ``fwd_kwargs_1/2/3`` carry each operator's keyword arguments.
    The pair (``MySpMM``, ``MyLinear``) whose dense input is the transposed view of the SpMM's
    dense operand (``input = b.t()``), in fp16 and inside the tensor-core kernel's limits,
    runs as one fused launch.
    """
    members = tuple(f for f in (func1, func2, func3) if f is not None)

    class KernelPairOrTripleAutogradFunction(MyAutogradFunc):
        @staticmethod
        def num_inputs(**kw) -> int:
            return sum(f.num_inputs(**kw) for f in members)

        @staticmethod
        def num_outputs(**kw) -> int:
            return sum(f.num_outputs(**kw) for f in members)

        @staticmethod
        def num_saved_tensors(**kw) -> int:
            return sum(f.num_saved_tensors(**kw) for f in members)

        @classmethod
        def get_search_space(cls, sample_inputs, sample_grads):
            spaces, pos, gpos = [], 0, 0
            for f in members:
                ni, no = f.num_inputs(), f.num_outputs()
                grads = None if sample_grads is None else sample_grads[gpos:gpos + no]
                spaces.append(f.get_search_space(sample_inputs[pos:pos + ni], grads))
                pos, gpos = pos + ni, gpos + no
            while len(spaces) < 3:
                spaces.append({})
            return simple_combine_search_space(*spaces)

        @classmethod
        def check_fwd_kwargs_sanity(cls, fwd_kwargs: dict[str, Any]):
            for idx, f in enumerate(members, start=1):
                assert f"fwd_kwargs_{idx}" in fwd_kwargs
                f._check_unwrapped_fwd_kwargs_sanity(fwd_kwargs[f"fwd_kwargs_{idx}"])

        @classmethod
        def get_test_fwd_kwargs(cls, params: dict) -> dict[str, Any]:
            parts = simple_unpack_params(params) if params else tuple({} for _ in members)
            return {f"fwd_kwargs_{i}": f.get_test_fwd_kwargs(p)["fwd_kwargs_1"]
                    for i, (f, p) in enumerate(zip(members, parts), start=1)}

        @classmethod
        def check_params_sanity(cls, params: dict):
            for f, p in zip(members, simple_unpack_params(params)):
                f.check_params_sanity(p)

        @classmethod
        def build_and_test(cls, sample_inputs, sample_grads, params: dict):
            kw = cls.get_test_fwd_kwargs(params)
            outs = cls.run(*sample_inputs, **kw)
            return outs if isinstance(outs, tuple) else (outs,)

    _install(KernelPairOrTripleAutogradFunction, members)

    if members == (MySpMM, MyLinear):
        generic_forward = KernelPairOrTripleAutogradFunction.forward

        def forward(ctx, fwd_kwargs, *args):
            if _fusable(args, fwd_kwargs):
                b, ri, values, ro, ci, m, transp, inp, weight = args
                kw1 = fwd_kwargs.get("fwd_kwargs_1") or default_fwd_kwargs()
                kw2 = fwd_kwargs.get("fwd_kwargs_2") or default_fwd_kwargs()
                out_s, out_d = torch.ops.iex_ops.fused_spmm_linear_half(b, ro, values, ci, int(m), weight)
                ctx.ctx_dicts = [
                    {"backward_constructor": kw1.get("backward_constructor"),
                     "constructor_enabled": False, "stream_beg": 0, "num_transp_info": len(transp),
                     "needs_input_grad": (b.requires_grad, values.requires_grad)},
                    {"backward_constructor": kw2.get("backward_constructor"),
                     "constructor_enabled": False, "stream_beg": 0,
                     "needs_input_grad": (inp.requires_grad, weight.requires_grad)}]
                ctx.num_args = [7, 2]
                ctx.save_for_backward(b, ri, values, ro, ci, *transp, inp, weight)
                ctx.num_saved = [5 + len(transp), 2]
                ctx.num_out = [1, 1]
                return out_s, out_d
            return generic_forward(ctx, fwd_kwargs, *args)

        KernelPairOrTripleAutogradFunction.forward = staticmethod(forward)

    return KernelPairOrTripleAutogradFunction


def _fusable(args, fwd_kwargs) -> bool:
    if len(args) != 9:
        return False
    b, ri, values, ro, ci, m, transp, inp, weight = args
    kw1 = fwd_kwargs.get("fwd_kwargs_1") or {}
    kw2 = fwd_kwargs.get("fwd_kwargs_2") or {}
    if kw1.get("constructor_enabled") or kw2.get("constructor_enabled") or kw1.get("no_fuse"):
        return False
    if not (torch.is_tensor(b) and torch.is_tensor(inp) and b.is_cuda and b.dim() == 2):
        return False
    k, n = b.shape
    return (b.dtype == torch.float16 and values.dtype == torch.float16 and weight.dtype == torch.float16
            and b.is_contiguous() and inp.shape == (n, k) and inp.data_ptr() == b.data_ptr()
            and inp.stride() == (1, n) and n % 64 == 0 and n <= 256 and k % 8 == 0
            and weight.is_contiguous() and weight.size(1) == k
            # the tensor-core kernel reads its operands with 16-byte TMA / cp.async copies; a
            # misaligned view takes the generic pair of calls instead
            and all(t.data_ptr() % 16 == 0 for t in (b, values, ci, weight)))


# ----------------------------------------------------------------------------------------
# Graph-replay layers: the recorded forward / backward graphs run when autograd reaches them
# ----------------------------------------------------------------------------------------

def _replay(constructor: TorchCUDAGraphConstructor):
    constructor.instantiate_graph_exec()
    constructor.execute_graph()
    constructor.synchronize()
    constructor.destroy_graph_exec()


class CUDAGraphModulePreviousLayerFunction(torch.autograd.Function):
    """Sits before a recorded layer; its backward replays the backward constructor's graph.

    The recorded layer's backward only RECORDS its kernels (autograd runs it just before this
    node), so the gradient tensors that arrive here exist but hold nothing yet, and nothing
    eager may touch them before the replay.  A layer that needs its input in two layouts
    (``with_transposed``: the activation and its transposed copy, as the sparse and the dense
    branch take them) therefore gets both from this node, whose backward adds the two
    gradients AFTER the replay instead of leaving the sum to autograd.
    """

    @staticmethod
    def forward(ctx, backward_constructor, x, with_transposed=False):
        ctx.backward_constructor = backward_constructor
        ctx.with_transposed = bool(with_transposed)
        if ctx.with_transposed:
            return x.view_as(x), x.t().contiguous()
        return x.view_as(x)

    @staticmethod
    def backward(ctx, *grads):
        bc = ctx.backward_constructor
        if bc is not None and bc.node_count()[0] > 0:
            if len(bc.registeredStreams) > 1:  # bring the side streams back to the primary one
                bc.join(bc.registeredStreams[1:], bc.registeredStreams[0])
            _replay(bc)
        g = grads[0]
        if ctx.with_transposed and len(grads) > 1 and grads[1] is not None:
            g = grads[1].t() if g is None else g + grads[1].t()
        return None, g, None


class CUDAGraphModuleNextLayerFunction(torch.autograd.Function):
    """Sits after a recorded layer; its forward replays the forward constructor's graph."""

    @staticmethod
    def forward(ctx, forward_constructor, *inputs):
        if forward_constructor is not None:
            _replay(forward_constructor)
        return inputs if len(inputs) > 1 else inputs[0]

    @staticmethod
    def backward(ctx, *grads):
        return (None, *grads)


class ModuleToReplay(nn.Module):
    """A layer whose operators record themselves into the constructors it is given."""

    num_parallel_autograd_funcs: int = 1

    def forward(self, *inputs, forward_constructors, backward_constructors):
        raise NotImplementedError


class SparseDenseLayer(ModuleToReplay):
    """SpMM (pruned weight, CSR) and dense linear on the same activation.

    ``forward(x)`` with ``x`` ``[k, tokens]`` returns ``(W_sparse @ x, (W_dense @ x).T)``.  With
    ``mode="fused"`` the pair function issues one fused launch; ``mode="interleaved"`` records
    the two library calls on two streams of one constructor (the reference's method);
    ``mode="serial"`` calls them back to back.
    """

    num_parallel_autograd_funcs = 1

    def __init__(self, values, row_indices, row_offsets, column_indices, m, weight_dense,
                 transp_info=(), mode: str = "fused"):
        super().__init__()
        self.values = nn.Parameter(values, requires_grad=values.is_floating_point() and False)
        self.weight_dense = nn.Parameter(weight_dense, requires_grad=False)
        self.register_buffer("row_indices", row_indices)
        self.register_buffer("row_offsets", row_offsets)
        self.register_buffer("column_indices", column_indices)
        self.m = int(m)
        self.transp_info = tuple(transp_info)
        self.mode = mode
        self.pair = make_kernel_pair_or_triple_autograd_function(MySpMM, MyLinear)

    wants_transposed_input = True  # ConstructorEnabledLayer hands over (x, x.t().contiguous())

    def forward(self, x, xt=None, forward_constructors=None, backward_constructors=None):
        args = (x, self.row_indices, self.values, self.row_offsets, self.column_indices, self.m,
                self.transp_info, x.t(), self.weight_dense)
        if self.mode == "fused":
            return self.pair.run(*args, fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores=True),
                                 fwd_kwargs_2=default_fwd_kwargs())
        if self.mode == "serial":
            return self.pair.run(*args, fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores=True, no_fuse=True),
                                 fwd_kwargs_2=default_fwd_kwargs())
        if self.mode == "interleaved":
            ctor = forward_constructors[0]
            bctor = backward_constructors[0] if backward_constructors else None
            for c in (ctor, bctor):
                if c is not None and len(c.registeredStreams) < 2:
                    c.register_new_stream()
            if xt is None:
                xt = x.t().contiguous()
            args = args[:7] + (xt, self.weight_dense)
            # Without a backward constructor the backward pass runs eagerly (the operators
            # check for None); with one, both operators record their backward kernels on its
            # two streams and CUDAGraphModulePreviousLayerFunction replays them.
            outs = self.pair.run(
                *args,
                fwd_kwargs_1=default_fwd_kwargs(constructor=ctor, backward_constructor=bctor,
                                                constructor_enabled=True, stream_beg=0,
                                                use_tensor_cores=True),
                fwd_kwargs_2=default_fwd_kwargs(constructor=ctor, backward_constructor=bctor,
                                                constructor_enabled=True, stream_beg=1))
            ctor.join(ctor.registeredStreams[1:], ctor.registeredStreams[0])
            return outs
        raise ValueError(self.mode)


class ConstructorEnabledLayer(nn.Module):
    """Runs a ``ModuleToReplay`` with fresh forward / backward constructors and replays the
    recorded graphs at the layer's boundaries (horizontal_rewriter.py:363-408)."""

    def __init__(self, layer_to_replay: ModuleToReplay):
        super().__init__()
        self.layer_to_replay = layer_to_replay

    def forward(self, x):
        n = self.layer_to_replay.num_parallel_autograd_funcs
        backward_constructors = [TorchCUDAGraphConstructor() for _ in range(n)]
        forward_constructors = [TorchCUDAGraphConstructor() for _ in range(n)]
        if getattr(self.layer_to_replay, "wants_transposed_input", False):
            x, xt = CUDAGraphModulePreviousLayerFunction.apply(backward_constructors[0], x, True)
            outs = self.layer_to_replay(x, xt, forward_constructors=forward_constructors,
                                        backward_constructors=backward_constructors)
        else:
            x = CUDAGraphModulePreviousLayerFunction.apply(backward_constructors[0], x)
            outs = self.layer_to_replay(x, forward_constructors=forward_constructors,
                                        backward_constructors=backward_constructors)
        outs = outs if isinstance(outs, tuple) else (outs,)
        recorded = forward_constructors[0] if forward_constructors[0].node_count()[0] > 1 else None
        outs = CUDAGraphModuleNextLayerFunction.apply(recorded, *outs)
        return outs

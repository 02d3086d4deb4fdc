"""GPU: the Python operator layer — autograd classes, the pair function, the graph constructor.

Forward results are compared with the CPU oracle; gradients with torch autograd on the
dense equivalent of the same computation (fp32: rtol 1e-5 of the tensor scale).
"""
import numpy as np
import pytest
import torch

import intrasm_engine_b200  # noqa: F401
from intrasm_engine_b200 import synthetic as syn
from intrasm_engine_b200.pytorch import horizontal_rewriter as hr
from intrasm_engine_b200.pytorch import utils as U
from intrasm_engine_b200.pytorch.cpp_extensions.cuda_graph_constructor import (
    TorchCUDAGraphConstructor, combine_graphs)
from intrasm_engine_b200.pytorch.cpp_extensions.layers_and_funcs.sputnik import MySpMM, MySpMMPartitioned
from intrasm_engine_b200.pytorch.cpp_extensions.layers_and_funcs.torch import MyLinear, MyLinearPartitioned
from intrasm_engine_b200.pytorch.cpp_extensions.layers_and_funcs.utils import default_fwd_kwargs
from . import gpu_util as G

pytestmark = pytest.mark.gpu

hr.make_single_kernel_autograd_function(MySpMM)
hr.make_single_kernel_autograd_function(MyLinear)


def _scale_close(a, b, tol):
    return float((a - b).abs().max()) <= tol * max(float(b.abs().max()), 1e-30)


def test_dense_to_sparse_on_device(oracle):
    d = torch.randn(64, 96, device=G.DEV) * (torch.rand(64, 96, device=G.DEV) < 0.2)
    v, ri, ro, ci = U.dense_to_sparse(d)
    assert v.is_cuda and oracle.validate_csr(64, 96, ri.cpu().numpy(), ro.cpu().numpy(), ci.cpu().numpy()) == 0
    assert torch.equal(U.sparse_to_dense(v, ro, ci, 64, 96), d)


def test_myspmm_forward_backward_fp32(oracle):
    d = (torch.randn(80, 64, device=G.DEV) * (torch.rand(80, 64, device=G.DEV) < 0.25))
    v, ri, ro, ci = U.dense_to_sparse(d)
    info = U.get_transpose_info(80, 64, ri, ro, ci)
    b = torch.randn(64, 48, device=G.DEV, requires_grad=True)
    vals = v.clone().requires_grad_(True)
    out = MySpMM.run(b, ri, vals, ro, ci, 80, info)
    ref = oracle.spmm(ri.cpu().numpy(), v.cpu().numpy(), ro.cpu().numpy(), ci.cpu().numpy(),
                      b.detach().cpu().numpy(), 80)[0]
    np.testing.assert_array_equal(out.detach().cpu().numpy(), ref)
    g = torch.randn_like(out)
    out.backward(g)
    dd = d.clone().requires_grad_(True)
    bb = b.detach().clone().requires_grad_(True)
    (dd @ bb).backward(g)
    assert _scale_close(b.grad, bb.grad, 1e-5)
    rows = torch.repeat_interleave(torch.arange(80, device=G.DEV), (ro[1:] - ro[:-1]).long())
    assert _scale_close(vals.grad, dd.grad[rows, ci.long()], 1e-5)


def test_myspmm_fp16_and_partitioned(oracle):
    a, b = syn.pruned_sweep_case(3, 256, 512, 0.7, 128)
    da = G.DevCSR(a)
    info = U.get_transpose_info(256, 512, da.row_indices, da.row_offsets, da.column_indices)
    bd = G.dev(b)
    out = MySpMM.run(bd, da.row_indices, da.values, da.row_offsets, da.column_indices, 256, info)
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, 256)[0].astype(np.float16)
    np.testing.assert_array_equal(out.cpu().numpy(), ref)
    out_tc = MySpMM.run(bd, da.row_indices, da.values, da.row_offsets, da.column_indices, 256, info,
                        fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores=True))
    assert torch.allclose(out_tc.float(), out.float(), rtol=2e-3, atol=2e-3 * float(out.abs().max()))
    (part,), _, _ = MySpMMPartitioned._forward(bd, da.values, da.row_offsets, da.column_indices, 256, 3)
    assert torch.equal(part, out)
    # "auto": the cost model picks the tensor-core kernel for this case (30 % dense) ...
    from intrasm_engine_b200.pytorch import tuning
    assert tuning.choose_spmm_kernel(256, 512, 128, a.nnz) == "tensor_core"
    out_auto = MySpMM.run(bd, da.row_indices, da.values, da.row_offsets, da.column_indices, 256, info,
                          fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores="auto"))
    assert torch.equal(out_auto, out_tc)
    # ... and the CUDA-core kernel for a 98 % sparse one
    a2, b2 = syn.pruned_sweep_case(4, 256, 512, 0.98, 128)
    d2 = G.DevCSR(a2)
    assert tuning.choose_spmm_kernel(256, 512, 128, a2.nnz) == "cuda_core"
    info2 = U.get_transpose_info(256, 512, d2.row_indices, d2.row_offsets, d2.column_indices)
    out2 = MySpMM.run(G.dev(b2), d2.row_indices, d2.values, d2.row_offsets, d2.column_indices, 256, info2,
                      fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores="auto"))
    ref2 = oracle.spmm(a2.row_indices, a2.values, a2.row_offsets, a2.column_indices, b2, 256)[0].astype(np.float16)
    np.testing.assert_array_equal(out2.cpu().numpy(), ref2)


def test_mylinear_forward_backward():
    x = torch.randn(64, 256, device=G.DEV, dtype=torch.float16, requires_grad=True)
    w = (torch.randn(384, 256, device=G.DEV) * 0.05).half().requires_grad_(True)
    out = MyLinear.run(x, w)
    ref = x.detach().float() @ w.detach().float().t()
    assert torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-2)
    g = torch.randn_like(out)
    out.backward(g)
    assert torch.allclose(x.grad.float(), (g.float() @ w.detach().float()), rtol=2e-2, atol=2e-2)
    assert torch.allclose(w.grad.float(), (g.float().t() @ x.detach().float()), rtol=2e-2, atol=5e-2)
    (part,), _, _ = MyLinearPartitioned._forward(x.detach(), w.detach(), 4)
    assert torch.allclose(part.float(), out.float(), rtol=2e-3, atol=2e-3)
    # a shape outside the tensor-core kernel's range takes the library GEMM
    x2 = torch.randn(20, 256, device=G.DEV, dtype=torch.float16)
    assert MyLinear.run(x2, w.detach()).shape == (20, 384)


def test_pair_function_fused_equals_separate(oracle):
    a, w, x = syn.fused_layer_case(2, 384, 512, 64, 256)
    da = G.DevCSR(a)
    info = U.get_transpose_info(384, 512, da.row_indices, da.row_offsets, da.column_indices)
    xd, wd = G.dev(x), G.dev(w)
    pair = hr.make_kernel_pair_or_triple_autograd_function(MySpMM, MyLinear)
    assert pair.num_inputs() == 9 and pair.num_outputs() == 2
    args = (xd, da.row_indices, da.values, da.row_offsets, da.column_indices, 384, info, xd.t(), wd)
    assert hr._fusable(args, {})
    fs, fd = pair.run(*args, fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores=True),
                      fwd_kwargs_2=default_fwd_kwargs())
    ss, sd = pair.run(*args, fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores=True, no_fuse=True),
                      fwd_kwargs_2=default_fwd_kwargs())
    assert torch.equal(fs, ss)
    assert torch.allclose(fd.float(), sd.float(), rtol=2e-3, atol=2e-3)
    ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, 384)
    assert G.tc_close(fs.cpu().numpy(), ref_s, sabs_s)
    ref_d, sabs_d = G.linear_ref_and_sum_abs(x.T, w)
    assert G.tc_close(fd.cpu().numpy(), ref_d, sabs_d)


def test_pair_function_backward_fp32():
    d = torch.randn(48, 64, device=G.DEV) * (torch.rand(48, 64, device=G.DEV) < 0.3)
    v, ri, ro, ci = U.dense_to_sparse(d)
    info = U.get_transpose_info(48, 64, ri, ro, ci)
    b = torch.randn(64, 32, device=G.DEV, requires_grad=True)
    inp = torch.randn(32, 64, device=G.DEV, requires_grad=True)
    w = torch.randn(40, 64, device=G.DEV, requires_grad=True)
    pair = hr.make_kernel_pair_or_triple_autograd_function(MySpMM, MyLinear)
    o1, o2 = pair.run(b, ri, v, ro, ci, 48, info, inp, w)
    (o1.sum() + 2 * o2.sum()).backward()
    bb = b.detach().clone().requires_grad_(True)
    ii = inp.detach().clone().requires_grad_(True)
    ww = w.detach().clone().requires_grad_(True)
    ((d @ bb).sum() + 2 * (ii @ ww.t()).sum()).backward()
    assert _scale_close(b.grad, bb.grad, 1e-5)
    assert _scale_close(inp.grad, ii.grad, 1e-4) and _scale_close(w.grad, ww.grad, 1e-4)


def test_graph_constructor_two_streams_replay(oracle):
    """Sparse and dense library calls recorded on two streams of one graph, replayed twice."""
    a, w, x = syn.fused_layer_case(4, 256, 512, 64, 384)
    da = G.DevCSR(a)
    xd, wd, xt = G.dev(x), G.dev(w), G.dev(np.ascontiguousarray(x.T))
    ops = torch.ops.iex_ops
    ctor = TorchCUDAGraphConstructor()
    s1 = ctor.register_new_stream()
    with ctor.get_primary_stream():
        with ctor:
            out_s = ops.spmm_tc_half(xd, da.row_offsets, da.values, da.column_indices, 256)
    with s1:
        ctor.capture_library_call_begin()
        out_d = ops.linear_fp16(xt, wd)
        ctor.capture_library_call_end()
    ctor.join([s1], ctor.get_primary_stream())
    nodes, edges = ctor.node_count()
    assert nodes >= 4 and edges >= 4  # root, two kernels, join
    ctor.instantiate_graph_exec()
    for _ in range(2):
        out_s.zero_()
        out_d.zero_()
        ctor.execute_graph()
        ctor.synchronize()
        ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, 256)
        assert G.tc_close(out_s.cpu().numpy(), ref_s, sabs_s)
        ref_d, sabs_d = G.linear_ref_and_sum_abs(x.T, w)
        assert G.tc_close(out_d.cpu().numpy(), ref_d, sabs_d)
    ctor.destroy_graph_exec()
    with pytest.raises(Exception):
        ctor.execute_graph()  # no executable any more


def test_graph_constructor_events_and_combine():
    ctor = TorchCUDAGraphConstructor()
    s1 = ctor.register_new_stream()
    x = torch.ones(1024, device=G.DEV)
    y = torch.zeros(1024, device=G.DEV)
    ev = torch.cuda.Event()
    ev.record()
    with ctor.get_primary_stream():
        with ctor:
            x.mul_(2.0)
    ctor.add_event_record_node(ev, ctor.get_primary_stream().torch_stream)
    ctor.add_stream_wait_event_node(s1.torch_stream, ev)
    with s1:
        with ctor:
            y.copy_(x)
    ctor.join([s1], ctor.get_primary_stream())
    other = TorchCUDAGraphConstructor()
    z = torch.zeros(16, device=G.DEV)
    with other.get_primary_stream():
        with other:
            z.add_(1.0)
    both = combine_graphs([ctor, other])
    both.instantiate_graph_exec()
    both.execute_graph()
    both.synchronize()
    assert float(x[0]) == 2.0 and float(y[0]) == 2.0 and float(z[0]) == 1.0
    both.print_graph()


def test_sparse_dense_layer_modes(oracle):
    a, w, x = syn.fused_layer_case(6, 256, 512, 64, 256)
    da = G.DevCSR(a)
    xd, wd = G.dev(x), G.dev(w)
    outs = {}
    for mode in ("fused", "serial", "interleaved"):
        layer = hr.SparseDenseLayer(da.values, da.row_indices, da.row_offsets, da.column_indices, 256, wd,
                                    mode=mode)
        if mode == "interleaved":
            outs[mode] = hr.ConstructorEnabledLayer(layer)(xd)
        else:
            outs[mode] = layer(xd)
        torch.cuda.synchronize()
    ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, 256)
    for mode, (os_, od) in outs.items():
        assert G.tc_close(os_.cpu().numpy(), ref_s, sabs_s), mode
        assert torch.allclose(od.float(), outs["fused"][1].float(), rtol=2e-3, atol=2e-3), mode


def test_interleaved_backward_graph_matches_serial():
    """The backward kernels of the recorded layer go into the backward constructor's graph and
    are replayed by the layer in front of it; the input gradient must equal the one of the
    same layer run eagerly ("serial"), and the dense autograd reference within fp16 bounds."""
    a, w, x = syn.fused_layer_case(7, 256, 512, 64, 256)
    da = G.DevCSR(a)
    wd = G.dev(w)
    info = U.get_transpose_info(256, 512, da.row_indices, da.row_offsets, da.column_indices)
    g_s = torch.randn(256, 64, device=G.DEV).half()
    g_d = torch.randn(64, 256, device=G.DEV).half()
    grads = {}
    for mode in ("serial", "interleaved"):
        layer = hr.SparseDenseLayer(da.values, da.row_indices, da.row_offsets, da.column_indices, 256, wd,
                                    transp_info=info, mode=mode)
        xd = G.dev(x).requires_grad_(True)
        net = hr.ConstructorEnabledLayer(layer) if mode == "interleaved" else layer
        out_s, out_d = net(xd)
        torch.autograd.backward((out_s, out_d), (g_s, g_d))
        torch.cuda.synchronize()
        grads[mode] = xd.grad.clone()
    assert torch.equal(grads["interleaved"], grads["serial"])
    dense_a = torch.zeros(256, 512, device=G.DEV)
    rows = torch.repeat_interleave(torch.arange(256, device=G.DEV), (da.row_offsets[1:] - da.row_offsets[:-1]).long())
    dense_a[rows, da.column_indices.long()] = da.values.float()
    ref = dense_a.t() @ g_s.float() + (g_d.float() @ wd.float()).t()
    assert _scale_close(grads["serial"].float(), ref, 2e-3)


def test_misaligned_operands_take_the_unfused_pair():
    a, w, x = syn.fused_layer_case(8, 128, 256, 64, 128)
    da = G.DevCSR(a)
    info = ()
    xd = G.dev(x)
    wbuf = torch.empty(128 * 256 + 1, device=G.DEV, dtype=torch.float16)
    wmis = wbuf[1:].view(128, 256)
    wmis.copy_(G.dev(w))
    assert wmis.data_ptr() % 16 != 0
    args = (xd, da.row_indices, da.values, da.row_offsets, da.column_indices, 128, info, xd.t(), wmis)
    assert not hr._fusable(args, {})
    pair = hr.make_kernel_pair_or_triple_autograd_function(MySpMM, MyLinear)
    out_s, out_d = pair.run(*args, fwd_kwargs_1=default_fwd_kwargs(use_tensor_cores=True),
                            fwd_kwargs_2=default_fwd_kwargs())
    ref_d = x.astype(np.float32).T @ w.astype(np.float32).T
    assert G.close(out_d.cpu().numpy(), ref_d, 2e-3, 2e-3)

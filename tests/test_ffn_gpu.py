"""GPU parity: the ReLU-sparse FFN down projection (activation CSR x W_down) at the benchmark
shape -- 256 tokens, 11008 -> 4096, 90 % zeros, 32-bit indices -- on one GPU: the whole weight
and the 2048 / 1024 / 512-column slabs a rank holds when the weight is sharded over 2 / 4 / 8
GPUs, against torch.sparse.mm on CPU (the task's reference path); and the chain
pre-activation -> ReLU -> CSR (this library's converter) -> down projection.
"""
import numpy as np
import pytest
import torch

from intrasm_engine_b200 import _lib, synthetic as syn
from intrasm_engine_b200.pytorch.ffn import ReluSparseDownProj, relu_down_proj, split_k_parts
from . import gpu_util as G

pytestmark = pytest.mark.gpu


def _status_clean():
    torch.cuda.synchronize()
    assert _lib.lib.iex_last_device_status(1) == 0


@pytest.fixture(scope="module")
def cfg5_case(oracle):
    a, w = syn.relu_ffn_layer_case(0, 0)          # act 256 x 11008 CSR, W_down 11008 x 4096
    ref = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, w, 256)
    sabs = oracle.torch_spmm(a.row_offsets, a.column_indices, np.abs(a.values), np.abs(w), 256)
    return a, w, ref, sabs


@pytest.mark.parametrize("shards", [1, 2, 4, 8])
def test_down_proj_cfg5_slabs(cfg5_case, shards):
    """Every rank's slab of the column-sharded layer, computed one after the other on this GPU,
    reassembles to the full product."""
    a, w, ref, sabs = cfg5_case
    da = G.DevCSR(a)
    n_local = 4096 // shards
    layer = ReluSparseDownProj(256, 11008, n_local, device=G.DEV, gather="none")
    assert layer.parts == split_k_parts(n_local)
    out = np.empty((256, 4096), np.float16)
    for r in range(shards):
        slab = G.dev(np.ascontiguousarray(w[:, r * n_local:(r + 1) * n_local].T))  # [n_local, k]
        out[:, r * n_local:(r + 1) * n_local] = layer(da.values, da.row_offsets, da.column_indices, slab).cpu().numpy()
    assert G.close(out, ref, 1e-2, 1e-2)      # the task's bar
    assert G.tc_close(out, ref, sabs)         # what the arithmetic earns
    _status_clean()


def test_down_proj_int16_indices_and_small_shapes(oracle):
    for tokens, k, n, idx in ((64, 1024, 512, np.int16), (32, 520, 256, np.int32), (256, 2048, 1000, np.int16)):
        a, w = syn.relu_ffn_layer_case(1, 2, tokens, k, n, 0.1, index_dtype=idx)
        da = G.DevCSR(a)
        layer = ReluSparseDownProj(tokens, k, n, device=G.DEV, gather="none")
        got = layer(da.values, da.row_offsets, da.column_indices, G.dev(np.ascontiguousarray(w.T))).cpu().numpy()
        ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, w, tokens)
        assert G.tc_close(got, ref, sabs), (tokens, k, n)
    _status_clean()


def test_relu_to_csr_to_down_proj_chain(oracle):
    """hidden -> ReLU -> CSR on the device -> down projection equals relu(hidden) @ W on CPU."""
    rng = np.random.default_rng(12)
    tokens, k, n = 256, 11008, 1024
    hidden = rng.standard_normal((tokens, k)).astype(np.float16)
    hidden[rng.random((tokens, k)) < 0.8] -= np.float16(4.0)        # about 90 % negative
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float16)
    got = relu_down_proj(G.dev(hidden), G.dev(np.ascontiguousarray(w.T))).cpu().numpy()
    act = np.maximum(hidden.astype(np.float32), 0.0)
    assert 0.05 < (act > 0).mean() < 0.2
    a = syn.dense_to_csr(act.astype(np.float16))
    ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, w, tokens)
    assert G.tc_close(got, ref, sabs)
    _status_clean()


def test_down_proj_exact_on_small_integers(oracle):
    rng = np.random.default_rng(2)
    tokens, k, n = 256, 11008, 512
    a, _ = syn.relu_ffn_layer_case(3, 0, tokens, k, n, 0.1, with_weight=False)
    a.values[:] = rng.integers(1, 4, size=a.nnz).astype(np.float16)
    w = rng.integers(-2, 3, size=(k, n)).astype(np.float16)
    da = G.DevCSR(a)
    layer = ReluSparseDownProj(tokens, k, n, device=G.DEV, gather="none")
    got = layer(da.values, da.row_offsets, da.column_indices, G.dev(np.ascontiguousarray(w.T))).cpu().numpy()
    ref = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, w, tokens)
    assert np.abs(ref).max() < 2048
    np.testing.assert_array_equal(got, ref.astype(np.float16))
    _status_clean()

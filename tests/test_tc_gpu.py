"""GPU parity: the tensor-core (tcgen05) entry points through the C ABI.

fp16 inputs, fp32 accumulation inside the tensor core, fp16 output.  The task's bar is 1e-2
relative to the fp32 result; the tests hold the kernels to what the arithmetic earns instead
(``gpu_util.tc_close``: the final fp16 rounding plus 1e-5 of the sum of the terms'
magnitudes), so that a single dropped nonzero fails, and inputs of small integers, whose
products and sums are exact in fp16 / fp32, must match the oracle bit for bit (the method of
the reference's own graph tests, tests/test_CUDAGraphConstructor.py:75-191).  The fp32
reference is the CPU oracle / torch CPU path on the same inputs.
"""
import numpy as np
import pytest
import torch

from intrasm_engine_b200 import _lib, synthetic as syn
from . import gpu_util as G

pytestmark = pytest.mark.gpu
RTOL = 1e-2


def _linear(x, w):
    tokens, cin = x.shape
    out = torch.empty((tokens, w.shape[0]), dtype=torch.float16, device=G.DEV)
    _lib.call("iex_linear_f16", tokens, cin, w.shape[0], x.data_ptr(), w.data_ptr(), out.data_ptr(),
              G.stream_ptr())
    return out


def _spmm_tc(a, dense):
    k, n = dense.shape
    out = torch.empty((a.m, n), dtype=torch.float16, device=G.DEV)
    bits = 16 if a.column_indices.dtype == torch.int16 else 32
    _lib.call("iex_spmm_f16_tc", a.m, k, n, a.nnz, a.row_offsets.data_ptr(), G.ptr(a.column_indices), bits,
              G.ptr(a.values), dense.data_ptr(), out.data_ptr(), G.stream_ptr())
    return out


def _fused(a, w, x):
    k, n = x.shape
    out_s = torch.empty((a.m, n), dtype=torch.float16, device=G.DEV)
    out_d = torch.empty((n, w.shape[0]), dtype=torch.float16, device=G.DEV)
    bits = 16 if a.column_indices.dtype == torch.int16 else 32
    _lib.call("iex_fused_spmm_linear_f16", a.m, w.shape[0], k, n, a.nnz, a.row_offsets.data_ptr(),
              G.ptr(a.column_indices), bits, G.ptr(a.values), w.data_ptr(), x.data_ptr(), out_s.data_ptr(),
              out_d.data_ptr(), 1, G.stream_ptr())
    return out_s, out_d


def _status_clean():
    torch.cuda.synchronize()
    assert _lib.lib.iex_last_device_status(1) == 0


def test_linear_golden(oracle, golden_dir):
    g = np.load(golden_dir + "/linear_f16_16x64x48.npz")
    got = _linear(G.dev(g["input"]), G.dev(g["weight"])).cpu().numpy()
    assert G.close(got, g["out"], RTOL, RTOL)
    assert G.close(got, oracle.linear(g["input"], g["weight"]), RTOL, RTOL)
    _status_clean()


@pytest.mark.parametrize("tokens,cin,cout", [(16, 8, 8), (16, 64, 128), (64, 128, 128), (64, 256, 384),
                                             (32, 520, 200), (128, 1024, 1000), (256, 328, 640),
                                             (48, 4096, 256), (64, 4096, 12288),
                                             # 128 tokens and more: 64- and 96-KB stages, two-deep ring
                                             # (even, odd and single tile counts)
                                             (128, 512, 512), (192, 776, 384), (256, 2048, 1000),
                                             (256, 11008, 640), (256, 64, 128), (144, 1024, 300)])
def test_linear_shapes(tokens, cin, cout):
    rng = np.random.default_rng(tokens + cin + cout)
    x = rng.standard_normal((tokens, cin)).astype(np.float16)
    w = (rng.standard_normal((cout, cin)) * 0.05).astype(np.float16)
    got = _linear(G.dev(x), G.dev(w)).cpu().numpy()
    ref, sabs = G.linear_ref_and_sum_abs(x, w)
    assert G.close(got, ref, RTOL, RTOL), G.max_violation(got, ref, RTOL, RTOL)
    assert G.tc_close(got, ref, sabs)  # fp16 rounding only
    _status_clean()


@pytest.mark.parametrize("tokens", [16, 48, 144])
def test_linear_writes_nothing_past_the_output(tokens):
    """Token counts that are not a multiple of the 32 accumulator columns read at a time: the
    rows after the output (here a guard region of the same buffer) stay untouched."""
    rng = np.random.default_rng(tokens)
    cin, cout = 256, 384
    x = G.dev(rng.standard_normal((tokens, cin)).astype(np.float16))
    w = G.dev((rng.standard_normal((cout, cin)) * 0.05).astype(np.float16))
    buf = torch.full((tokens + 32, cout), 7.0, dtype=torch.float16, device=G.DEV)
    _lib.call("iex_linear_f16", tokens, cin, cout, x.data_ptr(), w.data_ptr(), buf.data_ptr(), G.stream_ptr())
    ref = x.float() @ w.float().t()
    assert torch.allclose(buf[:tokens].float(), ref, rtol=1e-2, atol=1e-2)
    assert bool((buf[tokens:] == 7.0).all())
    _status_clean()


@pytest.mark.parametrize("tokens,cin,cout", [(64, 4096, 512), (256, 11008, 1024), (48, 4096, 512), (64, 256, 384)])
def test_linear_op_splits_few_tile_weights(tokens, cin, cout):
    """torch.ops.iex_ops.linear_fp16 spreads a weight of few 128-row tiles over the SMs by
    itself (split-K with a scratch tensor from the caching allocator) where the shape allows;
    either way the result is the product."""
    rng = np.random.default_rng(tokens + cout)
    x = G.dev(rng.standard_normal((tokens, cin)).astype(np.float16))
    w = G.dev((rng.standard_normal((cout, cin)) * 0.05).astype(np.float16))
    out = torch.ops.iex_ops.linear_fp16(x, w)
    ref = x.float() @ w.float().t()
    assert torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-2 * float(ref.abs().max()))
    assert torch.allclose(out.float(), _linear(x, w).float(), rtol=2e-3, atol=2e-3 * float(ref.abs().max()))
    _status_clean()


@pytest.mark.parametrize("seed", range(32))
def test_linear_random_shapes(seed):
    """Seeded random shapes for the dense linear, plain and split-K (workspace and built-in
    scratch), against the fp32 product."""
    rng = np.random.default_rng(300 + seed)
    tokens = int(rng.integers(1, 17)) * 16
    cin = int(rng.integers(1, 400)) * 8
    cout = int(rng.integers(1, 1500))
    x = G.dev(rng.standard_normal((tokens, cin)).astype(np.float16))
    w = G.dev((rng.standard_normal((cout, cin)) * 0.05).astype(np.float16))
    ref = (x.float() @ w.float().t()).cpu().numpy()
    sabs = (x.float().abs() @ w.float().abs().t()).cpu().numpy()
    got = _linear(x, w)
    assert G.tc_close(got.cpu().numpy(), ref, sabs), (tokens, cin, cout)
    if tokens % 32 == 0:
        parts = int(rng.integers(2, 9))
        need = _lib.lib.iex_tc_workspace_bytes(0, 1, cout, parts, tokens)
        ws = _workspace(need)
        out = torch.zeros((tokens, cout), dtype=torch.float16, device=G.DEV)
        _lib.call("iex_linear_f16_splitk", tokens, cin, cout, x.data_ptr(), w.data_ptr(), out.data_ptr(),
                  parts, ws.data_ptr(), ws.numel(), G.stream_ptr())
        assert G.tc_close(out.cpu().numpy(), ref, sabs), (tokens, cin, cout, parts)
        if need <= _lib.lib.iex_static_workspace_capacity():
            out2 = torch.zeros_like(out)
            _lib.call("iex_linear_f16_splitk_static", tokens, cin, cout, x.data_ptr(), w.data_ptr(),
                      out2.data_ptr(), parts, G.stream_ptr())
            assert torch.equal(out2, out)
    _status_clean()


def test_linear_rejects_unsupported():
    x = torch.zeros((20, 64), dtype=torch.float16, device=G.DEV)
    w = torch.zeros((64, 64), dtype=torch.float16, device=G.DEV)
    with pytest.raises(_lib.IexError) as e:
        _linear(x, w)  # tokens not a multiple of 16
    assert e.value.status == -2
    x = torch.zeros((512, 64), dtype=torch.float16, device=G.DEV)
    with pytest.raises(_lib.IexError):
        _linear(x, w)  # tokens > 256


@pytest.mark.parametrize("m,k,n,density,idx", [
    (128, 128, 64, 0.5, np.int16), (1, 8, 64, 1.0, np.int16), (130, 264, 64, 0.5, np.int32),
    (300, 1024, 64, 0.3, np.int16), (256, 512, 128, 0.1, np.int32), (256, 512, 128, 0.9, np.int16),
    (64, 2048, 64, 1.0, np.int16), (200, 640, 64, 0.0, np.int16), (512, 4096, 64, 0.02, np.int16),
    (1024, 2048, 128, 0.5, np.int16),
])
def test_spmm_tc_shapes(oracle, m, k, n, density, idx):
    rng = np.random.default_rng(m * 7 + k + n)
    mask = rng.random((m, k)) < density
    if density > 0:
        mask[0] = True        # a fully dense row exercises the long-run path
        mask[m // 2] = False  # and an empty one
    a = syn.csr_from_mask(mask, rng=rng, std=0.05, dtype=np.float16, index_dtype=idx)
    b = rng.standard_normal((k, n)).astype(np.float16)
    got = _spmm_tc(G.DevCSR(a), G.dev(b)).cpu().numpy()
    ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, b, m)
    assert G.close(got, ref, RTOL, RTOL), G.max_violation(got, ref, RTOL, RTOL)
    assert G.tc_close(got, ref, sabs)
    _status_clean()


@pytest.mark.parametrize("m,k,n,idx", [(300, 520, 64, np.int16), (1100, 1024, 128, np.int32)])
def test_spmm_tc_bias_relu(oracle, m, k, n, idx):
    """Bias + ReLU epilogue of the tensor-core SpMM against the oracle's (fp32 bias per row)."""
    rng = np.random.default_rng(m + n)
    mask = rng.random((m, k)) < 0.3
    a = syn.csr_from_mask(mask, rng=rng, std=0.05, dtype=np.float16, index_dtype=idx)
    b = rng.standard_normal((k, n)).astype(np.float16)
    bias = rng.standard_normal(m).astype(np.float32)
    da = G.DevCSR(a)
    db, dbias = G.dev(b), G.dev(bias)  # kept alive: the calls below are asynchronous
    out = torch.empty((m, n), dtype=torch.float16, device=G.DEV)
    _lib.call("iex_spmm_f16_tc_bias_relu", m, k, n, a.nnz, da.row_offsets.data_ptr(), da.column_indices.data_ptr(),
              16 if idx == np.int16 else 32, da.values.data_ptr(), db.data_ptr(), dbias.data_ptr(),
              out.data_ptr(), G.stream_ptr())
    ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, b, m, bias=bias)
    got = out.cpu().numpy()
    assert G.tc_close(got, ref, sabs), G.max_violation(got, ref, RTOL, RTOL)
    assert (got >= 0).all() and (got == 0).any()
    # no bias pointer: the plain product
    _lib.call("iex_spmm_f16_tc_bias_relu", m, k, n, a.nnz, da.row_offsets.data_ptr(), da.column_indices.data_ptr(),
              16 if idx == np.int16 else 32, da.values.data_ptr(), db.data_ptr(), None, out.data_ptr(),
              G.stream_ptr())
    assert torch.equal(out, _spmm_tc(da, db))
    _status_clean()


@pytest.mark.parametrize("seed", range(48))
def test_spmm_tc_random_shapes(oracle, seed):
    """Seeded random shapes and row patterns for the tensor-core SpMM and the fused launch:
    rows that are empty, nearly empty, half full or full in one matrix, K that is not a multiple
    of the 64-column slots, every token count and both index widths."""
    rng = np.random.default_rng(1000 + seed)
    m = int(rng.integers(1, 700))
    k = int(rng.integers(1, 257)) * 8
    n = int(rng.choice([64, 128, 192, 256]))
    idx = np.int16 if rng.random() < 0.5 else np.int32
    row_density = rng.choice([0.0, 0.01, 0.1, 0.5, 1.0], size=m, p=[0.1, 0.2, 0.3, 0.3, 0.1])
    mask = rng.random((m, k)) < row_density[:, None]
    a = syn.csr_from_mask(mask, rng=rng, std=0.05, dtype=np.float16, index_dtype=idx)
    b = rng.standard_normal((k, n)).astype(np.float16)
    da, db = G.DevCSR(a), G.dev(b)
    got = _spmm_tc(da, db)
    ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, b, m)
    assert G.tc_close(got.cpu().numpy(), ref, sabs), (m, k, n, idx)
    if seed % 3 == 0:  # the same sparse matrix beside a dense one in the fused launch
        md = int(rng.integers(1, 40)) * 8
        w = (rng.standard_normal((md, k)) * 0.05).astype(np.float16)
        out_s, out_d = _fused(da, G.dev(w), db)
        assert torch.equal(out_s, got)
        ref_d, sabs_d = G.linear_ref_and_sum_abs(b.T, w)
        assert G.tc_close(out_d.cpu().numpy(), ref_d, sabs_d), (m, md, k, n)
    _status_clean()


def test_spmm_tc_matches_cuda_core_kernel():
    """Two independent kernels (CUDA cores, bit-exact with the oracle; tensor cores) agree."""
    a, b = syn.pruned_sweep_case(7, 2048, 512, 0.7, 128)
    da = G.DevCSR(a)
    simt = G.spmm_f16(da, G.dev(b)[None])[0].float()
    tc = _spmm_tc(da, G.dev(b)).float()
    assert torch.allclose(simt, tc, rtol=2e-3, atol=2e-3 * float(simt.abs().max()))
    _status_clean()


def test_spmm_tc_rejects_unsupported():
    a, b = syn.pruned_sweep_case(1, 64, 128, 0.5, 64)
    da = G.DevCSR(a)
    with pytest.raises(_lib.IexError):
        _spmm_tc(da, G.dev(b[:, :48].copy()))  # n not a multiple of 64
    with pytest.raises(_lib.IexError):
        _lib.call("iex_spmm_f16_tc", 64, 128, 64, a.nnz, da.row_offsets.data_ptr(), da.column_indices.data_ptr(),
                  8, da.values.data_ptr(), G.dev(b).data_ptr(), G.dev(b).data_ptr(), None)


@pytest.mark.parametrize("ms,md,k,n", [(256, 256, 512, 64), (100, 300, 264, 64), (384, 128, 1024, 128),
                                        (128, 0, 256, 64), (0, 256, 256, 64)])
def test_fused_small(oracle, ms, md, k, n):
    a, w, x = syn.fused_layer_case(ms + md, max(ms, 1), k, n, max(md, 1))
    if ms == 0:
        a = syn.csr_from_mask(np.zeros((0, k), bool), rng=np.random.default_rng(0), dtype=np.float16,
                              index_dtype=np.int16)
    if md == 0:
        w = w[:0]
    da = G.DevCSR(a)
    dw = G.dev(w) if md else torch.zeros((0, k), dtype=torch.float16, device=G.DEV)
    out_s, out_d = _fused(da, dw, G.dev(x))
    if ms:
        ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, ms)
        assert G.tc_close(out_s.cpu().numpy(), ref_s, sabs_s)
    if md:
        ref_d, sabs_d = G.linear_ref_and_sum_abs(x.T, w)
        assert G.tc_close(out_d.cpu().numpy(), ref_d, sabs_d)
    _status_clean()


@pytest.mark.parametrize("ms,md,k,n,idx", [
    (15360, 15360, 264, 64, np.int16),   # 120 + 120 units on 148 CTAs: 64 CTAs run a dense unit, then a sparse one
    (25664, 128, 256, 64, np.int32),     # 201 sparse units: CTAs run two sparse units back to back
    (2048, 20480, 192, 128, np.int16),   # three waves, dense before and after the sparse units
])
def test_fused_more_units_than_ctas(oracle, ms, md, k, n, idx):
    """CTAs that take several units, of one kind or of both (the two kinds lay shared memory
    out differently, so a CTA that changes kind waits for its previous unit to finish)."""
    rng = np.random.default_rng(ms + md)
    mask = rng.random((ms, k)) < 0.4
    mask[0] = True
    mask[ms // 2] = False
    a = syn.csr_from_mask(mask, rng=rng, std=0.05, dtype=np.float16, index_dtype=idx)
    w = (rng.standard_normal((md, k)) * 0.05).astype(np.float16)
    x = rng.standard_normal((k, n)).astype(np.float16)
    da = G.DevCSR(a)
    out_s, out_d = _fused(da, G.dev(w), G.dev(x))
    ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, ms)
    ref_d, sabs_d = G.linear_ref_and_sum_abs(x.T, w)
    assert G.tc_close(out_s.cpu().numpy(), ref_s, sabs_s)
    assert G.tc_close(out_d.cpu().numpy(), ref_d, sabs_d)
    # same bits from the sparse launch alone and from a second fused launch
    assert torch.equal(_spmm_tc(da, G.dev(x)), out_s)
    again_s, again_d = _fused(da, G.dev(w), G.dev(x))
    assert torch.equal(again_s, out_s) and torch.equal(again_d, out_d)
    _status_clean()


@pytest.mark.parametrize("n", [192, 256])
@pytest.mark.parametrize("idx", [np.int16, np.int32])
def test_spmm_tc_wide_n(oracle, n, idx):
    """Token counts whose B slots leave room for fewer A slots (other shared-memory plans)."""
    rng = np.random.default_rng(n)
    m, k = 300, 1160
    mask = rng.random((m, k)) < 0.25
    mask[3] = True
    a = syn.csr_from_mask(mask, rng=rng, std=0.05, dtype=np.float16, index_dtype=idx)
    b = rng.standard_normal((k, n)).astype(np.float16)
    got = _spmm_tc(G.DevCSR(a), G.dev(b)).cpu().numpy()
    ref, sabs = G.spmm_ref_and_sum_abs(oracle, a, b, m)
    assert G.tc_close(got, ref, sabs), G.max_violation(got, ref, RTOL, RTOL)
    _status_clean()


def test_fused_cfg4_full_size(oracle):
    """Benchmark configuration 4: W_up 11008x4096 CSR at 50 % times X 4096x64, fused with W_qkv 12288x4096."""
    a, w, x = syn.fused_layer_case(0)
    da = G.DevCSR(a)
    out_s, out_d = _fused(da, G.dev(w), G.dev(x))
    ref_s = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, x, 11008)
    sabs_s = oracle.torch_spmm(a.row_offsets, a.column_indices, np.abs(a.values), np.abs(x), 11008)
    ref_d = oracle.torch_linear(x.T, w)
    sabs_d = oracle.torch_linear(np.abs(x.T), np.abs(w))
    gs, gd = out_s.cpu().numpy(), out_d.cpu().numpy()
    assert G.close(gs, ref_s, RTOL, RTOL), G.max_violation(gs, ref_s, RTOL, RTOL)
    assert G.close(gd, ref_d, RTOL, RTOL), G.max_violation(gd, ref_d, RTOL, RTOL)
    assert G.tc_close(gs, ref_s, sabs_s) and G.tc_close(gd, ref_d, sabs_d)
    # the fused launch and the two separate launches give identical bits
    sep_s = _spmm_tc(da, G.dev(x))
    sep_d = _linear(G.dev(np.ascontiguousarray(x.T)), G.dev(w))
    assert torch.equal(sep_s, out_s)
    assert torch.allclose(sep_d.float(), out_d.float(), rtol=2e-3, atol=2e-3)
    # int32 indices: same values
    da.column_indices = da.column_indices.to(torch.int32)
    out_s32, _ = _fused(da, G.dev(w), G.dev(x))
    assert torch.equal(out_s32, out_s)
    _status_clean()


def test_torch_ops_tc(oracle):
    import intrasm_engine_b200  # noqa: F401
    ops = torch.ops.iex_ops
    a, w, x = syn.fused_layer_case(5, 256, 512, 64, 384)
    da = G.DevCSR(a)
    xs, ws = G.dev(x), G.dev(w)
    out_s, out_d = ops.fused_spmm_linear_half(xs, da.row_offsets, da.values, da.column_indices, 256, ws)
    assert torch.equal(out_s, ops.spmm_tc_half(xs, da.row_offsets, da.values, da.column_indices, 256))
    lin = ops.linear_fp16(xs.t().contiguous(), ws)
    assert lin.shape == out_d.shape
    assert torch.allclose(lin.float(), out_d.float(), rtol=2e-3, atol=2e-3)
    ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, 256)
    assert G.tc_close(out_s.cpu().numpy(), ref_s, sabs_s)
    with pytest.raises(RuntimeError):
        ops.linear_fp16(xs.t().contiguous().float(), ws)
    # a shape the kernel family refuses at launch time surfaces as a Python error too
    with pytest.raises(RuntimeError, match="not supported"):
        ops.spmm_tc_half(xs[:, :48].contiguous(), da.row_offsets, da.values, da.column_indices, 256)
    # more tokens than one kernel launch takes, and a ragged count: blocks of 256 + a padded tail
    xl = torch.randn(600 + 7, 512, device=G.DEV).half()
    big = ops.linear_fp16(xl, ws)
    ref = xl.float() @ ws.float().t()
    assert big.shape == (607, 384)
    assert torch.allclose(big.float(), ref, rtol=2e-3, atol=2e-3 * float(ref.abs().max()))


# ----------------------------------------------------------------------------------------
# split-K entry points (fp32 partial tiles in a caller-provided workspace + reduce kernel)
# ----------------------------------------------------------------------------------------

def _workspace(nbytes):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=G.DEV)


@pytest.mark.parametrize("tokens,cin,cout,parts", [(64, 4096, 2048, 4), (32, 1024, 1000, 3), (256, 2048, 512, 8),
                                                   (64, 256, 128, 16), (128, 640, 384, 2),
                                                   (256, 11008, 1024, 16), (192, 1000, 640, 5)])
def test_linear_splitk(tokens, cin, cout, parts):
    rng = np.random.default_rng(tokens + cin + cout)
    x = G.dev(rng.standard_normal((tokens, cin)).astype(np.float16))
    w = G.dev((rng.standard_normal((cout, cin)) * 0.05).astype(np.float16))
    ref = x.float() @ w.float().t()
    sabs = (x.float().abs() @ w.float().abs().t()).cpu().numpy()
    need = _lib.lib.iex_tc_workspace_bytes(0, 1, cout, parts, tokens)
    ws = _workspace(need)
    out = torch.zeros((tokens, cout), dtype=torch.float16, device=G.DEV)
    for _ in range(2):  # the workspace is reusable without clearing
        _lib.call("iex_linear_f16_splitk", tokens, cin, cout, x.data_ptr(), w.data_ptr(), out.data_ptr(),
                  parts, ws.data_ptr(), ws.numel(), G.stream_ptr())
        assert G.tc_close(out.cpu().numpy(), ref.cpu().numpy(), sabs)
    assert torch.allclose(out.float(), _linear(x, w).float(), rtol=2e-3, atol=2e-3 * float(ref.abs().max()))
    if need > 256 and parts <= (cin + 127) // 128:  # the kernel never uses more parts than k-blocks
        with pytest.raises(_lib.IexError) as e:
            _lib.call("iex_linear_f16_splitk", tokens, cin, cout, x.data_ptr(), w.data_ptr(), out.data_ptr(),
                      parts, ws.data_ptr(), need - 1, G.stream_ptr())
        assert e.value.status == -3
    _status_clean()


@pytest.mark.parametrize("parts", [2, 3, 5])
def test_spmm_tc_and_fused_splitk(oracle, parts):
    a, w, x = syn.fused_layer_case(11, 640, 1024, 64, 384)
    da = G.DevCSR(a)
    xd, wd = G.dev(x), G.dev(w)
    ref_s, sabs_s = G.spmm_ref_and_sum_abs(oracle, a, x, 640)
    ref_d, sabs_d = G.linear_ref_and_sum_abs(x.T, w)
    ws = _workspace(_lib.lib.iex_tc_workspace_bytes(640, parts, 384, 2, 64))
    out_s = torch.zeros((640, 64), dtype=torch.float16, device=G.DEV)
    _lib.call("iex_spmm_f16_tc_splitk", 640, 1024, 64, a.nnz, da.row_offsets.data_ptr(), da.column_indices.data_ptr(),
              16, da.values.data_ptr(), xd.data_ptr(), out_s.data_ptr(), parts, ws.data_ptr(), ws.numel(),
              G.stream_ptr())
    assert G.tc_close(out_s.cpu().numpy(), ref_s, sabs_s)
    first = out_s.clone()
    out_s.zero_()
    out_d = torch.zeros((64, 384), dtype=torch.float16, device=G.DEV)
    _lib.call("iex_fused_spmm_linear_f16_splitk", 640, 384, 1024, 64, a.nnz, da.row_offsets.data_ptr(),
              da.column_indices.data_ptr(), 16, da.values.data_ptr(), wd.data_ptr(), xd.data_ptr(),
              out_s.data_ptr(), out_d.data_ptr(), 1, parts, 2, ws.data_ptr(), ws.numel(), G.stream_ptr())
    assert torch.equal(out_s, first)  # parts are added in part order: same bits in either launch
    assert G.tc_close(out_d.cpu().numpy(), ref_d, sabs_d)
    _status_clean()


@pytest.mark.parametrize("m,k,idx", [(256, 11008, np.int32), (33, 100, np.int16), (5, 7, np.int32),
                                     (2000, 520, np.int16), (64, 4096, np.int16), (1, 8, np.int32),
                                     (300, 2056, np.int32)])
def test_csr_to_dense(m, k, idx):
    """Shapes on both sides of every split the kernel makes: more rows than resident CTAs, one
    to eight column slices per row, k with and without the 8-column alignment of the vector
    stores, rows that are empty, full and longer than a block's first pass."""
    rng = np.random.default_rng(m + k)
    mask = rng.random((m, k)) < 0.1
    mask[0] = True
    mask[m // 2] = False
    a = syn.csr_from_mask(mask, rng=rng, std=1.0, dtype=np.float16, index_dtype=idx)
    da = G.DevCSR(a)
    out = torch.full((m, k), 7.0, dtype=torch.float16, device=G.DEV)
    _lib.call("iex_csr_to_dense_f16", m, k, da.row_offsets.data_ptr(), G.ptr(da.column_indices),
              16 if idx == np.int16 else 32, G.ptr(da.values), out.data_ptr(), G.stream_ptr())
    np.testing.assert_array_equal(out.cpu().numpy(), a.to_dense())


# ----------------------------------------------------------------------------------------
# Exact cases: small-integer inputs.  Every product and every partial sum is an integer far
# below 2^24 and every result below 2^11, so fp32 accumulation in any order and the final
# fp16 conversion are exact: the tensor-core kernels must match the oracle bit for bit.
# ----------------------------------------------------------------------------------------

def _int_csr(rng, m, k, density, idx, lo=-2, hi=3):
    mask = rng.random((m, k)) < density
    a = syn.csr_from_mask(mask, rng=rng, std=1.0, dtype=np.float16, index_dtype=idx)
    a.values[:] = rng.integers(lo, hi, size=a.nnz).astype(np.float16)
    return a


@pytest.mark.parametrize("m,k,n,density,idx", [(300, 1024, 64, 0.3, np.int16), (513, 2048, 128, 0.5, np.int32),
                                               (128, 520, 256, 0.05, np.int16), (1000, 264, 192, 0.9, np.int32)])
def test_spmm_tc_exact_on_small_integers(oracle, m, k, n, density, idx):
    rng = np.random.default_rng(m + k + n)
    a = _int_csr(rng, m, k, density, idx)
    b = rng.integers(-3, 4, size=(k, n)).astype(np.float16)
    da, db = G.DevCSR(a), G.dev(b)
    ref = oracle.spmm(a.row_indices, a.values, a.row_offsets, a.column_indices, b, m)[0]
    assert np.abs(ref).max() < 2048
    np.testing.assert_array_equal(_spmm_tc(da, db).cpu().numpy(), ref.astype(np.float16))
    ws = _workspace(_lib.lib.iex_tc_workspace_bytes(m, 3, 0, 1, n))
    out = torch.zeros((m, n), dtype=torch.float16, device=G.DEV)
    _lib.call("iex_spmm_f16_tc_splitk", m, k, n, a.nnz, da.row_offsets.data_ptr(), da.column_indices.data_ptr(),
              16 if idx == np.int16 else 32, da.values.data_ptr(), db.data_ptr(), out.data_ptr(), 3,
              ws.data_ptr(), ws.numel(), G.stream_ptr())
    np.testing.assert_array_equal(out.cpu().numpy(), ref.astype(np.float16))
    _status_clean()


@pytest.mark.parametrize("tokens,cin,cout,parts", [(64, 1024, 384, 1), (256, 2048, 1000, 4), (32, 520, 200, 3),
                                                   (128, 4096, 512, 8)])
def test_linear_exact_on_small_integers(tokens, cin, cout, parts):
    rng = np.random.default_rng(tokens + cin + cout)
    x = rng.integers(-3, 4, size=(tokens, cin)).astype(np.float16)
    w = rng.integers(-2, 3, size=(cout, cin)).astype(np.float16)
    ref = x.astype(np.float32) @ w.astype(np.float32).T
    assert np.abs(ref).max() < 2048
    dx, dw = G.dev(x), G.dev(w)
    np.testing.assert_array_equal(_linear(dx, dw).cpu().numpy(), ref.astype(np.float16))
    ws = _workspace(_lib.lib.iex_tc_workspace_bytes(0, 1, cout, parts, tokens))
    out = torch.zeros((tokens, cout), dtype=torch.float16, device=G.DEV)
    _lib.call("iex_linear_f16_splitk", tokens, cin, cout, dx.data_ptr(), dw.data_ptr(), out.data_ptr(), parts,
              ws.data_ptr(), ws.numel(), G.stream_ptr())
    np.testing.assert_array_equal(out.cpu().numpy(), ref.astype(np.float16))
    _status_clean()


def test_fused_exact_on_small_integers_cfg4_shape(oracle):
    """The benchmark's fused layer shape (W_up 11008x4096 at 50 %, W_qkv 12288x4096, 64 tokens)
    with small-integer weights and activations: both outputs bit-exact."""
    rng = np.random.default_rng(44)
    ms, md, k, n = 11008, 12288, 4096, 64
    a = _int_csr(rng, ms, k, 0.5, np.int16, lo=-1, hi=2)
    w = rng.integers(-1, 2, size=(md, k)).astype(np.float16)
    x = rng.integers(-2, 3, size=(k, n)).astype(np.float16)
    out_s, out_d = _fused(G.DevCSR(a), G.dev(w), G.dev(x))
    ref_s = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, x, ms)
    ref_d = oracle.torch_linear(x.T, w)
    assert max(np.abs(ref_s).max(), np.abs(ref_d).max()) < 2048
    np.testing.assert_array_equal(out_s.cpu().numpy(), ref_s.astype(np.float16))
    np.testing.assert_array_equal(out_d.cpu().numpy(), ref_d.astype(np.float16))
    _status_clean()


# ----------------------------------------------------------------------------------------
# Backward of the dense branch: dgrad = grad @ W and wgrad = grad^T @ X on the tensor-core
# kernel (A operand MN-major; wgrad also B MN-major over blocks of 256 columns)
# ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("tokens,cin,cout", [(64, 256, 384), (16, 8, 8), (256, 1024, 1000), (128, 4096, 512),
                                             (48, 520, 200), (64, 4096, 12288), (256, 200, 136)])
def test_linear_dgrad_wgrad(tokens, cin, cout):
    rng = np.random.default_rng(tokens + cin + cout)
    x = rng.standard_normal((tokens, cin)).astype(np.float16)
    w = (rng.standard_normal((cout, cin)) * 0.05).astype(np.float16)
    g = rng.standard_normal((tokens, cout)).astype(np.float16)
    dx, dw = G.dev(x), G.dev(w)
    dg = G.dev(g)
    dinput = torch.full((tokens, cin), 9.0, dtype=torch.float16, device=G.DEV)
    dweight = torch.full((cout, cin), 9.0, dtype=torch.float16, device=G.DEV)
    _lib.call("iex_linear_f16_dgrad", tokens, cin, cout, dg.data_ptr(), dw.data_ptr(), dinput.data_ptr(), G.stream_ptr())
    _lib.call("iex_linear_f16_wgrad", tokens, cin, cout, dg.data_ptr(), dx.data_ptr(), dweight.data_ptr(), G.stream_ptr())
    ref_i, sabs_i = G.linear_ref_and_sum_abs(g, w.T)
    ref_w, sabs_w = G.linear_ref_and_sum_abs(g.T, x.T)
    assert G.tc_close(dinput.cpu().numpy(), ref_i, sabs_i)
    assert G.tc_close(dweight.cpu().numpy(), ref_w, sabs_w)
    _status_clean()


def test_linear_backward_exact_on_small_integers_and_ops():
    rng = np.random.default_rng(77)
    tokens, cin, cout = 72 + 256, 520, 392      # ragged token count through the operators
    x = rng.integers(-2, 3, size=(tokens, cin)).astype(np.float16)
    w = rng.integers(-2, 3, size=(cout, cin)).astype(np.float16)
    g = rng.integers(-2, 3, size=(tokens, cout)).astype(np.float16)
    ops = torch.ops.iex_ops
    di = ops.linear_fp16_dgrad(G.dev(g), G.dev(w)).cpu().numpy()
    dw = ops.linear_fp16_wgrad(G.dev(g), G.dev(x)).cpu().numpy()
    ref_i = g.astype(np.float32) @ w.astype(np.float32)
    ref_w = g.astype(np.float32).T @ x.astype(np.float32)
    assert max(np.abs(ref_i).max(), np.abs(ref_w).max()) < 2048
    np.testing.assert_array_equal(di, ref_i.astype(np.float16))
    np.testing.assert_array_equal(dw, ref_w.astype(np.float16))
    _status_clean()

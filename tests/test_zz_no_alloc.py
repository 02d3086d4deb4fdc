"""GPU: the allocation-free split-K linear (collected last on purpose).

``iex_linear_f16_splitk_static`` is for hosts that must not allocate device memory while
they run — a serving process or plugin host with a memory budget fixed at start-up, where a
late ``cudaMalloc`` would synchronise the device or fail on a fragmented heap.  Its partial
tiles live in an 8 MiB array inside the library instead of a caller workspace.  The test
calls it through the C ABI twice in a row and checks both results against
``iex_linear_f16_splitk`` with an ordinary workspace: the two entry points run the same
kernels, so the outputs must be bit-identical, and the second call must not be disturbed by
what the first left in the shared array.
"""
import numpy as np
import pytest
import torch

from intrasm_engine_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_pair(tokens, cin, cout, parts, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, cin, generator=g).half().to(DEV)
    w = (torch.randn(cout, cin, generator=g) * 0.05).half().to(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    need = _lib.lib.iex_tc_workspace_bytes(0, 1, cout, parts, tokens)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=DEV)
    ref = torch.zeros((tokens, cout), dtype=torch.float16, device=DEV)
    _lib.call("iex_linear_f16_splitk", tokens, cin, cout, x.data_ptr(), w.data_ptr(), ref.data_ptr(), parts,
              ws.data_ptr(), ws.numel(), stream)
    got = torch.zeros_like(ref)
    _lib.call("iex_linear_f16_splitk_static", tokens, cin, cout, x.data_ptr(), w.data_ptr(), got.data_ptr(),
              parts, stream)
    torch.cuda.synchronize()
    return got, ref, x, w


def test_static_workspace_two_calls_in_a_row():
    assert _lib.lib.iex_static_workspace_capacity() == 8 << 20
    # two different problems back to back: the second overwrites the first one's partial tiles
    got1, ref1, x1, w1 = _run_pair(64, 4096, 2048, 4, seed=1)
    got2, ref2, x2, w2 = _run_pair(128, 1024, 1000, 3, seed=2)
    assert torch.equal(got1, ref1)
    assert torch.equal(got2, ref2)
    for got, x, w in ((got1, x1, w1), (got2, x2, w2)):
        exact = x.float() @ w.float().t()
        tol = 1e-2 * float(exact.abs().max())
        assert float((got.float() - exact).abs().max()) <= tol
    assert _lib.lib.iex_last_device_status(1) == 0


def test_static_workspace_rejects_oversize():
    x = torch.zeros((256, 4096), dtype=torch.float16, device=DEV)
    w = torch.zeros((8192, 4096), dtype=torch.float16, device=DEV)
    out = torch.zeros((256, 8192), dtype=torch.float16, device=DEV)
    # 64 tiles * 8 parts * 128 * 256 * 4 bytes = 64 MiB > 8 MiB
    with pytest.raises(_lib.IexError) as e:
        _lib.call("iex_linear_f16_splitk_static", 256, 4096, 8192, x.data_ptr(), w.data_ptr(), out.data_ptr(),
                  8, torch.cuda.current_stream().cuda_stream)
    assert e.value.status == -3 and "exceeds" in str(e.value)
    # parts = 1 needs no scratch at all and is accepted at any size
    _lib.call("iex_linear_f16_splitk_static", 256, 4096, 8192, x.data_ptr(), w.data_ptr(), out.data_ptr(), 1,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()

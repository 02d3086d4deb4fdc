"""GPU parity: the SDDMM -> SpMM chain over heads (two streams) against the two operators called
head by head on one stream, and against the oracle."""
import numpy as np
import pytest
import torch

from intrasm_engine_b200 import synthetic as syn
from intrasm_engine_b200.pytorch.attention import SparseAttentionChain
from . import gpu_util as G

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,d,density,heads", [(1024, 1024, 64, 0.05, 5), (300, 520, 48, 0.2, 3), (2048, 4096, 64, 0.03, 4)])
def test_chain_over_heads(oracle, m, n, d, density, heads):
    rng = np.random.default_rng(m + n + heads)
    mask = syn.csr_from_mask(rng.random((m, n)) < density, rng=rng)
    dm = G.DevCSR(mask)
    q = G.dev(rng.standard_normal((heads, m, d)).astype(np.float32))
    k = G.dev(rng.standard_normal((heads, n, d)).astype(np.float32))
    v = G.dev(rng.standard_normal((heads, n, d)).astype(np.float32))
    chain = SparseAttentionChain(dm.row_offsets, dm.column_indices, m, n)
    out, scores = chain(q, k, v, return_scores=True)
    torch.cuda.synchronize()
    one = SparseAttentionChain(dm.row_offsets, dm.column_indices, m, n, streams=1)
    out1, scores1 = one(q, k, v, return_scores=True)
    assert torch.equal(out, out1) and torch.equal(scores, scores1)  # the streams change no arithmetic
    for h in (0, heads - 1):
        qs, ks = q[h].cpu().numpy()[None], k[h].cpu().numpy()[None]
        exact = oracle.sddmm(qs, ks, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
        sabs = oracle.sddmm(np.abs(qs), np.abs(ks), mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
        assert G.sddmm_close(scores[h].cpu().numpy(), exact, sabs)
        ref = oracle.spmm(mask.row_indices, scores[h].cpu().numpy(), mask.row_offsets, mask.column_indices,
                          v[h].cpu().numpy(), m)[0]
        np.testing.assert_array_equal(out[h].cpu().numpy(), ref)  # the SpMM is bit-reproducible


def test_chain_empty_mask():
    m, n, d = 128, 256, 32
    ro = torch.zeros(m + 1, dtype=torch.int32, device=G.DEV)
    ci = torch.zeros(0, dtype=torch.int32, device=G.DEV)
    chain = SparseAttentionChain(ro, ci, m, n)
    out = chain(torch.randn(2, m, d, device=G.DEV), torch.randn(2, n, d, device=G.DEV), torch.randn(2, n, d, device=G.DEV))
    assert out.shape == (2, m, d) and not out.any()

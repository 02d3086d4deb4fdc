"""GPU parity: SDDMM through the C ABI against the CPU oracle and the golden vectors.

The kernel splits each dot product over the lanes of a sub-warp, so the fp32 summation
order differs from the oracle's: values must agree to 1e-5 relative (plus 1e-5 of the
tensor's max magnitude for cancelled sums) with the double-precision oracle.  The output
ORDER (aligned with column_indices) is exact by construction and checked through the
position-dependent reference.
"""
import glob
import os

import numpy as np
import pytest
import torch

from intrasm_engine_b200 import synthetic as syn
from . import gpu_util as G

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "sddmm_*.npz")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_sddmm_golden(oracle, path):
    g = np.load(path)
    mask = syn.CSR(np.zeros(len(g["column_indices"]), np.float32), g["row_indices"], g["row_offsets"],
                   g["column_indices"], (int(g["m"]), int(g["n"])))
    got = G.sddmm_f32(G.DevCSR(mask), G.dev(g["lhs"])[None], G.dev(g["rhs"])[None]).cpu().numpy()
    assert G.close(got, g["out"], 1e-5, 1e-5)
    exact = oracle.sddmm(g["lhs"], g["rhs"], g["row_indices"], g["row_offsets"], g["column_indices"], f64=True)
    assert G.close(got, exact, 1e-5, 1e-5)


@pytest.mark.parametrize("m,n,k,density,batch", [
    (1, 1, 1, 1.0, 1), (9, 11, 3, 0.5, 1), (64, 64, 8, 0.3, 1), (70, 90, 16, 0.2, 2),
    (128, 128, 32, 0.1, 1), (100, 300, 36, 0.2, 1), (256, 256, 64, 0.05, 3), (60, 500, 100, 0.3, 1),
    (64, 64, 128, 0.5, 1), (48, 80, 260, 0.2, 2), (33, 47, 7, 0.6, 1), (128, 64, 64, 0.0, 1),
    (16, 2000, 64, 0.4, 1),
])
def test_sddmm_shapes(oracle, m, n, k, density, batch):
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    mask = syn.csr_from_mask(rng.random((m, n)) < density, rng=rng)
    lhs = rng.standard_normal((batch, m, k)).astype(np.float32)
    rhs = rng.standard_normal((batch, n, k)).astype(np.float32)
    got = G.sddmm_f32(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    exact = oracle.sddmm(lhs, rhs, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    assert got.shape == exact.shape
    assert G.close(got, exact, 1e-5, 1e-5), G.max_violation(got, exact, 1e-5, 1e-5)


@pytest.mark.parametrize("seed", range(24))
def test_sddmm_random_shapes(oracle, seed):
    """Seeded random shapes: ragged rows (empty to full), every k alignment class, batches."""
    rng = np.random.default_rng(500 + seed)
    m, n = int(rng.integers(1, 400)), int(rng.integers(1, 600))
    k = int(rng.choice([1, 3, 4, 8, 20, 32, 36, 64, 100, 128, 200, 260]))
    batch = int(rng.integers(1, 4))
    row_density = rng.choice([0.0, 0.02, 0.2, 1.0], size=m, p=[0.15, 0.4, 0.35, 0.1])
    mask = syn.csr_from_mask(rng.random((m, n)) < row_density[:, None], rng=rng)
    lhs = rng.standard_normal((batch, m, k)).astype(np.float32)
    rhs = rng.standard_normal((batch, n, k)).astype(np.float32)
    got = G.sddmm_f32(G.DevCSR(mask), G.dev(lhs), G.dev(rhs)).cpu().numpy()
    exact = oracle.sddmm(lhs, rhs, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    assert got.shape == exact.shape
    assert G.close(got, exact, 1e-5, 1e-5), (m, n, k, batch, G.max_violation(got, exact, 1e-5, 1e-5))


def test_sddmm_accumulate_and_determinism(oracle):
    mask, q, k, _ = syn.sddmm_chain_case(2, 128, 160, 64, 0.1)
    dm = G.DevCSR(mask)
    o1 = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    o2 = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    assert torch.equal(o1, o2)
    start = torch.ones_like(o1)
    o3 = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None], out=start.clone(), accumulate=True)
    assert torch.allclose(o3, o1 + 1, rtol=1e-6, atol=1e-6)


def test_sddmm_cfg2_chain_full_size(oracle):
    """Benchmark configuration 2: SDDMM over a 4096x4096 mask at 95 % sparsity (K=64), then SpMM with V."""
    mask, q, k, v = syn.sddmm_chain_case(0)
    dm = G.DevCSR(mask)
    scores = G.sddmm_f32(dm, G.dev(q)[None], G.dev(k)[None])
    exact = oracle.sddmm(q, k, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    got = scores.cpu().numpy()
    assert G.close(got, exact, 1e-5, 1e-5), G.max_violation(got, exact, 1e-5, 1e-5)
    tref = oracle.torch_sddmm(q, k, mask.row_offsets, mask.column_indices)
    assert G.close(got, tref, 1e-5, 1e-5)
    dm.values = scores
    out = G.spmm_f32(dm, G.dev(v)[None])[0].cpu().numpy()
    ref = oracle.spmm(mask.row_indices, got, mask.row_offsets, mask.column_indices, v, 4096)[0]
    np.testing.assert_array_equal(out, ref)  # SpMM is bit-exact given the same values


def test_torch_ops_sddmm(oracle):
    import intrasm_engine_b200  # noqa: F401
    mask, q, k, _ = syn.sddmm_chain_case(4, 96, 80, 32, 0.2)
    dm = G.DevCSR(mask)
    out = torch.ops.iex_ops.sddmm_sputnik_atomic_upd_weight(G.dev(q)[None], G.dev(k)[None], dm.row_indices,
                                                            dm.row_offsets, dm.column_indices)
    exact = oracle.sddmm(q, k, mask.row_indices, mask.row_offsets, mask.column_indices, f64=True)
    assert G.close(out.cpu().numpy(), exact, 1e-5, 1e-5)
    with pytest.raises(RuntimeError):
        torch.ops.iex_ops.sddmm_sputnik_atomic_upd_weight(G.dev(q)[None], G.dev(k[:, :16])[None],
                                                          dm.row_indices, dm.row_offsets, dm.column_indices)

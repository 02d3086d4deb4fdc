"""CPU: the C oracle against the committed golden vectors (made with the torch CPU path)."""
import glob
import os

import numpy as np
import pytest

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _close(got, ref, rtol, scale_tol):
    """|got-ref| <= rtol*|ref| + scale_tol*max|ref|  (the second term covers cancellation)."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    bound = rtol * np.abs(ref) + scale_tol * (np.abs(ref).max() if ref.size else 0.0)
    return bool(np.all(np.abs(got - ref) <= bound))


def test_golden_files_present():
    assert len(GOLDEN) >= 10


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_matches_golden(oracle, path):
    g = np.load(path)
    kind = str(g["kind"])
    if kind == "spmm":
        m = int(g["m"])
        assert oracle.validate_csr(m, int(g["k"]), g["row_indices"], g["row_offsets"],
                                   g["column_indices"]) == 0
        got = oracle.spmm(g["row_indices"], g["values"], g["row_offsets"],
                          g["column_indices"], g["dense"], m)[0]
        exact = oracle.spmm(g["row_indices"], g["values"], g["row_offsets"],
                            g["column_indices"], g["dense"], m, f64=True)[0]
        # fp32 sums in a different order agree to 1e-5 relative (tolerance of the task).
        assert _close(got, g["out"], 1e-5, 1e-5)
        assert _close(g["out"], exact, 1e-5, 1e-5)
        assert _close(got, exact, 1e-5, 1e-5)
    elif kind == "sddmm":
        got = oracle.sddmm(g["lhs"], g["rhs"], g["row_indices"], g["row_offsets"],
                           g["column_indices"])
        exact = oracle.sddmm(g["lhs"], g["rhs"], g["row_indices"], g["row_offsets"],
                             g["column_indices"], f64=True)
        assert got.shape == g["out"].shape
        assert _close(got, g["out"], 1e-5, 1e-5)
        assert _close(got, exact, 1e-5, 1e-5)
    elif kind == "linear":
        got = oracle.linear(g["input"], g["weight"])
        assert _close(got, g["out"], 1e-5, 1e-5)
    else:
        raise AssertionError(kind)


def test_oracle_spmm_bias_relu_and_accumulate(oracle):
    g = np.load(GOLDEN[[os.path.basename(p) for p in GOLDEN].index("spmm_f32_64x64x32_d10.npz")])
    m = int(g["m"])
    args = (g["row_indices"], g["values"], g["row_offsets"], g["column_indices"], g["dense"], m)
    plain = oracle.spmm(*args)
    bias = np.linspace(-1, 1, m).astype(np.float32)
    fused = oracle.spmm(*args, bias=bias)
    np.testing.assert_array_equal(fused, np.maximum(plain + bias[None, :, None], 0))
    start = np.ones_like(plain)
    np.testing.assert_array_equal(oracle.spmm(*args, out=start), plain + 1)


def test_oracle_batched_values(oracle):
    g = np.load(GOLDEN[[os.path.basename(p) for p in GOLDEN].index("spmm_f32_64x64x32_d10.npz")])
    m = int(g["m"])
    rng = np.random.default_rng(0)
    dense = rng.standard_normal((3,) + g["dense"].shape).astype(np.float32)
    vals = rng.standard_normal((3, g["values"].shape[0])).astype(np.float32)
    out = oracle.spmm(g["row_indices"], vals, g["row_offsets"], g["column_indices"], dense, m)
    for z in range(3):
        one = oracle.spmm(g["row_indices"], vals[z], g["row_offsets"], g["column_indices"],
                          dense[z], m)[0]
        np.testing.assert_array_equal(out[z], one)


def test_oracle_sddmm_batch_sums(oracle):
    g = np.load(GOLDEN[[os.path.basename(p) for p in GOLDEN].index("sddmm_f32_64x64x32_d10.npz")])
    lhs = np.stack([g["lhs"], 2 * g["lhs"]])
    rhs = np.stack([g["rhs"], g["rhs"]])
    both = oracle.sddmm(lhs, rhs, g["row_indices"], g["row_offsets"], g["column_indices"])
    one = oracle.sddmm(g["lhs"], g["rhs"], g["row_indices"], g["row_offsets"], g["column_indices"])
    np.testing.assert_allclose(both, 3 * one, rtol=1e-6, atol=1e-6)


def test_validate_csr_rejects(oracle):
    ro = np.array([0, 2, 1, 3], np.int32)
    assert oracle.validate_csr(3, 4, [0, 1, 2], ro, [0, 1, 2]) == 3
    assert oracle.validate_csr(2, 4, [0, 1], [0, 1, 2], [0, 4]) == 4
    assert oracle.validate_csr(2, 4, [0, 0], [0, 1, 2], [0, 1]) == 5
    assert oracle.validate_csr(2, 4, [0, 1], [1, 1, 2], [0, 1]) == 1

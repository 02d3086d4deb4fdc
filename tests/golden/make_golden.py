"""Generates tests/golden/*.npz: small seeded inputs with the outputs of the torch CPU path.

The reference ships no golden vectors for SpMM / SDDMM and cannot be built or imported
in this environment (its Sputnik submodule, xformers, pycuda, cupy and sparta are all
absent), so the fixtures pin the oracle to the path the task names as the reference CPU
path: torch.sparse.mm (CSR, fp32, int32 indices), torch.sparse.sampled_addmm and
torch.matmul.  Inputs are stored next to the outputs, so the fixtures do not depend on
any generator staying unchanged.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from intrasm_engine_b200 import synthetic as syn  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def spmm_case(name, seed, m, k, n, density, dtype=np.float32, empty_rows=()):
    rng = np.random.default_rng(seed)
    mask = rng.random((m, k)) < density
    for r in empty_rows:
        mask[r] = False
    a = syn.csr_from_mask(mask, rng=rng, std=1.0 if dtype == np.float32 else 0.5, dtype=dtype)
    b = rng.standard_normal((k, n)).astype(dtype)
    out = orc.torch_spmm(a.row_offsets, a.column_indices, a.values.astype(np.float32),
                         b.astype(np.float32), m)
    np.savez(os.path.join(HERE, name + ".npz"), kind="spmm", m=m, k=k, n=n,
             values=a.values, row_indices=a.row_indices, row_offsets=a.row_offsets,
             column_indices=a.column_indices, dense=b, out=out.astype(np.float32))


def sddmm_case(name, seed, m, n, k, density):
    rng = np.random.default_rng(seed)
    mask = syn.csr_from_mask(rng.random((m, n)) < density, rng=rng)
    lhs = rng.standard_normal((m, k)).astype(np.float32)
    rhs = rng.standard_normal((n, k)).astype(np.float32)
    out = orc.torch_sddmm(lhs, rhs, mask.row_offsets, mask.column_indices)
    np.savez(os.path.join(HERE, name + ".npz"), kind="sddmm", m=m, n=n, k=k,
             row_indices=mask.row_indices, row_offsets=mask.row_offsets,
             column_indices=mask.column_indices, lhs=lhs, rhs=rhs, out=out.astype(np.float32))


def linear_case(name, seed, tokens, cin, cout):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((tokens, cin)).astype(np.float16)
    w = (rng.standard_normal((cout, cin)) * 0.05).astype(np.float16)
    out = orc.torch_linear(x, w)
    np.savez(os.path.join(HERE, name + ".npz"), kind="linear", input=x, weight=w,
             out=out.astype(np.float32))


if __name__ == "__main__":
    torch.manual_seed(0)
    spmm_case("spmm_f32_64x64x32_d10", 1, 64, 64, 32, 0.10)
    spmm_case("spmm_f32_48x64x20_d30_emptyrows", 2, 48, 64, 20, 0.30, empty_rows=(0, 7, 47))
    spmm_case("spmm_f32_33x17x5_d50_odd", 3, 33, 17, 5, 0.50)
    spmm_case("spmm_f32_16x64x64_d100_full", 4, 16, 64, 64, 1.01)
    spmm_case("spmm_f16_64x64x64_d20", 5, 64, 64, 64, 0.20, dtype=np.float16)
    spmm_case("spmm_f16_40x56x24_d50_emptyrows", 6, 40, 56, 24, 0.50, dtype=np.float16,
              empty_rows=(3, 39))
    sddmm_case("sddmm_f32_64x64x32_d10", 7, 64, 64, 32, 0.10)
    sddmm_case("sddmm_f32_40x64x64_d25", 8, 40, 64, 64, 0.25)
    sddmm_case("sddmm_f32_33x29x7_d50_odd", 9, 33, 29, 7, 0.50)
    linear_case("linear_f16_16x64x48", 10, 16, 64, 48)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))

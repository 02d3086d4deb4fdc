"""``torch.ops.iex_ops.*`` — the reference's operator boundary.

The operators are registered by a compiled torch extension, ``libiex_torch_ext.so``
(source: ``torch_ext/iex_torch_ext.cpp``), the way the reference registers its own from
intrasm_engine/pytorch/csrc/extensions/sputnik_kernels.cpp:189-193.  The extension holds
the argument checks and output allocation and calls the C ABI of ``libiex_b200.so``; this
module only loads it.  Operators:

  spmm_sputnik_reuse_weight(b, row_indices, values, row_offsets, column_indices, m)
  spmm_sputnik_atomic(b, row_indices, values, row_offsets, column_indices, m)
  spmm_sputnik_reuse_weight_half(b, row_indices, values, row_offsets, column_indices, m)
  sddmm_sputnik_atomic_upd_weight(a, b, row_indices, row_offsets, column_indices)
  linear_fp16(input, weight)                                    input @ weight.T
  linear_fp16_dgrad(grad, weight)                               grad @ weight     (d input)
  linear_fp16_wgrad(grad, input)                                grad.T @ input    (d weight)
  spmm_tc_half(x, row_offsets, values, column_indices, m)       A_csr @ x on tensor cores
  fused_spmm_linear_half(x, row_offsets, values, column_indices, m, weight)
                                                                (A_csr @ x, (weight @ x).T)
  csr_to_dense_half(row_offsets, values, column_indices, m, k)  dense copy of a CSR matrix
  validate_csr(row_offsets, column_indices, m, k, require_ascending) -> int
                                                                0, or IEX_CSR_* bits
  sddmm_plan(row_offsets, column_indices, m, n)                 pattern-only plan (build once)
  sddmm_tc_planned(a, b, plan, nnz)                             SDDMM on tensor cores (fp32,
                                                                TF32 head/tail tiles), a [m, k],
                                                                b [n, k] -> [nnz]
  spmm_plan(row_offsets, column_indices, m, k)                  pattern-only plan (build once)
  spmm_tc_planned(b, values, plan, m)                           SpMM on tensor cores (fp32),
                                                                A [m, k] x b [k, n] -> [m, n]
With ``IEX_VALIDATE_CSR=1`` in the environment every sparse operator runs that check on its
arguments first and raises on a malformed matrix (debugging aid; one extra kernel and a
synchronisation per call).

All are implemented for the CUDA dispatch key only: there is no CPU path.
"""
from __future__ import annotations

import os

import torch

from . import _lib  # noqa: F401  (loads libiex_b200.so first and fails loudly without it)

EXT_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libiex_torch_ext.so")

if not os.path.exists(EXT_PATH):
    raise ImportError(
        f"{EXT_PATH} is missing: build it with `python intrasm_engine_b200/build.py` "
        "(there is no Python or CPU fallback for torch.ops.iex_ops)")

torch.ops.load_library(EXT_PATH)

OP_NAMES = (
    "spmm_sputnik_reuse_weight",
    "spmm_sputnik_atomic",
    "spmm_sputnik_reuse_weight_half",
    "sddmm_sputnik_atomic_upd_weight",
    "sddmm_sputnik_half",
    "linear_fp16",
    "linear_fp16_dgrad",
    "linear_fp16_wgrad",
    "spmm_tc_half",
    "fused_spmm_linear_half",
    "csr_to_dense_half",
    "validate_csr",
    "sddmm_plan",
    "sddmm_tc_planned",
    "spmm_plan",
    "spmm_tc_planned",
)

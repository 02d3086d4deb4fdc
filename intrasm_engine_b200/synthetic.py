"""Seeded synthetic workloads for the SpMM / SDDMM / fused sparse‖dense path (host, numpy).

These stand in for the datasets the reference points at but does not ship (the DLMC
collection fetched by benchmark/setup_sgk_dlmc.sh:2-7, pruned checkpoints, ReLU-LLaMA
activations): same shapes, sparsity levels and value distributions, generated from a
seed.  No item of any of those datasets is reproduced.

Everything here is host-side input preparation; the compute path lives in the CUDA
library.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class CSR:
    """CSR triple plus the row visiting order the kernels use.

    ``row_indices`` lists the rows by decreasing nnz (stable), the load-balancing order
    the reference obtains from its CSR conversion (intrasm_engine/pytorch/utils.py:143-153).
    ``column_indices`` are ascending inside a row.
    """

    values: np.ndarray
    row_indices: np.ndarray
    row_offsets: np.ndarray
    column_indices: np.ndarray
    shape: tuple

    @property
    def nnz(self) -> int:
        return int(self.column_indices.shape[0])

    def to_dense(self) -> np.ndarray:
        m, k = self.shape
        out = np.zeros((m, k), dtype=self.values.dtype)
        rows = np.repeat(np.arange(m), np.diff(self.row_offsets))
        out[rows, self.column_indices] = self.values
        return out


def swizzle_rows(row_offsets: np.ndarray) -> np.ndarray:
    """Row order by decreasing nnz, ties by row id."""
    nnz_per_row = np.diff(row_offsets.astype(np.int64))
    return np.argsort(-nnz_per_row, kind="stable").astype(np.int32)


def csr_from_mask(mask: np.ndarray, values_dense: np.ndarray | None = None,
                  rng: np.random.Generator | None = None, std: float = 1.0,
                  dtype=np.float32, index_dtype=np.int32) -> CSR:
    """CSR of the True entries of ``mask``; values from ``values_dense`` or N(0, std)."""
    m, k = mask.shape
    counts = mask.sum(axis=1, dtype=np.int64)
    row_offsets = np.zeros(m + 1, dtype=np.int32)
    np.cumsum(counts, out=row_offsets[1:])
    cols = np.nonzero(mask)[1].astype(index_dtype)
    if values_dense is not None:
        vals = values_dense[mask].astype(dtype)
    else:
        vals = (rng.standard_normal(cols.shape[0]) * std).astype(dtype)
    return CSR(vals, swizzle_rows(row_offsets), row_offsets, cols, (m, k))


def dense_to_csr(matrix: np.ndarray, index_dtype=np.int32) -> CSR:
    """CSR of the non-zero entries of a dense matrix (values keep the matrix dtype)."""
    return csr_from_mask(matrix != 0, values_dense=matrix, dtype=matrix.dtype,
                         index_dtype=index_dtype)


def csr_from_row_counts(counts: np.ndarray, k: int, rng: np.random.Generator,
                        std: float, dtype, index_dtype=np.int32) -> CSR:
    """Rows with prescribed nnz, distinct uniform columns (ascending), values N(0, std)."""
    m = counts.shape[0]
    row_offsets = np.zeros(m + 1, dtype=np.int32)
    np.cumsum(counts, out=row_offsets[1:])
    nnz = int(row_offsets[-1])
    cols = np.empty(nnz, dtype=index_dtype)
    for r in range(m):
        c = int(counts[r])
        if c:
            cols[row_offsets[r]:row_offsets[r + 1]] = np.sort(
                rng.choice(k, size=c, replace=False))
    vals = (rng.standard_normal(nnz) * std).astype(dtype)
    return CSR(vals, swizzle_rows(row_offsets), row_offsets, cols, (m, k))


# --------------------------------------------------------------------------------------
# The five benchmark configurations
# --------------------------------------------------------------------------------------

def spmm_fp32_case(seed: int = 0, m: int = 1024, k: int = 1024, n: int = 256,
                   density: float = 0.1):
    """fp32 SpMM: Bernoulli(density) mask, values N(0,1), int32 indices; B is k×n N(0,1)."""
    rng = np.random.default_rng(seed)
    a = csr_from_mask(rng.random((m, k)) < density, rng=rng)
    b = rng.standard_normal((k, n)).astype(np.float32)
    return a, b


def sddmm_chain_case(seed: int = 0, m: int = 4096, n: int = 4096, k: int = 64,
                     density: float = 0.05):
    """fp32 SDDMM then SpMM: Q m×k, K n×k, V n×k all N(0,1); Bernoulli(density) mask."""
    rng = np.random.default_rng(seed)
    mask = csr_from_mask(rng.random((m, n)) < density, rng=rng)
    mask.values[:] = 0
    q = rng.standard_normal((m, k)).astype(np.float32)
    kk = rng.standard_normal((n, k)).astype(np.float32)
    v = rng.standard_normal((n, k)).astype(np.float32)
    return mask, q, kk, v


def pruned_sweep_case(seed: int, rows: int, cols: int, sparsity: float, n: int,
                      index_dtype=np.int16, cv: float = 0.3):
    """fp16 pruned-weight SpMM: per-row nnz ~ lognormal (CV ``cv``) around the mean
    density, made even, uniform distinct columns, values N(0, 0.02); B cols×n N(0,1) fp16."""
    rng = np.random.default_rng(seed)
    mean = cols * (1.0 - sparsity)
    sigma = np.sqrt(np.log(1.0 + cv * cv))
    mu = np.log(max(mean, 1e-9)) - 0.5 * sigma * sigma
    counts = np.rint(rng.lognormal(mu, sigma, size=rows)).astype(np.int64)
    counts = np.clip(counts, 0, cols)
    counts -= counts % 2
    a = csr_from_row_counts(counts, cols, rng, 0.02, np.float16, index_dtype)
    b = rng.standard_normal((cols, n)).astype(np.float16)
    return a, b


def magnitude_prune(weight: np.ndarray, sparsity: float) -> np.ndarray:
    """Boolean keep-mask of the (1 - sparsity) largest |w| over the whole matrix."""
    flat = np.abs(weight).ravel()
    keep = int(round(flat.shape[0] * (1.0 - sparsity)))
    if keep <= 0:
        return np.zeros_like(weight, dtype=bool)
    thresh = np.partition(flat, flat.shape[0] - keep)[flat.shape[0] - keep]
    return np.abs(weight) >= thresh


def fused_layer_case(seed: int = 0, m_sparse: int = 11008, k: int = 4096,
                     tokens: int = 64, m_dense: int = 12288, sparsity: float = 0.5,
                     index_dtype=np.int16):
    """LLaMA-7B-shaped fused layer, fp16: W_up (m_sparse×k) magnitude-pruned to CSR,
    W_qkv (m_dense×k) dense, both N(0, 0.02); X k×tokens N(0,1) shared by both branches."""
    rng = np.random.default_rng(seed)
    w_up = (rng.standard_normal((m_sparse, k), dtype=np.float32) * 0.02).astype(np.float16)
    keep = magnitude_prune(w_up.astype(np.float32), sparsity) & (w_up != 0)
    a = csr_from_mask(keep, values_dense=w_up, dtype=np.float16, index_dtype=index_dtype)
    w_qkv = (rng.standard_normal((m_dense, k), dtype=np.float32) * 0.02).astype(np.float16)
    x = rng.standard_normal((k, tokens), dtype=np.float32).astype(np.float16)
    return a, w_qkv, x


def relu_ffn_layer_case(seed: int = 0, layer: int = 0, tokens: int = 256, k: int = 11008,
                        n: int = 4096, density: float = 0.1, index_dtype=np.int32,
                        with_weight: bool = True):
    """ReLU-sparse FFN down projection, fp16: activations tokens×k with Bernoulli(density)
    non-zeros |N(0,1)| as CSR; W_down k×n N(0, 0.02)."""
    rng = np.random.default_rng([seed, layer])
    mask = rng.random((tokens, k)) < density
    act = np.abs(rng.standard_normal((tokens, k), dtype=np.float32)).astype(np.float16)
    act[act == 0] = np.float16(6e-8)
    a = csr_from_mask(mask, values_dense=act, dtype=np.float16, index_dtype=index_dtype)
    w = None
    if with_weight:
        w = (rng.standard_normal((k, n), dtype=np.float32) * 0.02).astype(np.float16)
    return a, w


# --------------------------------------------------------------------------------------
# Algorithmic (compulsory) traffic and useful work, each array touched once
# --------------------------------------------------------------------------------------

def spmm_bytes(m, k, n, nnz, value_bytes, index_bytes):
    return nnz * (value_bytes + index_bytes) + 4 * (m + 1) + 4 * m + k * n * value_bytes \
        + m * n * value_bytes


def spmm_flops(nnz, n):
    return 2 * nnz * n


def sddmm_bytes(m, n, k, nnz):
    return (m + n) * k * 4 + 4 * nnz + 4 * (m + 1) + 4 * m + 4 * nnz


def sddmm_flops(nnz, k):
    return 2 * nnz * k


def gemm_bytes(m, n, k, elt=2):
    return elt * (m * k + k * n + m * n)


def gemm_flops(m, n, k):
    return 2 * m * n * k

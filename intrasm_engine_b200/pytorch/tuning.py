"""Kernel selection for the fp16 CSR SpMM on B200: CUDA cores or tensor cores.

The reference sketches a tuner that is meant to pick a kernel configuration per layer shape
(intrasm_engine/tuning/my_autograd_func_tuner.py; its build_and_test returns nothing).  Here
the choice is between two kernels and a cost model fitted to measurements decides it; no
search at run time, nothing read back from the device (nnz is the length of the values
tensor).

Measured behaviour the model encodes (B200, CUDA events, operands rotating through more than
L2):
  * CUDA-core kernel: every nonzero gathers a row of n fp16 values through L1/L2, and a row's
    nonzeros are walked in sequence by one sub-warp; time = 1.6 us + 0.06 us per MB gathered
    + 0.16 us per nonzero of an average row fits the four measurements below within 10 %.
      2048x512 @70 % sparse, n=128: 30.8 us    512x2048 @95 %, n=128: 18.5 us
      512x512 @90 %, n=256: 10.3 us            11008x4096 @50 %, n=64: 450 us
  * Tensor-core kernel: ~9 us per launch plus ~0.75 us per 64 columns of the matrix for
    every wave of tiles (one tile of up to 128 rows per SM and wave), nearly independent of
    density.
      2048x512 @70 %: 12.4 us    512x2048 @95 %: 20.7 us    11008x4096 @50 %: 49 us
"""
from __future__ import annotations

SMS = 148
CUDA_CORE_FIXED_US = 1.6
CUDA_CORE_US_PER_MB = 0.0605      # gathered bytes (nnz * n * sizeof(value))
CUDA_CORE_US_PER_ROW_NNZ = 0.158  # per nonzero of an average row (sequential walk)
TC_FIXED_US = 9.0
TC_US_PER_SLOT = 0.75     # per 64 columns and wave


def cuda_core_us(m: int, nnz: int, n: int, value_bytes: int = 2) -> float:
    return (CUDA_CORE_FIXED_US + CUDA_CORE_US_PER_MB * nnz * n * value_bytes / 1e6
            + CUDA_CORE_US_PER_ROW_NNZ * nnz / max(m, 1))


def tensor_core_us(m: int, k: int) -> float:
    tiles = -(-m // 128)
    if 0 < tiles < SMS:  # lower tiles, one per SM (the library does this for single-part launches)
        tiles = min(SMS, -(-m // 8))
    waves = max(1, -(-tiles // SMS))
    return TC_FIXED_US + TC_US_PER_SLOT * (-(-k // 64)) * waves


def tensor_core_supported(k: int, n: int, value_bits: int, index_bits: int) -> bool:
    """Shape limits of iex_spmm_f16_tc (column indices must also ascend inside each row, which
    every converter in this package guarantees)."""
    return (value_bits == 16 and index_bits in (16, 32) and n % 64 == 0 and 0 < n <= 256
            and k % 8 == 0 and k > 0 and (index_bits == 32 or k <= 65280))


def choose_spmm_kernel(m: int, k: int, n: int, nnz: int, value_bits: int = 16,
                       index_bits: int = 16) -> str:
    """``"tensor_core"`` or ``"cuda_core"`` for A [m, k] (CSR, nnz stored) times B [k, n]."""
    if not tensor_core_supported(k, n, value_bits, index_bits) or m <= 0:
        return "cuda_core"
    return "tensor_core" if tensor_core_us(m, k) < cuda_core_us(m, nnz, n) else "cuda_core"

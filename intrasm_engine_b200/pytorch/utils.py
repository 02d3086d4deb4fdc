"""CSR helpers on the device (torch tensors in, torch tensors out).

Counterparts of intrasm_engine/pytorch/utils.py: ``dense_to_sparse`` (there a call into
xformers, :143-153), ``partition_csr`` / ``partition_coo`` (:6-139, Python loops with
aliased lists) and the precision toggles (:173-198), plus the transpose bookkeeping that the
reference takes from xformers (``_transpose_with_info``,
layers_and_funcs/sputnik.py:4, :122).  Everything is vectorised torch code that runs
on the tensors' device; no host loop over nonzeros.
"""
from __future__ import annotations

import torch


def dense_to_sparse(matrix: torch.Tensor, device=None, index_dtype=torch.int32):
    """Dense 2-D matrix -> ``(values, row_indices, row_offsets, column_indices)``.

    ``row_indices`` orders the rows by decreasing nnz (stable); column indices ascend in a
    row; ``row_offsets`` / ``row_indices`` are int32, ``column_indices`` ``index_dtype``.
    """
    if matrix.dim() != 2:
        raise RuntimeError("dense_to_sparse expects a 2-D matrix")
    if device is not None:
        matrix = matrix.to(device)
    mask = matrix != 0
    counts = mask.sum(dim=1)
    row_offsets = torch.zeros(matrix.size(0) + 1, dtype=torch.int32, device=matrix.device)
    row_offsets[1:] = torch.cumsum(counts, 0)
    column_indices = mask.nonzero(as_tuple=True)[1].to(index_dtype)
    values = matrix[mask]
    row_indices = torch.argsort(counts, descending=True, stable=True).to(torch.int32)
    return values, row_indices, row_offsets, column_indices


def dense_to_sparse_cuda(matrix: torch.Tensor, index_dtype=torch.int32, relu: bool = False):
    """``dense_to_sparse`` for a CUDA matrix (fp16 / fp32) with this library's own kernels
    (``iex_dense_to_csr_count`` / ``_fill``): same four tensors, same ordering rules.  With
    ``relu`` the result is the CSR of ``relu(matrix)`` (what a ReLU-sparse FFN hands to its
    down projection).  One host read-back (nnz) sits between the two kernels' launches."""
    from .. import _lib
    if matrix.dim() != 2 or not matrix.is_cuda or not matrix.is_contiguous():
        raise RuntimeError("dense_to_sparse_cuda expects a contiguous 2-D CUDA matrix")
    if matrix.dtype not in (torch.float16, torch.float32) or index_dtype not in (torch.int16, torch.int32):
        raise RuntimeError("dense_to_sparse_cuda: fp16 / fp32 values, int16 / int32 indices")
    m, k = matrix.shape
    vbits = 16 if matrix.dtype == torch.float16 else 32
    ibits = 16 if index_dtype == torch.int16 else 32
    with torch.cuda.device(matrix.device):
        st = torch.cuda.current_stream(matrix.device).cuda_stream
        row_offsets = torch.empty(m + 1, dtype=torch.int32, device=matrix.device)
        row_indices = torch.empty(m, dtype=torch.int32, device=matrix.device)
        _lib.call("iex_dense_to_csr_count", m, k, matrix.data_ptr(), vbits, int(relu),
                  row_offsets.data_ptr(), row_indices.data_ptr(), st)
        nnz = int(row_offsets[m].item())
        values = torch.empty(nnz, dtype=matrix.dtype, device=matrix.device)
        column_indices = torch.empty(nnz, dtype=index_dtype, device=matrix.device)
        if nnz > 0:
            _lib.call("iex_dense_to_csr_fill", m, k, matrix.data_ptr(), vbits, int(relu),
                      row_offsets.data_ptr(), values.data_ptr(), column_indices.data_ptr(), ibits, st)
    return values, row_indices, row_offsets, column_indices


def sparse_to_dense(values, row_offsets, column_indices, m: int, k: int) -> torch.Tensor:
    rows = torch.repeat_interleave(torch.arange(m, device=values.device),
                                   (row_offsets[1:] - row_offsets[:-1]).long())
    out = torch.zeros((m, k), dtype=values.dtype, device=values.device)
    out[rows, column_indices.long()] = values
    return out


def swizzle_rows(row_offsets: torch.Tensor) -> torch.Tensor:
    counts = row_offsets[1:] - row_offsets[:-1]
    return torch.argsort(counts, descending=True, stable=True).to(torch.int32)


def get_transpose_info(m: int, k: int, row_indices, row_offsets, column_indices):
    """Pattern-only bookkeeping for A^T: ``(row_indices_t, row_offsets_t, column_indices_t, perm)``.

    ``perm`` maps a position in A^T's value array to the position of the same nonzero in
    A's, so ``values_t = values[perm]``.  Computed once per sparsity pattern.
    """
    del row_indices
    dev = column_indices.device
    counts = (row_offsets[1:] - row_offsets[:-1]).long()
    rows = torch.repeat_interleave(torch.arange(m, device=dev), counts)
    cols = column_indices.long()
    # stable sort by column keeps rows ascending inside each transposed row
    perm = torch.argsort(cols * m + rows)
    counts_t = torch.bincount(cols, minlength=k)
    row_offsets_t = torch.zeros(k + 1, dtype=torch.int32, device=dev)
    row_offsets_t[1:] = torch.cumsum(counts_t, 0)
    column_indices_t = rows[perm].to(column_indices.dtype)
    row_indices_t = torch.argsort(counts_t, descending=True, stable=True).to(torch.int32)
    return row_indices_t, row_offsets_t, column_indices_t, perm


def transpose_with_info(values: torch.Tensor, transp_info):
    """``(row_indices_t, values_t, row_offsets_t, column_indices_t)`` of A^T."""
    row_indices_t, row_offsets_t, column_indices_t, perm = transp_info
    return row_indices_t, values[perm], row_offsets_t, column_indices_t


def partition_csr(crow_indices, col_indices, values, num_rows: int, num_cols: int,
                  num_rows_per_partition: int, num_cols_per_partition: int):
    """Cuts a CSR matrix into a grid of CSR blocks.

    Returns three nested lists ``[row_block][col_block]`` of ``crow_indices`` (int64, length
    rows_per_partition + 1, starting at 0), block-local ``col_indices`` (int64) and values.
    Rows / columns beyond the last full partition are dropped, as in the reference
    (intrasm_engine/pytorch/utils.py:21-37 sizes the grid with floor division).
    """
    nrb, ncb = num_rows // num_rows_per_partition, num_cols // num_cols_per_partition
    dev = col_indices.device
    counts = (crow_indices[1:] - crow_indices[:-1]).long()
    rows = torch.repeat_interleave(torch.arange(num_rows, device=dev), counts)
    cols = col_indices.long()
    rb, cb = rows // num_rows_per_partition, cols // num_cols_per_partition
    crow_out, col_out, val_out = [], [], []
    for i in range(nrb):
        crow_row, col_row, val_row = [], [], []
        for j in range(ncb):
            sel = (rb == i) & (cb == j)
            local_rows = rows[sel] - i * num_rows_per_partition
            cnt = torch.bincount(local_rows, minlength=num_rows_per_partition)
            crow = torch.zeros(num_rows_per_partition + 1, dtype=torch.int64, device=dev)
            crow[1:] = torch.cumsum(cnt, 0)
            crow_row.append(crow)
            col_row.append(cols[sel] - j * num_cols_per_partition)
            val_row.append(values[sel])
        crow_out.append(crow_row)
        col_out.append(col_row)
        val_out.append(val_row)
    return crow_out, col_out, val_out


def partition_coo(row_indices, col_indices, values, num_rows: int, num_cols: int,
                  num_rows_per_partition: int, num_cols_per_partition: int):
    """Cuts a COO matrix into a grid of COO blocks with block-local coordinates."""
    nrb, ncb = num_rows // num_rows_per_partition, num_cols // num_cols_per_partition
    rows, cols = row_indices.long(), col_indices.long()
    rb, cb = rows // num_rows_per_partition, cols // num_cols_per_partition
    row_out, col_out, val_out = [], [], []
    for i in range(nrb):
        r_row, c_row, v_row = [], [], []
        for j in range(ncb):
            sel = (rb == i) & (cb == j)
            r_row.append(rows[sel] - i * num_rows_per_partition)
            c_row.append(cols[sel] - j * num_cols_per_partition)
            v_row.append(values[sel])
        row_out.append(r_row)
        col_out.append(c_row)
        val_out.append(v_row)
    return row_out, col_out, val_out


def nnz_balanced_row_split(row_offsets: torch.Tensor, parts: int) -> list[tuple[int, int]]:
    """Contiguous row ranges ``[(begin, end), ...]`` with about nnz / parts nonzeros each.

    The multi-GPU SpMM / SDDMM split: rows are independent, so each rank takes one range and
    no data-path communication is needed.
    """
    m = row_offsets.numel() - 1
    nnz = int(row_offsets[-1])
    targets = torch.arange(1, parts, device=row_offsets.device, dtype=torch.float64) * (nnz / parts)
    cuts = torch.searchsorted(row_offsets.to(torch.float64), targets).clamp(0, m).tolist()
    bounds = [0] + [int(c) for c in cuts] + [m]
    for i in range(1, len(bounds)):
        bounds[i] = max(bounds[i], bounds[i - 1])
    return [(bounds[i], bounds[i + 1]) for i in range(parts)]


def slice_csr_rows(values, row_offsets, column_indices, begin: int, end: int):
    """The CSR of rows ``[begin, end)`` (offsets rebased to 0), with its own swizzle order."""
    lo, hi = int(row_offsets[begin]), int(row_offsets[end])
    ro = (row_offsets[begin:end + 1] - lo).to(torch.int32)
    return values[lo:hi], swizzle_rows(ro), ro, column_indices[lo:hi]


def check_tensor_eligible_for_tensor_core(a: torch.Tensor) -> bool:
    return bool(a.is_cuda and a.dtype == torch.float16 and all(d % 8 == 0 for d in a.shape))


# The reference flips global matmul precision flags at import time
# (intrasm_engine/__init__.py:85).  The kernels here fix their arithmetic (fp32 accumulate)
# themselves, so the toggles only affect torch's own matmuls and are never called implicitly.
def set_tf32_use_tensor_core():
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True


def reset_tf32_use_tensor_core():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


def set_float_16_reduced_precision():
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = True
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = True


def reset_float_16_reduced_precision():
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False

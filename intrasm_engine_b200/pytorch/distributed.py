"""Multi-GPU use of the hot path: one process per GPU, ``torch.distributed`` for plumbing.

Two partitionings, matching how the work shards:
  * SpMM / SDDMM rows are independent, so a matrix is cut into nnz-balanced contiguous row
    ranges, one per rank, and NO data-path collective is needed
    (``shard_csr_rows`` / ``row_range_for_rank``);
  * the ReLU-sparse FFN down projection shards the dense weight by columns: every rank
    multiplies the (replicated) activation CSR with its ``[k, n / G]`` slab and the
    ``[tokens, n / G]`` results are all-gathered over NCCL (``ColumnShardedDownProj``).
The reference has no multi-GPU code at all (``MySpMMPartitioned`` / ``MyLinearPartitioned`` are
empty, layers_and_funcs/sputnik.py:152-154, torch.py:34-36).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .utils import nnz_balanced_row_split, slice_csr_rows


def row_range_for_rank(row_offsets: torch.Tensor, rank: int, world: int) -> tuple[int, int]:
    return nnz_balanced_row_split(row_offsets, world)[rank]


def shard_csr_rows(values, row_offsets, column_indices, rank: int, world: int):
    """This rank's rows of a CSR matrix: ``(values, row_indices, row_offsets, column_indices,
    (begin, end))`` with offsets rebased to zero."""
    begin, end = row_range_for_rank(row_offsets, rank, world)
    v, ri, ro, ci = slice_csr_rows(values, row_offsets, column_indices, begin, end)
    return v, ri, ro, ci, (begin, end)


def column_slab(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Columns ``[rank * n / G, (rank + 1) * n / G)`` of a ``[k, n]`` weight, contiguous."""
    n = weight.size(1)
    assert n % world == 0, "the column count must divide by the number of ranks"
    w = n // world
    return weight[:, rank * w:(rank + 1) * w].contiguous()


def all_gather_columns(local: torch.Tensor, group=None) -> torch.Tensor:
    """``[tokens, n / G]`` per rank -> ``[tokens, n]`` on every rank (rank r's columns at
    ``[r * n / G, (r + 1) * n / G)``)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    tokens, w = local.shape
    gathered = torch.empty((world * tokens, w), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered, local.contiguous(), group=group)
    return gathered.view(world, tokens, w).permute(1, 0, 2).reshape(tokens, world * w)


class ColumnShardedDownProj:
    """One FFN down-projection layer with the dense weight sharded by columns.

    ``spmm(values, row_indices, row_offsets, column_indices, dense, m) -> [m, n_local]`` is
    the local compute (the CUDA SpMM on GPU ranks; tests on CPU ranks pass a stand-in).
    """

    def __init__(self, w_down: torch.Tensor, rank: int, world: int, spmm, group=None):
        self.slab = column_slab(w_down, rank, world)
        self.rank, self.world, self.spmm, self.group = rank, world, spmm, group

    def local(self, values, row_indices, row_offsets, column_indices, tokens: int) -> torch.Tensor:
        return self.spmm(values, row_indices, row_offsets, column_indices, self.slab, tokens)

    def __call__(self, values, row_indices, row_offsets, column_indices, tokens: int) -> torch.Tensor:
        out = self.local(values, row_indices, row_offsets, column_indices, tokens)
        return all_gather_columns(out, self.group) if self.world > 1 else out


class PeerGather:
    """Buffers and calls for the all-gather that the linear kernel does with its own stores.

    Every rank owns ``slots`` result buffers ``[tokens, n]`` and a signal array in symmetric
    memory (``torch.distributed._symmetric_memory``: the same allocation on every GPU of the
    box, mapped into every process).  ``linear(...)`` computes this rank's column slab and
    stores it into all ranks' copies of result buffer ``slot``; ``barrier()`` then orders
    those stores before anybody's reads.  Alternate ``slot`` between consecutive layers: a
    rank may start storing layer L + 1 while a peer still reads layer L.
    """

    def __init__(self, tokens: int, n: int, rank: int, world: int, device, group=None, slots: int = 2):
        import ctypes

        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world, self.tokens, self.n, self.slots = rank, world, tokens, n, slots
        assert n % world == 0 and (n // world) % 8 == 0
        self.results = symm.empty((slots, tokens, n), dtype=torch.float16, device=device)
        self.signals = symm.empty((world + 1,), dtype=torch.int32, device=device)
        self.results.zero_()
        self.signals.zero_()
        self._h_res = symm.rendezvous(self.results, group)
        self._h_sig = symm.rendezvous(self.signals, group)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's signal words are zero before the first barrier
        slot_bytes = tokens * n * 2
        self._out_ptrs = [(ctypes.c_void_p * world)(*[int(p) + s * slot_bytes for p in self._h_res.buffer_ptrs])
                          for s in range(slots)]
        self._sig_ptrs = (ctypes.c_void_p * world)(*[int(p) for p in self._h_sig.buffer_ptrs])

    def result(self, slot: int) -> torch.Tensor:
        return self.results[slot]

    def linear(self, slot: int, input: torch.Tensor, weight_slab: torch.Tensor, parts: int,
               workspace: torch.Tensor, stream: int) -> None:
        """``result(slot)[:, rank * n/G : (rank + 1) * n/G] = input @ weight_slab.T`` on every rank."""
        from .. import _lib
        n_local = self.n // self.world
        _lib.call("iex_linear_f16_splitk_gather", self.tokens, input.size(1), n_local, input.data_ptr(),
                  weight_slab.data_ptr(), self._out_ptrs[slot], self.world, self.rank, self.n,
                  self.rank * n_local, parts, workspace.data_ptr(), workspace.numel(), stream)

    def barrier(self, stream: int) -> None:
        from .. import _lib
        _lib.call("iex_peer_barrier", self._sig_ptrs, self.world, self.rank, stream)

"""ReLU-activation-sparse FFN down projection, single GPU or column-sharded over the GPUs of a box.

    y [tokens, n] = act [tokens, k] (CSR, fp16, ~90 % zeros after ReLU)  @  W_down [k, n] (fp16)

This is the product path of the "activation-sparse FFN stack" workload: the reference only
leaves empty slots for it (``MyLinearPartitioned`` / ``MySpMMPartitioned``,
intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/torch.py:34-36, sputnik.py:152-154).

At 256 tokens the activation matrix is tiny (5.6 MB dense) and the weight is what streams
from HBM, so the layer runs as a tensor-core GEMM whose *B* operand is the activation: the
CSR is expanded to a dense fp16 tile operand once per layer (``iex_csr_to_dense_f16``) and
``iex_linear_f16_splitk`` multiplies it with this rank's weight slab, stored K-major
(``[n_local, k]``, i.e. W_down^T, the ``torch.nn.Linear`` convention).  Split-K spreads the
few 128-row weight tiles of a slab over all SMs.

Sharding: rank r owns output columns ``[r * n / G, (r + 1) * n / G)``.  The gathered
``[tokens, n]`` result appears on every rank either through the kernel's own peer stores
(``gather="peer"``: ``iex_linear_f16_splitk_gather`` writes the slab into every rank's result
buffer over NVLink, ``iex_peer_barrier`` orders the stores) or through an NCCL all-gather
(``gather="nccl"``); ``gather="none"`` leaves the local slab.
"""
from __future__ import annotations

import torch

from .. import _lib


def split_k_parts(n_local: int) -> int:
    """K parts per 128-row weight tile so that about 128 CTAs share a slab (measured optimum
    on B200: 32 tiles -> 4 parts, 16 -> 8, <= 8 -> 16)."""
    tiles = (n_local + 127) // 128
    return max(1, min(16, 128 // max(tiles, 1)))


class ReluSparseDownProj:
    """One down-projection layer (or a stack sharing its buffers: call it once per layer).

    ``weight_slab`` is this rank's ``[n_local, k]`` fp16 slab of W_down^T (contiguous).  All
    scratch (the dense activation tile, the split-K workspace, the result buffers) is
    allocated here, once; ``forward`` only launches kernels on the current stream, so a loop
    of layers can be captured into a CUDA graph.
    """

    def __init__(self, tokens: int, k: int, n: int, rank: int = 0, world: int = 1, device=None,
                 gather: str = "peer", group=None):
        assert n % world == 0, "the output width must divide by the number of ranks"
        assert gather in ("peer", "nccl", "none")
        self.tokens, self.k, self.n = int(tokens), int(k), int(n)
        self.rank, self.world, self.group = rank, world, group
        self.n_local = n // world
        self.gather = gather if world > 1 else "none"
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.parts = split_k_parts(self.n_local)
        need = _lib.lib.iex_tc_workspace_bytes(0, 1, self.n_local, self.parts, self.tokens)
        self.workspace = torch.empty(max(int(need), 256), dtype=torch.uint8, device=self.device)
        self.dense_act = torch.empty((self.tokens, self.k), dtype=torch.float16, device=self.device)
        self.out_local = torch.empty((self.tokens, self.n_local), dtype=torch.float16, device=self.device)
        self.peer = None
        self._slot = 0
        if self.gather == "peer":
            from .distributed import PeerGather
            self.peer = PeerGather(self.tokens, self.n, rank, world, self.device, group=group)

    # -- pieces ---------------------------------------------------------------------------
    def expand(self, values, row_offsets, column_indices, stream=None) -> torch.Tensor:
        """The activation CSR as the dense ``[tokens, k]`` tile operand (this object's buffer)."""
        st = stream if stream is not None else torch.cuda.current_stream(self.device).cuda_stream
        bits = 16 if column_indices.dtype == torch.int16 else 32
        _lib.call("iex_csr_to_dense_f16", self.tokens, self.k, row_offsets.data_ptr(), column_indices.data_ptr(),
                  bits, values.data_ptr(), self.dense_act.data_ptr(), st)
        return self.dense_act

    def forward(self, values, row_offsets, column_indices, weight_slab, stream=None) -> torch.Tensor:
        """``act_csr @ W_down``: ``[tokens, n]`` gathered on every rank (``gather`` "peer" /
        "nccl") or this rank's ``[tokens, n_local]`` slab ("none").  With "peer" the result is a
        view of one of two alternating buffers: it stays valid until the call after next."""
        assert weight_slab.shape == (self.n_local, self.k) and weight_slab.is_contiguous()
        st = stream if stream is not None else torch.cuda.current_stream(self.device).cuda_stream
        dense = self.expand(values, row_offsets, column_indices, st)
        if self.gather == "peer":
            slot, self._slot = self._slot, self._slot ^ 1
            self.peer.linear(slot, dense, weight_slab, self.parts, self.workspace, st)
            self.peer.barrier(st)
            return self.peer.result(slot)
        _lib.call("iex_linear_f16_splitk", self.tokens, self.k, self.n_local, dense.data_ptr(),
                  weight_slab.data_ptr(), self.out_local.data_ptr(), self.parts, self.workspace.data_ptr(),
                  self.workspace.numel(), st)
        if self.gather == "nccl":
            from .distributed import all_gather_columns
            return all_gather_columns(self.out_local, self.group)
        return self.out_local

    __call__ = forward


def relu_down_proj(hidden: torch.Tensor, weight_t: torch.Tensor, index_dtype=torch.int32) -> torch.Tensor:
    """``relu(hidden) @ weight_t.T`` on one GPU through the sparse path: ``hidden`` ``[tokens, k]``
    fp16 (pre-activation), ``weight_t`` ``[n, k]`` fp16.  The ReLU and the dense -> CSR conversion
    are one pass of this library's converter (``dense_to_sparse_cuda(relu=True)``), the product
    is ``ReluSparseDownProj``."""
    from .utils import dense_to_sparse_cuda
    values, _ri, row_offsets, column_indices = dense_to_sparse_cuda(hidden, index_dtype=index_dtype, relu=True)
    layer = ReluSparseDownProj(hidden.size(0), hidden.size(1), weight_t.size(0), device=hidden.device,
                               gather="none")
    return layer(values, row_offsets, column_indices, weight_t).clone()

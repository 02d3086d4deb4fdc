// Tensor-core (tcgen05 / TMEM / TMA) kernel for the fp16 branches of the hot path on sm_100a:
//   * dense linear          D[f, t] = sum_c W[f, c] * X[c, t]          (W streamed by TMA)
//   * CSR SpMM              D[r, t] = sum_p val[p] * X[col[p], t]      (CSR decoded to smem)
//   * fused sparse || dense both of the above in ONE launch, sharing X.
//
// One persistent, warp-specialised CTA design serves all three.  A CTA walks a list of
// work units; a unit is one 128-row tile of either branch over the whole K range (or one
// part of it).  Shared memory holds, for a dense unit, a ring of stages of a 128x128 fp16 A
// tile and a 128xN fp16 B tile; for a sparse unit, a ring of up to eight "A slots" (64
// columns of the tile, 16 KB each), a shorter ring of B slots (the matching 64 rows of X) and
// a ring of 128 nonzeros per row of the CSR stream -- all in the 128-byte-swizzled layout
// tcgen05.mma reads.  The two plans overlay each other; a CTA that changes kind between two
// units waits for the first to finish.
//
//   warp 0      TMA producer: B tiles (activations X) for every unit, A tiles (W) for dense
//               units, with cp.async.bulk.tensor + mbarrier complete_tx.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=tokens, K=16) into a
//               TMEM accumulator and releases stages / slots with tcgen05.commit.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (lane = output row), convert to
//               fp16, store.
//   warps 6..   CSR decoders (sparse units): stream the rows' values and column indices
//               with 16-byte cp.async copies straight from the CSR arrays (no re-packed
//               format, no per-tile metadata: a cursor per row advances through the
//               ascending column indices) and scatter every nonzero into whichever open A
//               slot its column falls in, then fence.proxy.async + mbarrier arrive for the
//               slots all their rows have passed.
//
// Dense units cost almost no instructions (TMA + MMA), sparse units are instruction-bound
// in the decoders, and both are fed from HBM, so co-resident CTAs working on units of
// different kinds overlap well: that is the horizontal fusion.  One CTA per SM; the work
// list is ordered so that the long (sparse) units start first and the CTAs that take a
// second unit are those that began with a short (dense) one.
//
// Every wait on an mbarrier is bounded; when a wait gives up the CTA raises a shared
// abort flag, records IEX_ERR_TIMEOUT in the status word, drains the copies it armed,
// frees its TMEM and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_prof.cuh"
#include "tc_ptx.cuh"

namespace iex {
namespace tc {

constexpr int BM = 128;                   // rows of A per unit (UMMA M)
constexpr int BK = 128;                   // K per stage: two 64-element swizzle atoms
constexpr int UMMA_K = 16;                // K per tcgen05.mma.kind::f16
constexpr int A_ATOM_BYTES = BM * 128;    // [128 rows x 64 fp16]
constexpr int A_STAGE_BYTES = 2 * A_ATOM_BYTES;
constexpr int kFirstDecodeWarp = 6;
constexpr int kDecodeWarps = 16;          // CSR decoder warps of the sparse-capable instance
constexpr int kMaxPeers = 8;              // GPUs of one box
constexpr int kMaxStages = 6;             // dense stages (barrier slots reserved)
constexpr int kMaxASlots = 8;             // sparse A slots of 64 columns (a power of two)
constexpr int kMaxBSlots = 4;             // sparse B slots (X rows of one 64-column block)
constexpr int kRingGranules = 16;         // 8-nonzero granules per row ring (128 nonzeros)

struct Params {
  // dense branch: out[f * d_stride_m + t * d_stride_n]
  int d_tiles, d_m;
  __half* d_out;
  long long d_stride_m, d_stride_n;
  // further copies of the dense output (the same slab in peer GPUs' buffers), written with
  // plain stores over NVLink by the same threads that write d_out
  __half* d_out_copies[kMaxPeers - 1];
  int d_num_copies;
  int d_b_mn;  // B operand of the dense branch is MN-major ([K, N]) instead of K-major ([N, K])
  int d_a_mn;  // A operand of the dense branch is MN-major ([K, M]) instead of K-major ([M, K])
  // Dense units over column blocks: with d_ncols > 0 the B operand is [K, d_ncols] (MN-major),
  // a unit is (128-row tile, block of n columns), and d_parts = d_nblocks counts the blocks
  // (no split-K).
  int d_nblocks, d_ncols;
  // sparse branch: out[r * n + t]
  int s_tiles, s_m, s_nnz;
  int s_tile_rows;  // rows of a sparse tile (a multiple of 8, <= 128; rows above it stay zero)
  __half* s_out;
  const int* s_row_offsets;
  const void* s_cols;
  const __half* s_values;
  const float* s_bias;  // optional: out = relu(sum + bias[row]) for the sparse branch
  IEX_PROF_FIELD
  // shared
  int k, n;
  int num_stages, tmem_cols;
  int* status;
  // shared-memory plan of sparse units: s_a_slots (2, 4 or 8) A slots of 16 KB at offset 0,
  // s_b_slots (2 or 4) B slots after them, the CSR rings at s_ring_offset; mbarriers at
  // bar_offset (past the larger of the dense and the sparse plan, which overlay each other)
  int s_a_slots, s_b_slots;
  int s_ring_rows;      // rows the rings are laid out for (>= s_tile_rows)
  uint32_t s_ring_offset, bar_offset;
  // dense units with a tokens-major output: 16 KB where the epilogue warps turn their rows of
  // the tile into 16-byte runs along the output's contiguous dimension (0: not available)
  uint32_t epi_offset;
  // split-K: every tile's K range is cut into `parts` equal runs of k-blocks, one unit
  // each.  With parts > 1 a unit writes its fp32 partial tile to `partials`
  // ([tile][part][128][n], sparse tiles first) and a second, tiny kernel adds the parts in
  // part order and writes the fp16 output.
  int s_parts, d_parts;
  float* partials;
};

__device__ int g_status = 0;  // last device-side failure (IEX_ERR_TIMEOUT) of this library

// Position u of the work list -> (is_sparse, tile, part).  With S = s_tiles * s_parts sparse
// units and D = d_tiles * d_parts dense units the list is
//   dense[0, e)  ++  sparse[0, S)  ++  dense[e, D)      with e = clamp(D + S - grid, 0, D),
// and CTA c takes positions c, c + grid, ...  Sparse units are the long ones (their cost
// is decoder work), so with at most two waves the CTAs that get a second unit are the ones
// that started with a (short) dense unit.  Parts of one tile are neighbours in the list,
// so they run at the same time and reach the reduction together.
struct Unit {
  bool sparse;
  int tile, part, parts;
  int nblock;  // column block of the B operand (dense units over column blocks), else 0
};
__device__ __forceinline__ Unit unit_of(int u, const Params& prm, int grid) {
  const int S = prm.s_tiles * prm.s_parts, D = prm.d_tiles * prm.d_parts;
  int e = D + S - grid;
  e = e < 0 ? 0 : (e > D ? D : e);
  Unit un;
  int idx;
  if (u < e) { un.sparse = false; idx = u; }
  else if (u < e + S) { un.sparse = true; idx = u - e; }
  else { un.sparse = false; idx = u - S; }
  un.parts = un.sparse ? prm.s_parts : prm.d_parts;
  un.tile = idx / un.parts;
  un.part = idx - un.tile * un.parts;
  un.nblock = 0;
  if (!un.sparse && prm.d_ncols > 0) {  // the "parts" of the list are column blocks
    un.nblock = un.part;
    un.part = 0;
    un.parts = 1;
  }
  return un;
}

// Eight consecutive nonzeros of one row as loaded: raw fp16 bit patterns and indices.
template <typename IT> struct Window {
  uint32_t v[4];
  uint32_t c[8 * sizeof(IT) / 4];
};
__device__ __forceinline__ uint32_t window_index(const Window<uint16_t>& w, int e) {
  return (e & 1) ? (w.c[e >> 1] >> 16) : (w.c[e >> 1] & 0xffffu);
}
__device__ __forceinline__ uint32_t window_index(const Window<int>& w, int e) { return w.c[e]; }
__device__ __forceinline__ void window_kill(Window<uint16_t>& w, int e) {
  w.c[e >> 1] |= (e & 1) ? 0xffff0000u : 0x0000ffffu;
}
__device__ __forceinline__ void window_kill(Window<int>& w, int e) { w.c[e] = 0xffffffffu; }

// Ring staging of the CSR stream.  Every row of the tile has a ring of 128 nonzeros
// (values and indices; kRingGranules "granules" of 8 nonzeros) in shared memory, addressed
// by position modulo the ring size, that is kept filled up to one ring size past the row's
// cursor with 16-byte cp.async copies.  Granules may start before the row or run past its
// end; what they hold there is masked when a window is read.

template <typename IT>
__device__ __forceinline__ void ring_issue(uint32_t vring, uint32_t cring, const __half* __restrict__ vals,
                                           const IT* __restrict__ cols, int g, int rend, int nnz,
                                           uint32_t rg_mask) {
  const int p = g * 8;
  if (p >= rend) return;  // nothing of this row there
  const uint32_t slot = static_cast<uint32_t>(g) & rg_mask;
  const uint32_t vdst = vring + slot * 16u;
  const uint32_t cdst = cring + slot * static_cast<uint32_t>(8 * sizeof(IT));
  if (p + 8 <= nnz) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vdst), "l"(vals + p) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(cdst), "l"(cols + p) : "memory");
    if constexpr (sizeof(IT) == 4)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(cdst + 16u), "l"(cols + p + 4)
                   : "memory");
  } else {  // last granule of the arrays: element-wise, inside the arrays
    for (int e = 0; e < 8 && p + e < nnz; ++e) {
      const uint16_t hv = __half_as_ushort(__ldg(vals + p + e));
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(vdst + 2u * e), "h"(hv) : "memory");
      if constexpr (sizeof(IT) == 2) {
        const uint16_t cv = __ldg(cols + p + e);
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(cdst + 2u * e), "h"(cv) : "memory");
      } else {
        const uint32_t cv = static_cast<uint32_t>(__ldg(cols + p + e));
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(cdst + 4u * e), "r"(cv) : "memory");
      }
    }
  }
}

// Reads nonzeros [my, my + 8) (my a multiple of 8) from the ring.  Positions outside
// [lo, rend) -- before the row's cursor or past the row's end -- get the largest index,
// which no open column range contains, so that the scatter loop needs a single unsigned
// compare per nonzero.
template <typename IT>
__device__ __forceinline__ void ring_read(Window<IT>& w, uint32_t vring, uint32_t cring, int my,
                                          int lo, int rend, uint32_t rg_mask) {
  constexpr int kC = 8 * sizeof(IT) / 4;
  if (my >= rend) {
#pragma unroll
    for (int e = 0; e < kC; ++e) w.c[e] = 0xffffffffu;
    return;
  }
  const uint32_t slot = static_cast<uint32_t>(my >> 3) & rg_mask;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(w.v[0]), "=r"(w.v[1]), "=r"(w.v[2]), "=r"(w.v[3])
               : "r"(vring + slot * 16u));
#pragma unroll
  for (int q = 0; q < kC / 4; ++q)
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w.c[4 * q]), "=r"(w.c[4 * q + 1]), "=r"(w.c[4 * q + 2]), "=r"(w.c[4 * q + 3])
                 : "r"(cring + slot * static_cast<uint32_t>(8 * sizeof(IT)) + 16u * q));
  if (my + 8 > rend || my < lo) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (my + e >= rend || my + e < lo) window_kill(w, e);
  }
}

// Writing a window into the A slots.  A slot is one 64-column swizzle atom ([128 rows x 128
// bytes]); the slots of consecutive 64-column blocks lie 16 KB apart in a power-of-two ring,
// so the slot of a column is a bit field of the column index:
//   address = (row part ^ column-in-atom part) + slot part.
// row_swz = (A region + row * 128) ^ ((row & 7) << 4); XOR-ing the byte column into it
// applies the 128-byte swizzle.  slot_bits = (slots - 1) << 6 selects the slot field.
__device__ __forceinline__ uint32_t slot_address(uint32_t c, uint32_t row_swz, uint32_t slot_bits) {
  return (row_swz ^ ((c << 1) & 126u)) + ((c & slot_bits) << 8);
}
template <typename IT>
__device__ __forceinline__ uint16_t window_value(const Window<IT>& w, int e) {
  return static_cast<uint16_t>((e & 1) ? (w.v[e >> 1] >> 16) : w.v[e >> 1]);
}
// Writes the window's nonzeros whose column is below open_end (masked positions hold the
// largest index and never are) and returns how many those were.
template <typename IT>
__device__ __forceinline__ int scatter_open(const Window<IT>& w, uint32_t open_end, uint32_t row_swz,
                                            uint32_t slot_bits) {
  int nvalid = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t c = window_index(w, e);
    if (c < open_end) {
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(slot_address(c, row_swz, slot_bits)),
                   "h"(window_value(w, e))
                   : "memory");
      ++nvalid;
    }
  }
  return nvalid;
}
// Sum over the 8 lanes of a row group (xor butterfly; all four groups of a warp at once).
__device__ __forceinline__ int group8_sum(int v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

// For each of a warp's kIters rows (one per group of 8 lanes): the first position p in
// [lo, hi) with cols[p] >= key (hi when there is none).  Every step each lane probes one
// position of its row's range -- the first step around the position a uniform spread of the
// row's columns would put the key at (16 apart), later steps evenly over what is left -- and
// the range shrinks to the gap between the last probe below the key and the first one not
// below it.  The rows of all groups and iterations advance together, so a step costs one
// global-memory round trip for the whole warp; with roughly uniform columns two or three
// steps suffice and they touch neighbouring cache lines.  lo[] is the answer on return.
template <typename IT, int kIters>
__device__ __forceinline__ void rows_lower_bound(const IT* __restrict__ cols, int (&lo)[kIters],
                                                 int (&hi)[kIters], int key, int k, int sl, unsigned gmask) {
  const int shift = __ffs(gmask) - 1;
  bool first = true;
  for (int guard = 0; guard < 40; ++guard) {
    bool open = false;
#pragma unroll
    for (int i = 0; i < kIters; ++i) open = open || hi[i] > lo[i];
    if (!__any_sync(0xffffffffu, open)) break;
    int base[kIters], stride[kIters];
    bool below[kIters];
#pragma unroll
    for (int i = 0; i < kIters; ++i) {
      const int len = hi[i] - lo[i];
      if (first) {  // around the estimate, 16 apart
        const int est = lo[i] + static_cast<int>(static_cast<long long>(len) * key / (k > 0 ? k : 1));
        base[i] = est - 56;
        stride[i] = 16;
      } else {      // evenly: the probes split the range into nine runs
        stride[i] = (len + 8) / 9;
        base[i] = lo[i] + stride[i] - 1;
      }
      int q = base[i] + sl * stride[i];
      q = q < lo[i] ? lo[i] : (q > hi[i] - 1 ? hi[i] - 1 : q);
      below[i] = len > 0 && to_index(__ldg(cols + q)) < key;
    }
#pragma unroll
    for (int i = 0; i < kIters; ++i) {
      const int nb = __popc((__ballot_sync(gmask, below[i]) >> shift) & 0xffu);  // monotone: a prefix
      if (hi[i] > lo[i]) {
        const int l0 = lo[i], h0 = hi[i];
        auto probe = [&](int j) {
          const int q = base[i] + j * stride[i];
          return q < l0 ? l0 : (q > h0 - 1 ? h0 - 1 : q);
        };
        if (nb > 0) lo[i] = probe(nb - 1) + 1;
        if (nb < 8) hi[i] = probe(nb);
        if (hi[i] < lo[i]) hi[i] = lo[i];
      }
    }
    first = false;
  }
}

// ND = number of CSR decoder warps (0: dense-only instance).
template <int ND, typename IT>
__global__ void __launch_bounds__((kFirstDecodeWarp + ND) * 32, 1)
tc_units_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b_dense,
                const __grid_constant__ CUtensorMap tma_b_sparse, const Params prm) {
  extern __shared__ uint8_t smem_raw[];
  IEX_PROF_STAMP(threadIdx.x == 0, 42)
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int n = prm.n;
  // dense units: ring of S stages, each [A 128x128 | B 128xN]
  const uint32_t b_stage_bytes = static_cast<uint32_t>(n) * 256u;
  const uint32_t stage_bytes = A_STAGE_BYTES + b_stage_bytes;
  const int S = prm.num_stages;
  // sparse units: SA A slots of 64 columns, then SB B slots (X rows of a 64-column block),
  // then the CSR rings
  const int SA = prm.s_a_slots, SB = prm.s_b_slots;
  const uint32_t s_b_slot_bytes = static_cast<uint32_t>(n) * 128u;
  const uint32_t s_b_region = smem_base + static_cast<uint32_t>(SA) * A_ATOM_BYTES;
  const uint32_t bar_base = smem_base + prm.bar_offset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                          // dense
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  // sparse: A slots are filled by the decoder warps and released by the tensor-core warp;
  // B slots are filled by the producer's TMA loads
  auto a_full_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + s); };
  auto a_empty_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + kMaxASlots + s); };
  auto b_full_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + 2 * kMaxASlots + s); };
  auto b_empty_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + 2 * kMaxASlots + kMaxBSlots + s); };
  constexpr uint32_t kBarCount = 2 * kMaxStages + 2 * kMaxASlots + 2 * kMaxBSlots;
  const uint32_t accum_full = bar_base + 8u * kBarCount;
  const uint32_t accum_empty = accum_full + 8u;
  const uint32_t tmem_slot = accum_full + 16u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_generic =
      reinterpret_cast<volatile uint32_t*>(smem_aligned + prm.bar_offset + 8u * kBarCount + 16u);
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_aligned + prm.bar_offset + 8u * kBarCount + 20u);
  // number of this CTA's units whose accumulator is complete (all tensor-core reads of
  // shared memory done); written by the first epilogue warp
  volatile uint32_t* units_done =
      reinterpret_cast<volatile uint32_t*>(smem_aligned + prm.bar_offset + 8u * kBarCount + 24u);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_units = prm.d_tiles * prm.d_parts + prm.s_tiles * prm.s_parts;
  const int k_blocks = (prm.k + BK - 1) / BK;   // dense: 128 columns per stage
  const int k_slots = (prm.k + 63) / 64;        // sparse: 64 columns per slot

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < kMaxASlots; ++s) {
      mbar_init(a_full_bar(s), ND > 0 ? ND : 1);
      mbar_init(a_empty_bar(s), 1);
    }
    for (int s = 0; s < kMaxBSlots; ++s) {
      mbar_init(b_full_bar(s), 1);
      mbar_init(b_empty_bar(s), 1);
    }
    mbar_init(accum_full, 1);
    mbar_init(accum_empty, 4);
    *abort_flag = 0;
    *units_done = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(static_cast<uint32_t>(prm.tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_generic;
  IEX_PROF_STAMP(threadIdx.x == 0, 43)
  // Everything above touched only this CTA's own shared and tensor memory and may overlap the
  // end of the kernel before this one in the stream; global memory comes next.
  grid_dependency_wait();
  grid_launch_dependents();
  IEX_PROF_STAMP(threadIdx.x == 0, 45)

  // Dense stages and sparse slots / rings overlay the same shared memory.  A role that writes
  // shared memory for a unit whose kind differs from the CTA's previous unit first waits until
  // the previous unit's accumulator is complete (units_done): every tensor-core read and
  // every TMA copy of that unit has finished by then, and so have the decoders' ring copies,
  // which have all landed before they release a unit's last slot.
  auto wait_units_done = [&](uint32_t want) -> bool {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
      if (*units_done >= want) { __threadfence_block(); return true; }
      __nanosleep(64);
      if ((i & 63u) == 63u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(prm.status, IEX_ERR_TIMEOUT);
    return false;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_b_dense) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_b_sparse) : "memory");
      uint32_t it = 0, unit_it = 0, b_empty_ph = 0;
      bool ok = true, prev_sparse = false;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++unit_it) {
        const Unit un = unit_of(u, prm, gridDim.x);
        const int tile = un.tile;
        if (unit_it > 0 && un.sparse != prev_sparse && !wait_units_done(unit_it)) { ok = false; break; }
        prev_sparse = un.sparse;
        if (un.sparse) {
          const int kb0 = un.part * k_slots / un.parts, kb1 = (un.part + 1) * k_slots / un.parts;
          for (int kb = kb0; kb < kb1; ++kb) {
            const int s = kb & (SB - 1);
            if (!mbar_wait(b_empty_bar(s), ((b_empty_ph >> s) & 1u) ^ 1u, abort_flag, prm.status, 64)) {
              ok = false;
              break;
            }
            b_empty_ph ^= 1u << s;
            const uint32_t b_dst = s_b_region + s * s_b_slot_bytes;
            mbar_arrive_expect_tx(b_full_bar(s), s_b_slot_bytes);
            // X [K, N]: one [64 k-rows x 64 cols] box per 64 columns
            for (int j = 0; j < n / 64; ++j)
              tma_load_2d(b_dst + j * (64 * 128), &tma_b_sparse, b_full_bar(s), j * 64, kb * 64);
          }
        } else {
          const int kb0 = un.part * k_blocks / un.parts, kb1 = (un.part + 1) * k_blocks / un.parts;
          const bool b_mn = prm.d_b_mn;
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const int s = it % S;
            const uint32_t ph = (it / S) & 1u;
            if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, prm.status, 64)) { ok = false; break; }
            const uint32_t a_dst = smem_base + s * stage_bytes;
            const uint32_t b_dst = a_dst + A_STAGE_BYTES;
            mbar_arrive_expect_tx(full_bar(s), b_stage_bytes + A_STAGE_BYTES);
            if (prm.d_a_mn) {  // A [K, M]: two [128 k-rows x 64 cols] boxes
              tma_load_2d(a_dst, &tma_a, full_bar(s), tile * BM, kb * BK);
              tma_load_2d(a_dst + A_ATOM_BYTES, &tma_a, full_bar(s), tile * BM + 64, kb * BK);
            } else {
              tma_load_2d(a_dst, &tma_a, full_bar(s), kb * BK, tile * BM);
              tma_load_2d(a_dst + A_ATOM_BYTES, &tma_a, full_bar(s), kb * BK + 64, tile * BM);
            }
            if (b_mn) {  // X [K, N]: one [128 k-rows x 64 cols] box per 64 columns
              for (int j = 0; j < n / 64; ++j)
                tma_load_2d(b_dst + j * (BK * 128), &tma_b_dense, full_bar(s), un.nblock * n + j * 64, kb * BK);
            } else {  // X^T [N, K]: two [N rows x 64 k] boxes
              tma_load_2d(b_dst, &tma_b_dense, full_bar(s), kb * BK, 0);
              tma_load_2d(b_dst + n * 128, &tma_b_dense, full_bar(s), kb * BK + 64, 0);
            }
          }
        }
      }
      if (!ok) {
        // Drain: give the copies this thread armed a bounded time (~0.2 ms) to land.
        for (uint32_t i = 0; i < 2048u; ++i) __nanosleep(100);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_k = (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (8u << 24);
      const uint32_t idesc_mn = idesc_k | (1u << 16);
      uint32_t it = 0, unit_it = 0, a_full_ph = 0, b_full_ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++unit_it) {
        const Unit un = unit_of(u, prm, gridDim.x);
        if (!mbar_wait(accum_empty, (unit_it & 1u) ^ 1u, abort_flag, prm.status, 64)) { ok = false; break; }
        tcgen05_fence_after();
        if (un.sparse) {
          const int kb0 = un.part * k_slots / un.parts, kb1 = (un.part + 1) * k_slots / un.parts;
          for (int kb = kb0; kb < kb1; ++kb) {
            const int sa = kb & (SA - 1), sb = kb & (SB - 1);
            if (!mbar_wait(b_full_bar(sb), (b_full_ph >> sb) & 1u, abort_flag, prm.status, 32)) { ok = false; break; }
            b_full_ph ^= 1u << sb;
            if (!mbar_wait(a_full_bar(sa), (a_full_ph >> sa) & 1u, abort_flag, prm.status, 32)) { ok = false; break; }
            a_full_ph ^= 1u << sa;
            tcgen05_fence_after();
            const uint32_t a_base = smem_base + sa * A_ATOM_BYTES;
            const uint32_t b_base = s_b_region + sb * s_b_slot_bytes;
            const uint64_t adesc0 = smem_desc(a_base, 16, 1024);
            const uint64_t bdesc0 = smem_desc(b_base, 64 * 128, 1024);
#pragma unroll
            for (int ks = 0; ks < 64 / UMMA_K; ++ks)
              umma_f16(tmem_base, desc_advance(adesc0, ks * 32), desc_advance(bdesc0, ks * (UMMA_K * 128)),
                       idesc_mn, (kb != kb0 || ks != 0) ? 1u : 0u);
            umma_commit(a_empty_bar(sa));
            umma_commit(b_empty_bar(sb));
          }
        } else {
          const int kb0 = un.part * k_blocks / un.parts, kb1 = (un.part + 1) * k_blocks / un.parts;
          const bool b_mn = prm.d_b_mn, a_mn = prm.d_a_mn;
          const uint32_t idesc = (b_mn ? idesc_mn : idesc_k) | (a_mn ? (1u << 15) : 0u);
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const int s = it % S;
            const uint32_t ph = (it / S) & 1u;
            if (!mbar_wait(full_bar(s), ph, abort_flag, prm.status, 32)) { ok = false; break; }
            IEX_PROF_STAMP(it == 0, 46)
            tcgen05_fence_after();
            const uint32_t a_base = smem_base + s * stage_bytes;
            const uint32_t b_base = a_base + A_STAGE_BYTES;
            // K-major A: two 64-wide K atoms of 128 rows; MN-major A: two 64-wide M atoms of 128 k-rows
            const uint64_t adesc0 = a_mn ? smem_desc(a_base, BK * 128, 1024) : smem_desc(a_base, 16, 1024);
            auto a_step = [&](int ks) {
              return a_mn ? desc_advance(adesc0, ks * (UMMA_K * 128))
                          : desc_advance(adesc0, (ks >> 2) * A_ATOM_BYTES + (ks & 3) * 32);
            };
            if (b_mn) {
              const uint64_t bdesc0 = smem_desc(b_base, BK * 128, 1024);
#pragma unroll
              for (int ks = 0; ks < BK / UMMA_K; ++ks)
                umma_f16(tmem_base, a_step(ks), desc_advance(bdesc0, ks * (UMMA_K * 128)), idesc,
                         (kb != kb0 || ks != 0) ? 1u : 0u);
            } else {
              const uint64_t bdesc0 = smem_desc(b_base, 16, 1024);
              const uint32_t b_atom = static_cast<uint32_t>(n) * 128u;  // second 64-wide K atom of B
#pragma unroll
              for (int ks = 0; ks < BK / UMMA_K; ++ks)
                umma_f16(tmem_base, a_step(ks), desc_advance(bdesc0, (ks >> 2) * b_atom + (ks & 3) * 32), idesc,
                         (kb != kb0 || ks != 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(s));
          }
        }
        if (ok) umma_commit(accum_full);
        IEX_PROF_STAMP(true, 47)
      }
    }
  } else if (warp < kFirstDecodeWarp) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t unit_it = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++unit_it) {
      const Unit un = unit_of(u, prm, gridDim.x);
      const bool sparse = un.sparse;
      const int tile = un.tile;
      if (!mbar_wait(accum_full, unit_it & 1u, abort_flag, prm.status, 256)) { ok = false; break; }
      IEX_PROF_STAMP(warp == 2 && lane == 0, 48)
      tcgen05_fence_after();
      if (warp == 2 && lane == 0) {
        __threadfence_block();
        *units_done = unit_it + 1u;
      }
      const int row_local = q * 32 + lane;
      const int tile_rows = sparse ? prm.s_tile_rows : BM;
      const int row = tile * tile_rows + row_local;
      const bool row_stored = row_local < tile_rows && row < (sparse ? prm.s_m : prm.d_m);
      __half* out = sparse ? prm.s_out : prm.d_out;
      const long long sm = sparse ? static_cast<long long>(n) : prm.d_stride_m;
      const long long sn = sparse ? 1ll : prm.d_stride_n;
      // partial tiles of this output tile: [part][n columns][128 rows] fp32
      float* part_base = prm.partials == nullptr ? nullptr
          : prm.partials + (static_cast<size_t>(sparse ? tile * prm.s_parts
                                                        : prm.s_tiles * prm.s_parts + tile * prm.d_parts)) *
                               (static_cast<size_t>(BM) * n);
      // final (not partial) dense tiles whose output runs along the rows take the staged path
      const bool staged = !sparse && un.parts == 1 && prm.epi_offset != 0u;
      for (int c0 = 0; c0 < n; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 >= n) {  // accumulator fully read: let the next unit's MMAs start
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(accum_empty);
        }
        if (staged) {
          // Tokens-major output: column c of the tile is a run of 128 rows in memory.  Each warp
          // turns its 32 rows x 32 columns into 16-byte pieces (8 rows of one column) through
          // its own 2 KB of shared memory and stores those: 4 vector stores per lane instead of
          // 32 two-byte ones.  Only lanes of the warp meet, so no barrier beyond __syncwarp.
          const uint32_t mine = smem_base + prm.epi_offset + static_cast<uint32_t>(q) * 2048u;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint16_t h = __half_as_ushort(__float2half_rn(__uint_as_float(r[i])));
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(mine + i * 64 + lane * 2), "h"(h) : "memory");
          }
          __syncwarp();
          const int row0 = tile * BM + q * 32;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int v = lane + 32 * j;         // piece v: column v >> 2 of the chunk, rows 8 * (v & 3) ..
            const int col = v >> 2, piece = v & 3;
            uint4 pk;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(pk.x), "=r"(pk.y), "=r"(pk.z), "=r"(pk.w)
                         : "r"(mine + col * 64 + piece * 16)
                         : "memory");
            const int rr = row0 + piece * 8;
            if (rr < prm.d_m && c0 + col < n) {
              const long long off = static_cast<long long>(c0 + col) * prm.d_stride_n + rr;
              *reinterpret_cast<uint4*>(prm.d_out + off) = pk;
              for (int pe = 0; pe < prm.d_num_copies; ++pe) *reinterpret_cast<uint4*>(prm.d_out_copies[pe] + off) = pk;
            }
          }
          __syncwarp();  // the pieces are read before the next chunk overwrites them
        } else if (un.parts > 1) {
          // partial tile stored column-major ([n][128]): the 32 lanes of a warp hold 32
          // consecutive rows, so every store below is one coalesced 128-byte line
          float* dst = part_base + static_cast<size_t>(un.part) * BM * n + static_cast<size_t>(c0) * BM +
                       row_local;
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[i * BM] = __uint_as_float(r[i]);
        } else if (row_stored) {
          if (sparse && prm.s_bias != nullptr) {  // bias + ReLU epilogue of the sparse branch
            const float bias = __ldg(prm.s_bias + row);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(fmaxf(__uint_as_float(r[i]) + bias, 0.f));
          }
          const int copies = sparse ? 0 : prm.d_num_copies;
          // dense units over column blocks: this unit's columns start at col0, the last block
          // may be narrower (a multiple of 8 columns)
          const int col0 = un.nblock * n;
          const int n_valid = (!sparse && prm.d_ncols > 0) ? min(n, prm.d_ncols - col0) : n;
          for (int pe = 0; pe <= copies; ++pe) {
            __half* o = pe == 0 ? out : prm.d_out_copies[pe - 1];
            if (sn == 1) {
              uint4* dst = reinterpret_cast<uint4*>(o + row * sm + col0 + c0);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 pk;
                __half2* h = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  h[i] = __floats2half2_rn(__uint_as_float(r[v * 8 + 2 * i]),
                                           __uint_as_float(r[v * 8 + 2 * i + 1]));
                if (c0 + v * 8 < n_valid) dst[v] = pk;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c0 + i < n_valid)  // n need not be a multiple of the 32 columns read at a time
                  o[row * sm + (col0 + c0 + i) * sn] = __float2half_rn(__uint_as_float(r[i]));
            }
          }
        }
      }
    }
  } else if (ND > 0) {
    // ------------------------------------------------------------------ CSR decoders
    // Each warp owns kRowsPerWarp rows of the tile; a group of 8 lanes works on one row,
    // four rows per pass.  The rows are decoded as a data flow: in every round a row group
    // reads the next 64 nonzeros of its row (a "window", from the row's shared-memory ring)
    // and writes those whose column lies below the end of the open slots -- wherever they
    // fall among these -- so no nonzero is read twice except where a window is cut at that
    // end.  Open slots are the ones the tensor-core warp is done with (the warp then clears
    // its own rows of the slot) and this warp has not yet released.  A warp releases slot j
    // (arrives on its full barrier) once every one of its rows has moved past column
    // 64 * (j + 1); the tensor-core warp consumes a slot when all decoder warps have released
    // it and X's rows for it have landed.
    // After each round the ring is topped up to one ring size past the new cursor, so
    // global-memory latency is a round away from use.
    constexpr int kNd = ND > 0 ? ND : 1;
    constexpr int kRowsPerWarp = BM / kNd;
    constexpr int kIters = kRowsPerWarp / 4;
    static_assert(ND == 0 || (BM % kNd == 0 && kRowsPerWarp % 4 == 0), "decoder split");
    const int dw = warp - kFirstDecodeWarp;
    const int grp = lane >> 3, sl = lane & 7;
    const unsigned gmask = 0xffu << (grp * 8);
    const IT* cols = static_cast<const IT*>(prm.s_cols);
    const __half* vals = prm.s_values;
    const int nnz = prm.s_nnz;
    const uint32_t ring_base = smem_base + prm.s_ring_offset;  // 16-byte aligned
    constexpr int rg = kRingGranules;
    constexpr uint32_t rg_mask = static_cast<uint32_t>(rg - 1);
    const uint32_t slot_bits = static_cast<uint32_t>(SA - 1) << 6;
    uint32_t unit_it = 0, a_empty_ph = 0;
    bool ok = true, prev_sparse = false;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++unit_it) {
      const Unit un = unit_of(u, prm, gridDim.x);
      if (!un.sparse) { prev_sparse = false; continue; }
      const int tile = un.tile;
      const int kb0 = un.part * k_slots / un.parts, kb1 = (un.part + 1) * k_slots / un.parts;
      // the rings overlay the stages of a dense unit before this one
      if (unit_it > 0 && !prev_sparse && !wait_units_done(unit_it)) { ok = false; break; }
      prev_sparse = true;
      if (dw * kRowsPerWarp >= prm.s_tile_rows) {
        // None of this warp's rows belongs to the (lower than 128 rows) tile.  Its part of the
        // protocol: keep its rows of every slot zero -- cleared once per unit, nobody writes
        // them afterwards -- and release each slot as soon as the tensor-core warp has let go
        // of the slot's previous contents.
        bool cleared = false;
        for (int kb = kb0; kb < kb1; ++kb) {
          const int s = kb & (SA - 1);
          if (!mbar_wait(a_empty_bar(s), ((a_empty_ph >> s) & 1u) ^ 1u, abort_flag, prm.status, 128)) {
            ok = false;
            break;
          }
          a_empty_ph ^= 1u << s;
          if (!cleared) {
            if (kb - kb0 + 1 >= SA || kb + 1 == kb1) cleared = true;
#pragma unroll
            for (int q4 = 0; q4 < kRowsPerWarp / 4; ++q4)
              asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(
                               smem_base + s * A_ATOM_BYTES + (dw * kRowsPerWarp + q4 * 4) * 128 + lane * 16),
                           "r"(0u)
                           : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(a_full_bar(s));
        }
        continue;
      }
      int cur[kIters], rend[kIters], filled[kIters];
      uint32_t vring[kIters], cring[kIters], row_swz[kIters];
#pragma unroll
      for (int i = 0; i < kIters; ++i) {
        const int row_local = dw * kRowsPerWarp + i * 4 + grp;
        const int row = tile * prm.s_tile_rows + row_local;
        const bool in = row_local < prm.s_tile_rows && row < prm.s_m;
        cur[i] = in ? __ldg(prm.s_row_offsets + row) : 0;
        rend[i] = in ? __ldg(prm.s_row_offsets + row + 1) : 0;
      }
      if (kb0 > 0) {  // this part starts inside the rows: first nonzero with column >= kb0 * 64
        int hi_s[kIters];
#pragma unroll
        for (int i = 0; i < kIters; ++i) hi_s[i] = rend[i];
        rows_lower_bound<IT, kIters>(cols, cur, hi_s, kb0 * 64, prm.k, sl, gmask);
      }
#pragma unroll
      for (int i = 0; i < kIters; ++i) {
        const int row_local = dw * kRowsPerWarp + i * 4 + grp;
        vring[i] = ring_base + row_local * (rg * 16u);
        cring[i] = ring_base + prm.s_ring_rows * (rg * 16u) +
                   row_local * (rg * 8u * static_cast<uint32_t>(sizeof(IT)));
        row_swz[i] = (smem_base + row_local * 128) ^ (static_cast<uint32_t>(row_local & 7) << 4);
        const int g0 = cur[i] >> 3;
        for (int j = 0; j < rg; j += 8)
          ring_issue<IT>(vring[i], cring[i], vals, cols, g0 + j + sl, rend[i], nnz, rg_mask);
        filled[i] = g0 + rg;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.commit_group;" ::: "memory");  // so that wait_group 1 covers the fill
      int lo = kb0, hi = kb0;  // slots [lo, hi) are open for this warp
      while (lo < kb1) {
        // open further slots that the tensor-core warp has released; wait when none is open
        while (hi < kb1 && hi < lo + SA) {
          const int s = hi & (SA - 1);
          const uint32_t ph = ((a_empty_ph >> s) & 1u) ^ 1u;
          if (hi == lo) {
            if (!mbar_wait(a_empty_bar(s), ph, abort_flag, prm.status, 32)) { ok = false; break; }
          } else if (!mbar_test_wait(a_empty_bar(s), ph)) {
            break;
          }
          a_empty_ph ^= 1u << s;
          ++hi;
          // clear this warp's rows of the slot: 8 rows x 128 bytes, 32 bytes per lane
          // (16 bytes per lane and 4 rows)
          const uint32_t slot_addr = smem_base + s * A_ATOM_BYTES;
#pragma unroll
          for (int q4 = 0; q4 < kRowsPerWarp / 4; ++q4)
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(
                             slot_addr + (dw * kRowsPerWarp + q4 * 4) * 128 + lane * 16), "r"(0u)
                         : "memory");
        }
        if (!ok) break;
        const uint32_t open_end = static_cast<uint32_t>(hi) * 64u;
        // everything but the newest top-ups has landed; make it (and the cleared rows)
        // visible to the warp
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncwarp();
        Window<IT> w[kIters];
        int base[kIters];
#pragma unroll
        for (int i = 0; i < kIters; ++i) {
          base[i] = cur[i] & ~7;
          ring_read<IT>(w[i], vring[i], cring[i], base[i] + sl * 8, cur[i], rend[i], rg_mask);
        }
        uint32_t bound = 0xffffffffu;  // every row of this warp is done below this column
        int tots[kIters];
#pragma unroll
        for (int i = 0; i < kIters; ++i)
          tots[i] = group8_sum(scatter_open<IT>(w[i], open_end, row_swz[i], slot_bits));
#pragma unroll
        for (int i = 0; i < kIters; ++i) {
          const int tot = tots[i];
          const int avail = min(rend[i], base[i] + 64) - cur[i];  // nonzeros of the row in the window
          const uint32_t last_col = __shfl_sync(0xffffffffu, window_index(w[i], 7), grp * 8 + 7);
          cur[i] += tot;
          // cut at the end of the open slots | row finished | window used up: the row's next
          // column is above the window's last one
          const uint32_t b = tot < avail ? open_end : (cur[i] >= rend[i] ? 0xffffffffu : last_col + 1u);
          bound = b < bound ? b : bound;
        }
        // top the rings up to one ring size past the new window bases
#pragma unroll
        for (int i = 0; i < kIters; ++i) {
          const int limit = (cur[i] >> 3) + rg;
          const int g = filled[i] + sl;
          if (g < limit) ring_issue<IT>(vring[i], cring[i], vals, cols, g, rend[i], nnz, rg_mask);
          filled[i] = limit > filled[i] ? limit : filled[i];
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        {
          const uint32_t o8 = __shfl_xor_sync(0xffffffffu, bound, 8);
          bound = o8 < bound ? o8 : bound;
          const uint32_t o16 = __shfl_xor_sync(0xffffffffu, bound, 16);
          bound = o16 < bound ? o16 : bound;
        }
        int ready = static_cast<int>(bound >> 6);
        ready = ready > hi ? hi : ready;
        if (ready > lo) {
          if (ready == kb1)  // nothing of this unit may still be landing when its last slot goes
            asm volatile("cp.async.wait_group 0;" ::: "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0)
            for (int j = lo; j < ready; ++j) mbar_arrive(a_full_bar(j & (SA - 1)));
          lo = ready;
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
    }
  }

  // ---------------------------------------------------------------------- teardown
  IEX_PROF_STAMP(warp == 2 && lane == 0, 49)
  tcgen05_fence_before();
  __syncthreads();
  IEX_PROF_STAMP(threadIdx.x == 0, 44)
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(prm.tmem_cols))
                 : "memory");
  }
}

// Second pass of split-K: out tile = sum over parts (in part order) of the fp32 partial
// tiles, converted to fp16.  grid = (split tiles, slices) with one float4 of output per
// thread, so the whole reduction is a handful of dependent L2 round trips deep no matter how
// large the tile is; the loads of eight parts are in flight per thread.
constexpr int kReduceThreads = 256;

__global__ void __launch_bounds__(kReduceThreads)
tc_reduce_kernel(const Params prm) {
  grid_dependency_wait();  // the partial tiles come from the kernel before this one
  grid_launch_dependents();
  const int n = prm.n;
  const int s_split = prm.s_parts > 1 ? prm.s_tiles : 0;
  const bool sparse = static_cast<int>(blockIdx.x) < s_split;
  const int tile = sparse ? blockIdx.x : blockIdx.x - s_split;
  const int parts = sparse ? prm.s_parts : prm.d_parts;
  const int rows = sparse ? prm.s_m : prm.d_m;
  __half* out = sparse ? prm.s_out : prm.d_out;
  const long long sm = sparse ? static_cast<long long>(n) : prm.d_stride_m;
  const long long sn = sparse ? 1ll : prm.d_stride_n;
  const size_t part_stride = static_cast<size_t>(BM) * n;
  const float* base = prm.partials +
      static_cast<size_t>(sparse ? tile * prm.s_parts : prm.s_tiles * prm.s_parts + tile * prm.d_parts) *
          part_stride;
  // Partial tiles are column-major ([n][128]); a float4 holds 4 consecutive rows of one column.
  const int total_vecs = n * (BM / 4);
  for (int f = blockIdx.y * kReduceThreads + threadIdx.x; f < total_vecs; f += gridDim.y * kReduceThreads) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    int pp = 0;
    for (; pp + 8 <= parts; pp += 8) {
      float4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        t[u] = __ldcg(reinterpret_cast<const float4*>(base + (pp + u) * part_stride) + f);
#pragma unroll
      for (int u = 0; u < 8; ++u) { sum.x += t[u].x; sum.y += t[u].y; sum.z += t[u].z; sum.w += t[u].w; }
    }
    {
      float4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        t[u] = (pp + u < parts) ? __ldcg(reinterpret_cast<const float4*>(base + (pp + u) * part_stride) + f)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (pp + u < parts) { sum.x += t[u].x; sum.y += t[u].y; sum.z += t[u].z; sum.w += t[u].w; }
    }
    const int col = f / (BM / 4), rl = (f - col * (BM / 4)) * 4;
    const int tile_rows = sparse ? prm.s_tile_rows : BM;
    if (rl >= tile_rows) continue;
    const int orow = tile * tile_rows + rl;
    const float vals4[4] = {sum.x, sum.y, sum.z, sum.w};
    const int copies = sparse ? 0 : prm.d_num_copies;
    for (int pe = 0; pe <= copies; ++pe) {
      __half* o = pe == 0 ? out : prm.d_out_copies[pe - 1];
      if (sm == 1 && orow + 3 < rows) {  // rows contiguous in the output: one 8-byte store
        uint2 pk;
        __half2* h = reinterpret_cast<__half2*>(&pk);
        h[0] = __floats2half2_rn(sum.x, sum.y);
        h[1] = __floats2half2_rn(sum.z, sum.w);
        __half* dst = o + orow + col * sn;
        if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) { *reinterpret_cast<uint2*>(dst) = pk; continue; }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (orow + j < rows) o[(orow + j) * sm + col * sn] = __float2half_rn(vals4[j]);
    }
  }
}

// Barrier among the GPUs of one box over peer memory.  sig[r] points at rank r's signal
// array of world + 1 words in memory every rank can reach: word q of rank r's array is
// written by rank q, the last word is rank r's own epoch counter.  One block per GPU:
// thread q publishes this rank's new epoch in rank q's array (after a system-wide fence, so
// that everything this GPU stored before -- the output slabs in the peers' buffers -- is
// visible first) and then waits, for a bounded time, until rank q's epoch has arrived here.
struct PeerSignals {
  uint32_t* sig[kMaxPeers];
  int world, rank;
  int* status;
  uint32_t max_polls;  // polls of ~100 ns each before the wait gives up
};
constexpr uint32_t kPeerSpinLimit = 1u << 22;  // default limit: a fraction of a second

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerSignals ps) {
  __shared__ uint32_t epoch_s;
  grid_dependency_wait();  // the stores this barrier publishes come from the kernel before it
  grid_launch_dependents();
  if (threadIdx.x == 0) {
    uint32_t* mine = ps.sig[ps.rank] + ps.world;
    epoch_s = *mine + 1u;
    *mine = epoch_s;
  }
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const int q = threadIdx.x;
  if (q < ps.world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ps.sig[q] + ps.rank), "r"(epoch) : "memory");
    const uint32_t* src = ps.sig[ps.rank] + q;
    bool arrived = false;
    for (uint32_t i = 0; i < ps.max_polls; ++i) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      if (static_cast<int>(v - epoch) >= 0) { arrived = true; break; }
      __nanosleep(100);
    }
    if (!arrived) {
      atomicExch(ps.status, IEX_ERR_TIMEOUT);
      atomicExch(&g_status, IEX_ERR_TIMEOUT);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Row-major fp16 matrix [rows, cols] (cols contiguous); box = [box_rows x 64 cols], 128B swizzle.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return IEX_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IEX_OK : IEX_ERR_DRIVER;
}

// Per-device host state.  One process may drive several GPUs (the torch operators accept
// tensors on any device), and both the SM count and the opt-in dynamic shared-memory limit of
// a kernel belong to a device, so they are remembered per device index under a mutex.
constexpr int kMaxDevices = 64;
std::mutex g_device_mutex;
int g_sm_count[kMaxDevices] = {};

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

int sm_count() {
  const int dev = current_device();
  if (dev < 0) return kNumSMs;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (g_sm_count[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = kNumSMs;
    g_sm_count[dev] = v;
  }
  return g_sm_count[dev];
}

int* status_word() {
  int* p = nullptr;
  cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status);
  return p;
}

// Shared-memory budget for stages / slots / rings (227 KB per CTA minus alignment slack and
// the mbarrier block).
constexpr int kBarBytes = 8 * (2 * kMaxStages + 2 * kMaxASlots + 2 * kMaxBSlots + 2) + 16;
constexpr int kDataBudget = 227 * 1024 - 1024 - kBarBytes - 64;

int dense_stages(int n, int cap) {
  const int stage_bytes = A_STAGE_BYTES + n * 256;
  const int stages = kDataBudget / stage_bytes;
  return stages > cap ? cap : stages;
}

// Sparse plan: as many A slots (64 columns of the 128-row tile, 16 KB) and B slots (the
// matching 64 rows of X) as fit beside the CSR rings; `rows` = rows of a tile that are in use
// (the rings are laid out for those only).  More A slots matter most; two B slots do as
// well as four (measured).
struct SparsePlan { int a_slots, b_slots; };
bool sparse_plan(int n, int index_bits, int rows, SparsePlan* plan) {
  static const SparsePlan kPlans[] = {{8, 4}, {8, 2}, {4, 4}, {4, 2}, {2, 2}};
  const int ring = rows * kRingGranules * 8 * (2 + index_bits / 8);
  for (const auto& pl : kPlans) {
    if (pl.a_slots * A_ATOM_BYTES + pl.b_slots * n * 128 + ring <= kDataBudget) {
      *plan = pl;
      return true;
    }
  }
  return false;
}

template <int ND, typename IT>
int launch_units(const CUtensorMap& ta, const CUtensorMap& tbd, const CUtensorMap& tbs, Params prm,
                 int stages, int ctas_per_sm, cudaStream_t stream) {
  prm.num_stages = stages;
  size_t data = static_cast<size_t>(stages) * (A_STAGE_BYTES + prm.n * 256);
  prm.s_a_slots = 1;
  prm.s_b_slots = 1;
  prm.s_ring_rows = BM;
  prm.s_ring_offset = 0;
  if (ND > 0) {
    SparsePlan plan{};
    prm.s_ring_rows = (prm.s_tile_rows + 7) & ~7;
    if (!sparse_plan(prm.n, 8 * static_cast<int>(sizeof(IT)), prm.s_ring_rows, &plan)) return IEX_ERR_UNSUPPORTED;
    prm.s_a_slots = plan.a_slots;
    prm.s_b_slots = plan.b_slots;
    const size_t ring = static_cast<size_t>(prm.s_ring_rows) * kRingGranules * 8 * (2 + sizeof(IT));
    prm.s_ring_offset = static_cast<uint32_t>(prm.s_a_slots * A_ATOM_BYTES + prm.s_b_slots * prm.n * 128);
    const size_t sparse = prm.s_ring_offset + ring;
    data = sparse > data ? sparse : data;
  }
  data = (data + 15) & ~static_cast<size_t>(15);
  // 8 KB behind everything for the staged epilogue of dense tiles whose output is tokens-major
  // (contiguous along the tile's rows) and 16-byte friendly; otherwise two-byte stores
  prm.epi_offset = 0;
  bool vec_ok = prm.d_tiles > 0 && prm.d_stride_m == 1 && prm.d_ncols == 0 && prm.d_stride_n % 8 == 0 &&
                prm.d_m % 8 == 0 && aligned16(prm.d_out);
  for (int i = 0; i < prm.d_num_copies; ++i) vec_ok = vec_ok && aligned16(prm.d_out_copies[i]);
  if (vec_ok && data + 8192 <= static_cast<size_t>(kDataBudget)) {
    prm.epi_offset = static_cast<uint32_t>(data);
    data += 8192;
  }
  if (stages > kMaxStages || data > static_cast<size_t>(kDataBudget)) return IEX_ERR_UNSUPPORTED;
  prm.bar_offset = static_cast<uint32_t>(data);
  const size_t smem = 1024 + data + kBarBytes;
  auto kern = tc_units_kernel<ND, IT>;
  {
    // high-water mark of the opt-in shared-memory size, per device and per instantiation
    static size_t configured[kMaxDevices] = {};
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (dev < 0 || smem > configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      if (dev >= 0) configured[dev] = smem;
    }
  }
  const int units = prm.d_tiles * prm.d_parts + prm.s_tiles * prm.s_parts;
  const int grid = units < sm_count() * ctas_per_sm ? units : sm_count() * ctas_per_sm;
  int st = launch_overlapped(kern, dim3(grid), dim3((kFirstDecodeWarp + ND) * 32), smem, stream, ta, tbd, tbs, prm);
  const int split_tiles = (prm.s_parts > 1 ? prm.s_tiles : 0) + (prm.d_parts > 1 && prm.d_ncols == 0 ? prm.d_tiles : 0);
  if (st == 0 && split_tiles > 0) {
    const int slices = (prm.n * (BM / 4) + kReduceThreads - 1) / kReduceThreads;
    st = launch_overlapped(tc_reduce_kernel, dim3(split_tiles, slices), dim3(kReduceThreads), 0, stream, prm);
  }
  return st;
}

int tmem_cols_for(int n) {
  int c = 32;
  while (c < n) c <<= 1;
  return c;
}

}  // namespace tc
}  // namespace iex

using namespace iex;
using namespace iex::tc;

extern "C" int iex_last_device_status(int clear) {
  int v = 0;
  // Work on non-blocking streams (torch's pool streams, graph replays) is not ordered before a
  // symbol copy, so wait for the whole device first: a kernel still running could record a
  // failure after the read.
  const cudaError_t sync = cudaDeviceSynchronize();
  if (sync != cudaSuccess) return static_cast<int>(sync);
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return IEX_ERR_DRIVER;
  if (clear && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_status, &z, sizeof(int));
  }
  return v;
}

#ifdef IEX_TC_PROFILE
static long long* g_tc_prof_buffer = nullptr;
extern "C" void iex_tc_set_profile_buffer(long long* device_buffer) { g_tc_prof_buffer = device_buffer; }
#endif

namespace {

// Height of a sparse tile.  A sparse unit's time depends little on how many of its 128 rows
// are in use (each decoder warp works through its own rows at the pace of its dependent
// instructions), so when full tiles would leave SMs without a unit, lower tiles that give
// (nearly) every SM one -- minus the SMs the dense units need, two units apiece -- finish
// sooner.  Split-K launches keep full tiles (the workspace size promises 128-row tiles).
int sparse_tile_rows(int m_sparse, int d_tiles, int sparse_parts) {
  if (m_sparse <= 0 || sparse_parts > 1) return BM;
  const int sms = sm_count();
  const int target = sms - (d_tiles + 1) / 2;  // CTAs left for sparse units in the first wave
  const int full = (m_sparse + BM - 1) / BM;
  if (target <= full) return BM;
  int h = ((m_sparse + target - 1) / target + 7) & ~7;
  h = h < 8 ? 8 : (h > BM ? BM : h);
  return h;
}

int sparse_args_ok(int m, int k, int n, int nnz, const int32_t* row_offsets, const void* cols,
                   const void* values, const void* dense, const void* out, int index_bits) {
  if (m < 0 || k < 0 || n < 0 || nnz < 0) return IEX_ERR_BAD_ARG;
  if (index_bits != 16 && index_bits != 32) return IEX_ERR_BAD_ARG;
  if (!row_offsets || !dense || !out || (nnz > 0 && (!cols || !values))) return IEX_ERR_BAD_ARG;
  if (n % 64 != 0 || n > 256 || n == 0 || k % 8 != 0 || k == 0) return IEX_ERR_UNSUPPORTED;
  if (index_bits == 16 && k > 65280) return IEX_ERR_UNSUPPORTED;  // 0xffff marks padding
  if (!aligned16(cols) || !aligned16(values) || !aligned16(dense) || !aligned16(out))
    return IEX_ERR_UNSUPPORTED;
  return IEX_OK;
}

size_t workspace_bytes(int s_tiles, int s_parts, int d_tiles, int d_parts, int n) {
  if (s_parts <= 1 && d_parts <= 1) return 0;
  return (static_cast<size_t>(s_tiles) * s_parts + static_cast<size_t>(d_tiles) * d_parts) * BM * n * 4;
}

// Clamps the part counts to the number of k-blocks and points the kernel at the workspace.
int bind_workspace(Params& p, int s_parts, int d_parts, void* workspace, size_t bytes) {
  const int k_blocks = (p.k + BK - 1) / BK;  // dense units advance 128 columns per stage
  const int k_slots = (p.k + 63) / 64;       // sparse units 64 columns per slot
  p.s_parts = s_parts < 1 ? 1 : (s_parts > k_slots ? k_slots : s_parts);
  p.d_parts = d_parts < 1 ? 1 : (d_parts > k_blocks ? k_blocks : d_parts);
  if (p.s_tiles == 0) p.s_parts = 1;
  if (p.d_tiles == 0) p.d_parts = 1;
  const size_t need = workspace_bytes(p.s_tiles, p.s_parts, p.d_tiles, p.d_parts, p.n);
  p.partials = nullptr;
  if (need == 0) return IEX_OK;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return IEX_ERR_BAD_ARG;
  if (bytes < need) return IEX_ERR_TOO_LARGE;
  p.partials = static_cast<float*>(workspace);
  return IEX_OK;
}

int linear_impl(int tokens, int in_features, int out_features, const void* input, const void* weight,
                void* out, int parts, void* workspace, size_t bytes, void* stream,
                long long ld_out = 0, void* const* copies = nullptr, int num_copies = 0) {
  if (tokens < 0 || in_features < 0 || out_features < 0) return IEX_ERR_BAD_ARG;
  if (tokens == 0 || out_features == 0) return IEX_OK;
  if (!input || !weight || !out) return IEX_ERR_BAD_ARG;
  if (tokens % 16 != 0 || tokens > 256 || in_features % 8 != 0 || in_features == 0)
    return IEX_ERR_UNSUPPORTED;
  if (!aligned16(input) || !aligned16(weight)) return IEX_ERR_UNSUPPORTED;
  if (parts > 1 && tokens % 32 != 0) return IEX_ERR_UNSUPPORTED;  // partial tiles are 32 columns wide
  CUtensorMap ta, tb;
  int st = make_map(&ta, weight, out_features, in_features, BM);
  if (st) return st;
  st = make_map(&tb, input, tokens, in_features, tokens);
  if (st) return st;
  Params p{};
  p.d_tiles = (out_features + BM - 1) / BM;
  p.d_m = out_features;
  p.d_out = static_cast<__half*>(out);
  p.d_stride_m = 1;
  p.d_stride_n = ld_out > 0 ? ld_out : out_features;
  p.d_num_copies = num_copies;
  for (int i = 0; i < num_copies; ++i) p.d_out_copies[i] = static_cast<__half*>(copies[i]);
  p.d_b_mn = 0;
  p.k = in_features;
  p.n = tokens;
  p.tmem_cols = tmem_cols_for(tokens);
  p.status = status_word();
#ifdef IEX_TC_PROFILE
  p.prof = g_tc_prof_buffer;
#endif
  st = bind_workspace(p, 1, parts, workspace, bytes);
  if (st) return st;
  const int stages = dense_stages(tokens, kMaxStages);
  if (stages < 2) return IEX_ERR_UNSUPPORTED;
  return launch_units<0, uint16_t>(ta, tb, tb, p, stages, 1, static_cast<cudaStream_t>(stream));
}

int fused_impl(int m_sparse, int m_dense, int k, int n, int nnz, const int32_t* row_offsets,
               const void* column_indices, int index_bits, const void* values, const void* weight,
               const void* x, void* out_sparse, void* out_dense, int dense_out_tokens_major,
               int sparse_parts, int dense_parts, void* workspace, size_t bytes, void* stream,
               const float* sparse_bias = nullptr) {
  if (m_dense < 0 || m_sparse < 0) return IEX_ERR_BAD_ARG;
  int st;
  if (m_sparse > 0) {
    st = sparse_args_ok(m_sparse, k, n, nnz, row_offsets, column_indices, values, x, out_sparse,
                        index_bits);
  } else {  // dense branch alone: same limits on k, n and x
    static const int32_t kNoRows[1] = {0};
    st = sparse_args_ok(0, k, n, 0, kNoRows, nullptr, nullptr, x, x, 16);
    index_bits = 16;
  }
  if (st) return st;
  if (m_dense > 0 && (!weight || !out_dense || !aligned16(weight))) return IEX_ERR_BAD_ARG;
  if (m_sparse == 0 && m_dense == 0) return IEX_OK;
  CUtensorMap ta, tb, tbs;
  st = make_map(&tb, x, k, n, BK);   // dense units: [128 k-rows x 64 cols] boxes of X
  if (st) return st;
  st = make_map(&tbs, x, k, n, 64);  // sparse units: [64 k-rows x 64 cols]
  if (st) return st;
  if (m_dense > 0) {
    st = make_map(&ta, weight, m_dense, k, BM);
    if (st) return st;
  } else {
    ta = tb;
  }
  Params p{};
  p.d_tiles = (m_dense + BM - 1) / BM;
  p.d_m = m_dense;
  p.d_out = static_cast<__half*>(out_dense);
  if (dense_out_tokens_major) { p.d_stride_m = 1; p.d_stride_n = m_dense; }
  else { p.d_stride_m = n; p.d_stride_n = 1; }
  p.d_b_mn = 1;
  p.s_tile_rows = sparse_tile_rows(m_sparse, (m_dense + BM - 1) / BM, sparse_parts);
  p.s_tiles = (m_sparse + p.s_tile_rows - 1) / p.s_tile_rows;
  p.s_m = m_sparse;
  p.s_nnz = nnz;
  p.s_out = static_cast<__half*>(out_sparse);
  p.s_row_offsets = row_offsets;
  p.s_cols = column_indices;
  p.s_values = static_cast<const __half*>(values);
  p.s_bias = sparse_bias;
  p.k = k;
  p.n = n;
  p.tmem_cols = tmem_cols_for(n);
  p.status = status_word();
  st = bind_workspace(p, sparse_parts, dense_parts, workspace, bytes);
  if (st) return st;
  const int stages = dense_stages(n, 4);
  if (stages < 2) return IEX_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (index_bits == 16) return launch_units<kDecodeWarps, uint16_t>(ta, tb, tbs, p, stages, 1, s);
  return launch_units<kDecodeWarps, int>(ta, tb, tbs, p, stages, 1, s);
}

}  // namespace

extern "C" size_t iex_tc_workspace_bytes(int m_sparse, int sparse_parts, int m_dense, int dense_parts,
                                         int n) {
  if (m_sparse < 0 || m_dense < 0 || n < 0) return 0;
  return workspace_bytes((m_sparse + BM - 1) / BM, sparse_parts < 1 ? 1 : sparse_parts,
                         (m_dense + BM - 1) / BM, dense_parts < 1 ? 1 : dense_parts, n);
}

extern "C" int iex_linear_f16(int tokens, int in_features, int out_features, const void* input,
                              const void* weight, void* out, void* stream) {
  return linear_impl(tokens, in_features, out_features, input, weight, out, 1, nullptr, 0, stream);
}

extern "C" int iex_linear_f16_splitk(int tokens, int in_features, int out_features, const void* input,
                                     const void* weight, void* out, int parts, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  return linear_impl(tokens, in_features, out_features, input, weight, out, parts, workspace,
                     workspace_bytes, stream);
}

// The two products of the dense branch's backward pass on the same tensor-core kernel.
//   dgrad:  dinput [tokens, in] = grad [tokens, out] * weight [out, in]
//           D[f = in, t] = sum_c W[c, f] * grad[t, c]: A = weight read as [K = out, M = in]
//           (MN-major), B = grad (K-major, like the forward's input).  tokens <= 256.
//   wgrad:  dweight [out, in] = grad^T [out, tokens] * input [tokens, in]
//           D[f = out, j = in] = sum_t grad[t, f] * input[t, j]: A = grad read as [K = tokens,
//           M = out] (MN-major), B = input [K = tokens, N = in] (MN-major), units over blocks of
//           256 columns of `in`.  Any number of tokens (K).
extern "C" int iex_linear_f16_dgrad(int tokens, int in_features, int out_features, const void* grad,
                                    const void* weight, void* dinput, void* stream) {
  if (tokens < 0 || in_features < 0 || out_features < 0) return IEX_ERR_BAD_ARG;
  if (tokens == 0 || in_features == 0) return IEX_OK;
  if (!grad || !weight || !dinput) return IEX_ERR_BAD_ARG;
  if (tokens % 16 != 0 || tokens > 256 || out_features % 8 != 0 || out_features == 0 || in_features % 8 != 0)
    return IEX_ERR_UNSUPPORTED;
  if (!aligned16(grad) || !aligned16(weight)) return IEX_ERR_UNSUPPORTED;
  CUtensorMap ta, tb;
  int st = make_map(&ta, weight, out_features, in_features, BK);  // [K rows, M cols], boxes of 128 k-rows
  if (st) return st;
  st = make_map(&tb, grad, tokens, out_features, tokens);
  if (st) return st;
  Params p{};
  p.d_tiles = (in_features + BM - 1) / BM;
  p.d_m = in_features;
  p.d_out = static_cast<__half*>(dinput);
  p.d_stride_m = 1;
  p.d_stride_n = in_features;
  p.d_a_mn = 1;
  p.k = out_features;
  p.n = tokens;
  p.tmem_cols = tmem_cols_for(tokens);
  p.status = status_word();
  st = bind_workspace(p, 1, 1, nullptr, 0);
  if (st) return st;
  const int stages = dense_stages(tokens, kMaxStages);
  if (stages < 2) return IEX_ERR_UNSUPPORTED;
  return launch_units<0, uint16_t>(ta, tb, tb, p, stages, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int iex_linear_f16_wgrad(int tokens, int in_features, int out_features, const void* grad,
                                    const void* input, void* dweight, void* stream) {
  if (tokens < 0 || in_features < 0 || out_features < 0) return IEX_ERR_BAD_ARG;
  if (out_features == 0 || in_features == 0) return IEX_OK;
  if (!grad || !input || !dweight) return IEX_ERR_BAD_ARG;
  if (tokens % 8 != 0 || tokens == 0 || out_features % 8 != 0 || in_features % 8 != 0) return IEX_ERR_UNSUPPORTED;
  if (!aligned16(grad) || !aligned16(input) || !aligned16(dweight)) return IEX_ERR_UNSUPPORTED;
  const int nblk = in_features >= 256 ? 256 : ((in_features + 63) / 64) * 64;  // columns per unit
  CUtensorMap ta, tb;
  int st = make_map(&ta, grad, tokens, out_features, BK);  // [K = tokens rows, M = out cols]
  if (st) return st;
  st = make_map(&tb, input, tokens, in_features, BK);  // [K rows, N cols], boxes of 128 k-rows
  if (st) return st;
  Params p{};
  p.d_tiles = (out_features + BM - 1) / BM;
  p.d_m = out_features;
  p.d_out = static_cast<__half*>(dweight);
  p.d_stride_m = in_features;
  p.d_stride_n = 1;
  p.d_a_mn = 1;
  p.d_b_mn = 1;
  p.d_nblocks = (in_features + nblk - 1) / nblk;
  p.d_ncols = in_features;
  p.k = tokens;
  p.n = nblk;
  p.tmem_cols = tmem_cols_for(nblk);
  p.status = status_word();
  p.s_parts = 1;
  p.d_parts = p.d_nblocks;  // the unit list counts column blocks where it would count K parts
  p.partials = nullptr;
  const int stages = dense_stages(nblk, kMaxStages);
  if (stages < 2) return IEX_ERR_UNSUPPORTED;
  return launch_units<0, uint16_t>(ta, tb, tb, p, stages, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int iex_spmm_f16_tc(int m, int k, int n, int nnz, const int32_t* row_offsets,
                               const void* column_indices, int index_bits, const void* values,
                               const void* dense, void* out, void* stream) {
  if (m == 0) return IEX_OK;
  return fused_impl(m, 0, k, n, nnz, row_offsets, column_indices, index_bits, values, nullptr, dense, out,
                    nullptr, 1, 1, 1, nullptr, 0, stream);
}

extern "C" int iex_spmm_f16_tc_bias_relu(int m, int k, int n, int nnz, const int32_t* row_offsets,
                                         const void* column_indices, int index_bits, const void* values,
                                         const void* dense, const float* bias, void* out, void* stream) {
  if (m == 0) return IEX_OK;
  return fused_impl(m, 0, k, n, nnz, row_offsets, column_indices, index_bits, values, nullptr, dense, out,
                    nullptr, 1, 1, 1, nullptr, 0, stream, bias);
}

extern "C" int iex_spmm_f16_tc_splitk(int m, int k, int n, int nnz, const int32_t* row_offsets,
                                      const void* column_indices, int index_bits, const void* values,
                                      const void* dense, void* out, int parts, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  if (m == 0) return IEX_OK;
  return fused_impl(m, 0, k, n, nnz, row_offsets, column_indices, index_bits, values, nullptr, dense, out,
                    nullptr, 1, parts, 1, workspace, workspace_bytes, stream);
}

extern "C" int iex_fused_spmm_linear_f16(int m_sparse, int m_dense, int k, int n, int nnz,
                                         const int32_t* row_offsets, const void* column_indices,
                                         int index_bits, const void* values, const void* weight,
                                         const void* x, void* out_sparse, void* out_dense,
                                         int dense_out_tokens_major, void* stream) {
  return fused_impl(m_sparse, m_dense, k, n, nnz, row_offsets, column_indices, index_bits, values, weight, x,
                    out_sparse, out_dense, dense_out_tokens_major, 1, 1, nullptr, 0, stream);
}

extern "C" int iex_fused_spmm_linear_f16_splitk(int m_sparse, int m_dense, int k, int n, int nnz,
                                                const int32_t* row_offsets, const void* column_indices,
                                                int index_bits, const void* values, const void* weight,
                                                const void* x, void* out_sparse, void* out_dense,
                                                int dense_out_tokens_major, int sparse_parts,
                                                int dense_parts, void* workspace, size_t workspace_bytes,
                                                void* stream) {
  return fused_impl(m_sparse, m_dense, k, n, nnz, row_offsets, column_indices, index_bits, values, weight, x,
                    out_sparse, out_dense, dense_out_tokens_major, sparse_parts, dense_parts, workspace,
                    workspace_bytes, stream);
}

// ---------------------------------------------------------------------------------------
// Split-K linear without any allocation by anybody
//
// Some hosts of this library may not create device memory once they are running: a serving
// process or plugin host that sizes its memory pool at start-up and forbids later
// cudaMalloc calls (they synchronise the whole device and can fail once memory is
// fragmented), or a caller that has no allocator of its own to take a workspace from.
// For them the partial tiles of iex_linear_f16_splitk live in the fixed array below, which
// every GPU that loads this library carries until the process exits.
// ---------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticWorkspaceBytes = size_t(8) << 20;  // 8 MiB per device

}  // namespace

// In host code this name is only a handle for cudaGetSymbolAddress, not a device pointer.
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];

namespace {

std::mutex g_static_mutex;
void* g_static_address[kMaxDevices] = {};

// Device address of g_static_workspace on the CURRENT device, looked up once per device.
int static_workspace_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return IEX_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_address[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_workspace);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (p == nullptr) return IEX_ERR_DRIVER;
    g_static_address[dev] = p;
  }
  *out = g_static_address[dev];
  return IEX_OK;
}

}  // namespace

extern "C" size_t iex_static_workspace_capacity(void) { return kStaticWorkspaceBytes; }

extern "C" int iex_linear_f16_splitk_static(int tokens, int in_features, int out_features,
                                            const void* input, const void* weight, void* out, int parts,
                                            void* stream) {
  if (tokens < 0 || in_features < 0 || out_features < 0) return IEX_ERR_BAD_ARG;
  // Size check first, with the part count the kernel will really use (never more than k-blocks).
  const int k_blocks = (in_features + BK - 1) / BK;
  int used_parts = parts < 1 ? 1 : parts;
  if (used_parts > k_blocks) used_parts = k_blocks > 0 ? k_blocks : 1;
  const size_t need = workspace_bytes(0, 1, (out_features + BM - 1) / BM, used_parts, tokens);
  if (need > kStaticWorkspaceBytes) return IEX_ERR_TOO_LARGE;
  void* ws = nullptr;
  if (need > 0) {
    const int st = static_workspace_address(&ws);
    if (st != IEX_OK) return st;
  }
  return linear_impl(tokens, in_features, out_features, input, weight, out, used_parts, ws,
                     need > 0 ? kStaticWorkspaceBytes : 0, stream);
}

// ---------------------------------------------------------------------------------------
// Column-sharded linear with the all-gather done by the kernel's own stores
// ---------------------------------------------------------------------------------------
extern "C" int iex_linear_f16_splitk_gather(int tokens, int in_features, int out_features,
                                            const void* input, const void* weight, void* const* outs,
                                            int world, int rank, long long ld_out, long long col_offset,
                                            int parts, void* workspace, size_t workspace_bytes,
                                            void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || !outs) return IEX_ERR_BAD_ARG;
  if (ld_out < out_features || col_offset < 0 || col_offset + out_features > ld_out) return IEX_ERR_BAD_ARG;
  if (col_offset % 8 != 0 || ld_out % 8 != 0) return IEX_ERR_UNSUPPORTED;  // 16-byte stores
  void* copies[kMaxPeers];
  int n = 0;
  for (int r = 0; r < world; ++r) {
    if (!outs[r] || !aligned16(outs[r])) return IEX_ERR_BAD_ARG;
    if (r != rank) copies[n++] = static_cast<__half*>(outs[r]) + col_offset;
  }
  return linear_impl(tokens, in_features, out_features, input, weight,
                     static_cast<__half*>(outs[rank]) + col_offset, parts, workspace, workspace_bytes,
                     stream, ld_out, copies, n);
}

extern "C" int iex_peer_barrier_bounded(void* const* signals, int world, int rank, unsigned max_polls,
                                        void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || !signals) return IEX_ERR_BAD_ARG;
  PeerSignals ps{};
  for (int r = 0; r < world; ++r) {
    if (!signals[r] || (reinterpret_cast<uintptr_t>(signals[r]) & 3u)) return IEX_ERR_BAD_ARG;
    ps.sig[r] = static_cast<uint32_t*>(signals[r]);
  }
  ps.world = world;
  ps.rank = rank;
  ps.status = status_word();
  ps.max_polls = max_polls == 0 ? kPeerSpinLimit : (max_polls > kPeerSpinLimit ? kPeerSpinLimit : max_polls);
  return launch_overlapped(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), ps);
}

extern "C" int iex_peer_barrier(void* const* signals, int world, int rank, void* stream) {
  return iex_peer_barrier_bounded(signals, world, rank, 0, stream);
}

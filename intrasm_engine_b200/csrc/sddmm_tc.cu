// Sampled dense-dense matmul on tensor cores (tcgen05 / TMEM, sm_100a), fp32 in and out:
//   out[p] = dot(lhs[row(p), :], rhs[col[p], :])        for every stored position p.
//
// A CUDA-core SDDMM gathers one rhs row (4k bytes) through L1 / L2 per stored position; at a
// few per cent density that gather traffic is twenty times the matrices themselves and the
// L2 -> SM fabric bounds the kernel.  Here the DENSE product of a 128-row band of lhs with a
// 128-row tile of rhs is formed on the tensor cores -- every operand byte is loaded once per
// tile -- and only the stored positions of the 128 x 128 result are written out.
//
// fp32 accuracy on a TF32 pipe: every operand value x is split into hi = tf32(x) and
// lo = x - hi (exact), and the tile is accumulated as  lo*hi' + hi*lo' + hi*hi'  in an fp32
// TMEM accumulator: the dropped lo*lo' term and the rounding of lo are below 2^-20 of
// |x||x'| per term.
//
// Which positions a tile holds comes from a PLAN of the sparsity pattern, built once per
// pattern (the same kind of pattern-only argument as the reference's row_indices): the
// stored positions regrouped by 128 x 128 tile -- tile_ptr[tile] .. tile_ptr[tile + 1] index
// two arrays, `entry` (row and column inside the tile, 7 bits each) and `dest` (the position
// in storage order the value belongs at).  With it the sampling is one flat, branch-free
// pass per tile over a coalesced list, instead of every row walking its own column indices.
//
// One persistent CTA per SM walks "units": a band and a run of its tiles.
//   warps 0-6   converters: read tile after tile of rhs from global memory (coalesced 128-bit
//               loads, one tile ahead in registers), split into hi / lo and store both planes
//               into shared memory in the 128-byte-swizzled K-major layout tcgen05.mma reads
//               (two stages).
//   warp 7      one thread issues the 3 * k / 8 tcgen05.mma.kind::tf32 (M = N = 128, K = 8, A in
//               TMEM) of a tile into one of three TMEM accumulators and releases the operand
//               stage and the accumulator with tcgen05.commit.
//   warps 8-15  epilogue.  At the start of a unit they put the unit's lhs band, split like rhs,
//               into TENSOR memory (tcgen05.st, lane = row): the A operand of every MMA of the
//               unit comes from there, which halves the shared-memory bytes an MMA reads -- a
//               K = 8 TF32 instruction is otherwise bound by operand bandwidth.  Per tile: the eight warps copy the accumulator (tcgen05.ld,
//               two warps per TMEM lane quarter, 64 columns each) into a padded shared-memory
//               tile, meet, and then every thread takes entries of the tile's list -- already
//               in registers, loaded while the tensor core was busy -- reads the value at
//               (row, column) from shared memory and stores it at out[dest]; neighbouring
//               entries of a row go to neighbouring addresses.
// Every mbarrier wait is bounded.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_prof.cuh"
#include "tile_plan.cuh"

namespace iex {
namespace sddmm_tc {

using namespace iex::tc;

constexpr int TM = 128;          // rows of lhs per band (UMMA M)
constexpr int TN = 128;          // rows of rhs (= columns of the mask) per tile (UMMA N)
constexpr int kConvWarps = 7;      // 16 warps in all: 128 registers per thread
constexpr int kMmaWarp = 7;
constexpr int kFirstEpiWarp = 8;   // warps 8..15: (warp & 3) = 0, 1, 2, 3, 0, 1, 2, 3
constexpr int kEpiWarps = 8;
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
constexpr int kBStages = 2;              // rhs tiles in flight between converters and tensor core
constexpr int kAccs = 3;                 // TMEM accumulators of TN columns
constexpr int kParkStride = TN * 4 + 16; // bytes per row of the shared-memory copy of a tile
constexpr int kEntriesInRegs = 4;        // list entries per epilogue thread fetched ahead of a tile
constexpr int kAtomBytesB = TN * 128;    // one 32-float K atom of a 128-row rhs plane
constexpr int kBarBytes = 256;
// tensor memory (512 columns): accumulators at 0, 128, 256; the lhs band's hi plane at 384,
// its lo plane at 448 (k <= 64 columns each)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemAHi = 384, kTmemALo = 448;

constexpr int kMaxProblems = 32;  // products of one launch (same shape, own operands and plan)

struct Problem {
  const int* tile_ptr;         // [bands * tiles_per_band + 1]
  const uint16_t* entry;       // [nnz] (row in tile << 7) | column in tile
  const int* dest;             // [nnz] position in storage order
  const float* lhs;
  const float* rhs;
  float* out;
};

struct Params {
  int m, n, k;
  int count;                   // problems in this launch
  Problem prob[kMaxProblems];
  int accumulate;
  int tiles_per_band;
  // units of ONE problem: bands [0, bands_hi) are cut into base_splits + 1 runs of tiles, the
  // others into base_splits runs; the launch's units are those of problem 0, then problem 1, ...
  // and CTA c takes units c, c + grid, ...  A CTA that takes several units loads the next
  // unit's lhs band while the tensor core works on the current one.
  int units, base_splits, bands_hi;
  int* status;
  IEX_PROF_FIELD
};

__device__ __forceinline__ void unit_of(int u_all, const Params& p, int& pi, int& band, int& t0, int& t1) {
  pi = u_all / p.units;
  const int u = u_all - pi * p.units;
  const int hi_units = p.bands_hi * (p.base_splits + 1);
  int s, S;
  if (u < hi_units) {
    S = p.base_splits + 1;
    band = u / S;
    s = u - band * S;
  } else {
    S = p.base_splits;
    const int v = u - hi_units;
    band = p.bands_hi + v / S;
    s = v - (v / S) * S;
  }
  t0 = static_cast<int>(static_cast<long long>(s) * p.tiles_per_band / S);
  t1 = static_cast<int>(static_cast<long long>(s + 1) * p.tiles_per_band / S);
}

// D[tmem] (+)= A[tmem] * B[smem]: the lhs band stays in tensor memory for a whole unit, so an
// instruction reads only its 128 x 8 slice of the rhs tile from shared memory.
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// TN rows x k floats of a row-major [limit, k] matrix starting at row0, up to NV float4 per
// thread of the converter threads (consecutive threads read consecutive 16-byte pieces: the
// tile is one contiguous run of memory).  Rows past `limit` read as zero.
template <int NV>
__device__ __forceinline__ void load_rows(float4 (&v)[NV], const float* __restrict__ src, int row0,
                                          int limit, int k, int kv_shift, int ct) {
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = ct + j * (kConvWarps * 32);
    const int row = i >> kv_shift, c4 = i & ((1 << kv_shift) - 1);
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < TN && row0 + row < limit)
      v[j] = __ldg(reinterpret_cast<const float4*>(src + static_cast<size_t>(row0 + row) * k) + c4);
  }
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Where load_rows' j-th value of this thread goes inside an operand plane: [k / 32 atoms][rows]
// [128 bytes] (ATOM = rows * 128 bytes per atom) with the 16-byte pieces of a row XOR-swizzled
// by (row & 7); 0xffffffff for a value past the tile.  The same for every tile, so computed once.
template <int NV, int ATOM>
__device__ __forceinline__ void plane_offsets(uint32_t (&off)[NV], int kv_shift, int ct) {
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = ct + j * (kConvWarps * 32);
    const int row = i >> kv_shift, c4 = i & ((1 << kv_shift) - 1);
    off[j] = row < TN ? static_cast<uint32_t>((c4 >> 3) * ATOM + row * 128 + (((c4 & 7) ^ (row & 7)) << 4)) : 0xffffffffu;
  }
}

// Splits what load_rows fetched into the TF32 head and the remainder and stores both planes.
template <int NV>
__device__ __forceinline__ void store_split(const float4 (&v)[NV], const uint32_t (&off)[NV], uint32_t hi_plane,
                                            uint32_t lo_plane) {
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (off[j] == 0xffffffffu) continue;
    const float hx = tf32_round(v[j].x), hy = tf32_round(v[j].y), hz = tf32_round(v[j].z),
                hw = tf32_round(v[j].w);
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(hi_plane + off[j]), "f"(hx), "f"(hy), "f"(hz),
                 "f"(hw)
                 : "memory");
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(lo_plane + off[j]), "f"(v[j].x - hx),
                 "f"(v[j].y - hy), "f"(v[j].z - hz), "f"(v[j].w - hw)
                 : "memory");
  }
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}


// KA = k / 32 (K atoms per operand plane): 1 or 2.
template <int KA>
__global__ void __launch_bounds__(kThreads, 1) sddmm_tc_kernel(const Params prm) {
  extern __shared__ uint8_t smem_raw[];
  IEX_PROF_STAMP(threadIdx.x == 0, 42)
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kPlaneB = KA * kAtomBytesB;  // one hi or lo plane of a rhs tile
  auto b_hi = [&](int s) { return smem_base + static_cast<uint32_t>(s) * 2u * kPlaneB; };
  const uint32_t park_base = smem_base + kBStages * 2u * kPlaneB;  // [128 rows][128 floats + pad]
  const uint32_t bar_base = park_base + TM * kParkStride;
  const uint32_t a_full = bar_base, a_empty = bar_base + 8, epi_bar = bar_base + 16;
  auto b_full = [&](int s) { return bar_base + 24u + 8u * s; };
  auto b_empty = [&](int s) { return bar_base + 40u + 8u * s; };
  auto acc_full = [&](int s) { return bar_base + 56u + 8u * s; };
  auto acc_empty = [&](int s) { return bar_base + 80u + 8u * s; };
  const uint32_t tmem_slot = bar_base + 104u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_off = bar_base - smem_base;
  volatile uint32_t* tmem_ptr_generic = reinterpret_cast<volatile uint32_t*>(smem_aligned + bar_off + 104u);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_aligned + bar_off + 108u);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(a_full, kEpiWarps);
    mbar_init(a_empty, 1);
    mbar_init(epi_bar, kEpiWarps);
    for (int s = 0; s < kBStages; ++s) {
      mbar_init(b_full(s), kConvWarps);
      mbar_init(b_empty(s), 1);
    }
    for (int s = 0; s < kAccs; ++s) {
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), kEpiWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_generic;
  // Everything above touched only this CTA's own shared and tensor memory and may overlap the
  // end of the kernel before this one in the stream; global memory comes next.
  grid_dependency_wait();
  grid_launch_dependents();
  IEX_PROF_STAMP(threadIdx.x == 0, 43)

  const int k = prm.k;
  constexpr int kv_shift = KA == 1 ? 3 : 4;  // log2(float4 per row)
  // float4 per converter thread for a 128-row rhs tile (rounded up)
  constexpr int NVB = (TN * KA * 8 + kConvWarps * 32 - 1) / (kConvWarps * 32);

  if (warp < kConvWarps) {
    // ------------------------------------------------------------------ converters
    const int ct = threadIdx.x;
    uint32_t it = 0, ui = 0;
    bool ok = true;
    uint32_t off[NVB];
    plane_offsets<NVB, kAtomBytesB>(off, kv_shift, ct);
    IEX_PROF_BEGIN
    const int total_units = prm.units * prm.count;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
      int pi, band, t0, t1;
      unit_of(u, prm, pi, band, t0, t1);
      const float* __restrict__ rhs = prm.prob[pi].rhs;
      float4 v[NVB];
      load_rows<NVB>(v, rhs, t0 * TN, prm.n, k, kv_shift, ct);  // first tile: in flight meanwhile
      IEX_LAP(0)  // unit start: first rhs loads issued
      for (int t = t0; t < t1; ++t, ++it) {
        const int s = it % kBStages;
        if (!mbar_wait(b_empty(s), ((it / kBStages) & 1u) ^ 1u, abort_flag, prm.status, 32)) { ok = false; break; }
        IEX_LAP(1)  // waiting for a free stage
        store_split<NVB>(v, off, b_hi(s), b_hi(s) + kPlaneB);
        IEX_LAP(2)  // split + store
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(b_full(s));
        if (t + 1 < t1) load_rows<NVB>(v, rhs, (t + 1) * TN, prm.n, k, kv_shift, ct);
        IEX_LAP(3)  // fence, arrive, next loads issued
      }
    }
    IEX_PROF_DUMP(threadIdx.x == 0, 0)
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // D fp32, A and B tf32, both K-major, N = 128, M = 128
      constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(TN >> 3) << 17) |
                                 (static_cast<uint32_t>(TM >> 4) << 24);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      IEX_PROF_BEGIN
      const int total_units = prm.units * prm.count;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
        int pi, band, t0, t1;
        unit_of(u, prm, pi, band, t0, t1);
        if (!mbar_wait(a_full, ui & 1u, abort_flag, prm.status, 32)) { ok = false; break; }
        IEX_LAP(0)  // waiting for the lhs band
        for (int t = t0; t < t1; ++t, ++it) {
          const int s = it % kBStages, a = it % kAccs;
          if (!mbar_wait(b_full(s), (it / kBStages) & 1u, abort_flag, prm.status, 32)) { ok = false; break; }
          IEX_LAP(1)  // waiting for a rhs tile
          if (!mbar_wait(acc_empty(a), ((it / kAccs) & 1u) ^ 1u, abort_flag, prm.status, 32)) { ok = false; break; }
          IEX_LAP(2)  // waiting for a free accumulator
          tcgen05_fence_after();
          const uint32_t d = tmem_base + static_cast<uint32_t>(a) * TN;
          // small terms first: lo * hi', hi * lo', then hi * hi'
          const uint32_t a_col[3] = {kTmemALo, kTmemAHi, kTmemAHi};
          const uint32_t b_plane[3] = {b_hi(s), b_hi(s) + kPlaneB, b_hi(s)};
#pragma unroll
          for (int pr = 0; pr < 3; ++pr) {
#pragma unroll
            for (int ka = 0; ka < KA; ++ka) {
              const uint64_t bdesc0 = smem_desc(b_plane[pr] + ka * kAtomBytesB, 16, 1024);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)  // 8 tf32 per instruction: 8 TMEM columns of A, 32 bytes of B
                umma_tf32_ts(d, tmem_base + a_col[pr] + ka * 32 + ks * 8, desc_advance(bdesc0, ks * 32), idesc,
                             (pr | ka | ks) != 0 ? 1u : 0u);
            }
          }
          umma_commit(b_empty(s));
          umma_commit(acc_full(a));
          IEX_LAP(3)  // issuing
        }
        if (ok) umma_commit(a_empty);
      }
      IEX_PROF_DUMP(true, 8)
    }
  } else {
    // ------------------------------------------------------------------ sampling epilogue
    const int ew = warp - kFirstEpiWarp;          // 0..7
    const int et = ew * 32 + lane;                // 0..255
    const int q = warp & 3;                       // TMEM lane quarter
    const int half = ew >> 2;                     // which 64 columns of the tile this warp copies
    const uint32_t park_row = park_base + static_cast<uint32_t>(q * 32 + lane) * kParkStride + half * 256;
    const int T = prm.tiles_per_band;
    const int total_units = prm.units * prm.count;
    uint32_t it = 0, sync_it = 0;
    bool ok = true;
    IEX_PROF_BEGIN
    // all eight warps meet (bounded wait); orders the shared-memory accesses around it
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool done = mbar_wait(epi_bar, sync_it & 1u, abort_flag, prm.status, 20);
      ++sync_it;
      __syncwarp();
      return done;
    };
    uint32_t ui = 0;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
      int pi, band, t0, t1;
      unit_of(u, prm, pi, band, t0, t1);
      const int* __restrict__ tile_ptr = prm.prob[pi].tile_ptr;
      const uint16_t* __restrict__ entry = prm.prob[pi].entry;
      const int* __restrict__ dest = prm.prob[pi].dest;
      float* __restrict__ out = prm.prob[pi].out;
      int e_beg = __ldg(tile_ptr + band * T + t0), e_end = __ldg(tile_ptr + band * T + t0 + 1);
      // The unit's lhs band into tensor memory: thread = row (TMEM lane), this warp's half of
      // k, all loads of the row in flight together.  The epilogue warps do it because they sit
      // in the right lane quarters and have nothing else to do until the first tile is ready.
      {
        const int row = band * TM + q * 32 + lane;
        constexpr int kHalf = KA * 16;  // k-values per warp: 32 for k = 64, 16 for k = 32
        const float4* src =
            reinterpret_cast<const float4*>(prm.prob[pi].lhs + static_cast<size_t>(row) * k + half * kHalf);
        float4 x[kHalf / 4];
#pragma unroll
        for (int j = 0; j < kHalf / 4; ++j) {
          x[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (row < prm.m) x[j] = __ldg(src + j);
        }
        // the tensor core may still be reading the previous unit's band
        if (ui > 0 && !mbar_wait(a_empty, (ui - 1u) & 1u, abort_flag, prm.status, 64)) { ok = false; break; }
        __syncwarp();
        tcgen05_fence_after();
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * kHalf;
#pragma unroll
        for (int h16 = 0; h16 < kHalf / 16; ++h16) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float xs[4] = {x[h16 * 4 + j].x, x[h16 * 4 + j].y, x[h16 * 4 + j].z, x[h16 * 4 + j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float h = tf32_round(xs[e]);
              hi[4 * j + e] = __float_as_uint(h);
              lo[4 * j + e] = __float_as_uint(xs[e] - h);
            }
          }
          tmem_st16(lane_base + kTmemAHi + h16 * 16, hi);
          tmem_st16(lane_base + kTmemALo + h16 * 16, lo);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full);
      }
      IEX_LAP(0)  // lhs band into TMEM
      // this thread's entries of the first tile (later tiles: fetched one tile ahead)
      uint32_t en[kEntriesInRegs];
      int de[kEntriesInRegs];
#pragma unroll
      for (int i = 0; i < kEntriesInRegs; ++i) {
        const int e = e_beg + et + i * (kEpiWarps * 32);
        en[i] = e < e_end ? __ldg(entry + e) : 0u;
        de[i] = e < e_end ? __ldg(dest + e) : -1;
      }
      for (int t = t0; t < t1; ++t, ++it) {
        const int next_end = t + 1 < t1 ? __ldg(tile_ptr + band * T + t + 2) : e_end;
        const int a = it % kAccs;
        if (!mbar_wait(acc_full(a), (it / kAccs) & 1u, abort_flag, prm.status, 64)) { ok = false; break; }
        __syncwarp();
        IEX_LAP(1)  // waiting for an accumulator
        tcgen05_fence_after();
        // accumulator -> shared memory: row = TMEM lane, this warp's 64 columns
        const uint32_t tacc = tmem_base + static_cast<uint32_t>(a) * TN + half * 64 + (static_cast<uint32_t>(q * 32) << 16);
        {
          uint32_t r0[32], r1[32];
          tmem_ld32(tacc, r0);
          tmem_ld32(tacc + 32, r1);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(park_row + v4 * 16), "r"(r0[4 * v4]),
                         "r"(r0[4 * v4 + 1]), "r"(r0[4 * v4 + 2]), "r"(r0[4 * v4 + 3])
                         : "memory");
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(park_row + 128 + v4 * 16), "r"(r1[4 * v4]),
                         "r"(r1[4 * v4 + 1]), "r"(r1[4 * v4 + 2]), "r"(r1[4 * v4 + 3])
                         : "memory");
        }
        // accumulator read completely: the tensor core may overwrite it
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(a));
        IEX_LAP(2)  // copying the tile
        if (!epi_sync()) { ok = false; break; }
        IEX_LAP(3)  // meeting: tile complete in shared memory
        // the next tile's entries travel while this tile is sampled
        uint32_t en2[kEntriesInRegs];
        int de2[kEntriesInRegs];
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) {
          const int e = e_end + et + i * (kEpiWarps * 32);
          en2[i] = e < next_end ? __ldg(entry + e) : 0u;
          de2[i] = e < next_end ? __ldg(dest + e) : -1;
        }
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) {
          if (de[i] >= 0) {
            const uint32_t rc = en[i];  // (row << 7) | column
            float val = __uint_as_float(lds_u32(park_base + (rc >> 7) * kParkStride + (rc & 127u) * 4u));
            if (prm.accumulate) val += out[de[i]];
            out[de[i]] = val;
          }
        }
        for (int e = e_beg + et + kEntriesInRegs * (kEpiWarps * 32); e < e_end; e += kEpiWarps * 32) {
          const uint32_t rc = __ldg(entry + e);
          const int d = __ldg(dest + e);
          float val = __uint_as_float(lds_u32(park_base + (rc >> 7) * kParkStride + (rc & 127u) * 4u));
          if (prm.accumulate) val += out[d];
          out[d] = val;
        }
        IEX_LAP(4)  // sampling
        if (!epi_sync()) { ok = false; break; }  // everybody is done with the shared-memory tile
        IEX_LAP(5)  // meeting: tile released
        e_beg = e_end;
        e_end = next_end;
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) {
          en[i] = en2[i];
          de[i] = de2[i];
        }
      }
    }
    IEX_PROF_DUMP(lane == 0 && (ew == 0 || ew == 4), 16 + ew * 2)
  }

  // ---------------------------------------------------------------------- teardown
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
    IEX_PROF_STAMP(lane == 0, 44)
  }
}

template <int KA>
constexpr size_t smem_bytes() {
  return 1024 + kBStages * 2 * static_cast<size_t>(KA) * kAtomBytesB + TM * kParkStride + kBarBytes;
}

template <int KA>
int launch(Params prm, cudaStream_t stream) {
  constexpr size_t smem = smem_bytes<KA>();
  auto kern = sddmm_tc_kernel<KA>;
  {
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  const int sms = sm_count();
  const int total = prm.units * prm.count;
  const int grid = total < sms ? total : sms;
  return launch_overlapped(kern, dim3(grid), dim3(kThreads), smem, stream, prm);
}

}  // namespace sddmm_tc
}  // namespace iex

extern "C" int iex_sddmm_f32_tc_supported(int m, int k, int n, int batch) {
  return (m > 0 && n > 0 && batch == 1 && (k == 32 || k == 64)) ? 1 : 0;
}

extern "C" int iex_sddmm_f32_prefers_tc(int m, int k, int n, int nnz, int batch) {
  if (!iex_sddmm_f32_tc_supported(m, k, n, batch)) return 0;
  // The tensor-core kernel's time follows the number of 128 x 128 tiles, the CUDA-core
  // kernel's the number of stored positions: dense tiles pay from a few per cent density on,
  // once there are enough tiles to occupy the SMs.
  const long long tiles = static_cast<long long>((m + 127) / 128) * ((n + 127) / 128);
  return tiles >= 64 && static_cast<long long>(nnz) * 50 >= static_cast<long long>(m) * n ? 1 : 0;
}

#ifdef IEX_TC_PROFILE
static long long* g_prof_buffer = nullptr;
extern "C" void iex_sddmm_f32_tc_set_profile_buffer(long long* device_buffer) { g_prof_buffer = device_buffer; }
#endif

namespace {

// One launch over `count` products of the same shape (m, k, n), each with its own operands,
// result, number of stored positions and plan.
int sddmm_tc_launch(int m, int k, int n, int count, const int* nnz, const void* const* plans,
                    const float* const* lhs, const float* const* rhs, float* const* outs, int accumulate,
                    void* stream) {
  using namespace iex;
  using namespace iex::sddmm_tc;
  if (m < 0 || k < 0 || n < 0 || count < 0 || count > kMaxProblems) return IEX_ERR_BAD_ARG;
  if (m == 0 || count == 0) return IEX_OK;
  if (!nnz || !plans || !lhs || !rhs || !outs) return IEX_ERR_BAD_ARG;
  if (!iex_sddmm_f32_tc_supported(m, k, n, 1)) return IEX_ERR_UNSUPPORTED;
  Params p{};
  p.m = m;
  p.n = n;
  p.k = k;
  int used = 0;
  tile_plan::Layout L{};
  for (int i = 0; i < count; ++i) {
    if (nnz[i] < 0) return IEX_ERR_BAD_ARG;
    if (nnz[i] == 0) continue;  // nothing stored: nothing to write
    if (!plans[i] || !lhs[i] || !rhs[i] || !outs[i] || !aligned16(plans[i])) return IEX_ERR_BAD_ARG;
    if (!aligned16(lhs[i]) || !aligned16(rhs[i])) return IEX_ERR_UNSUPPORTED;
    L = tile_plan::layout(m, n, nnz[i], TN);
    const uint8_t* base = static_cast<const uint8_t*>(plans[i]);
    Problem& q = p.prob[used++];
    q.tile_ptr = reinterpret_cast<const int*>(base + L.tile_ptr);
    q.entry = reinterpret_cast<const uint16_t*>(base + L.entry);
    q.dest = reinterpret_cast<const int*>(base + L.dest);
    q.lhs = lhs[i];
    q.rhs = rhs[i];
    q.out = outs[i];
  }
  if (used == 0) return IEX_OK;
  p.count = used;
  p.accumulate = accumulate;
  p.status = tc::status_word();
#ifdef IEX_TC_PROFILE
  p.prof = g_prof_buffer;
#endif
  const int bands = (m + TM - 1) / TM;
  const int T = L.tiles_per_band;
  p.tiles_per_band = T;
  // runs per band: enough to give every SM a unit
  const int sms = tc::sm_count();
  int base_splits = bands >= sms ? 1 : sms / bands;
  int rem = bands >= sms ? 0 : sms % bands;
  if (base_splits >= T) { base_splits = T; rem = 0; }
  p.base_splits = base_splits;
  p.bands_hi = rem;
  p.units = p.bands_hi * (p.base_splits + 1) + (bands - p.bands_hi) * p.base_splits;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return k == 32 ? launch<1>(p, s) : launch<2>(p, s);
}

}  // namespace

extern "C" int iex_sddmm_f32_tc(int m, int k, int n, int nnz, const void* plan, const float* lhs,
                                const float* rhs, float* out, int accumulate, void* stream) {
  if (nnz < 0) return IEX_ERR_BAD_ARG;
  if (m == 0 || nnz == 0) return IEX_OK;
  if (!plan || !lhs || !rhs || !out) return IEX_ERR_BAD_ARG;
  return sddmm_tc_launch(m, k, n, 1, &nnz, &plan, &lhs, &rhs, &out, accumulate, stream);
}

extern "C" int iex_sddmm_f32_tc_batched(int count, int m, int k, int n, const int* nnz, const void* const* plans,
                                        const float* const* lhs, const float* const* rhs, float* const* outs,
                                        int accumulate, void* stream) {
  return sddmm_tc_launch(m, k, n, count, nnz, plans, lhs, rhs, outs, accumulate, stream);
}

extern "C" int iex_sddmm_f32_tc_max_batch(void) { return iex::sddmm_tc::kMaxProblems; }

// CSR SpMM on tensor cores (tcgen05 / TMEM, sm_100a), fp32 in and out:
//   out[r, :] = sum_p values[p] * dense[col[p], :]          dense [k, n], n = 32 or 64.
//
// A CUDA-core SpMM gathers one dense row (4n bytes) through L1 / L2 per nonzero; at a few per
// cent density that gather traffic is twenty times the operands and the L2 -> SM fabric bounds
// the kernel.  Here a 128-row band of the sparse matrix is expanded, 64 columns at a time, into
// a dense shared-memory operand and multiplied with the matching 64 rows of `dense` on the
// tensor cores, so every dense row is loaded once per band instead of once per nonzero.
//
// fp32 accuracy on a TF32 pipe: every value x of either operand is split into hi = tf32(x) and
// lo = x - hi (exact) and a tile is accumulated as lo*hi' + hi*lo' + hi*hi' in an fp32 TMEM
// accumulator (error below 2^-19 of sum |a||b|).
//
// The nonzeros of a (band, 64-column tile) come from a tile plan of the pattern (tile_plan.cuh,
// built once per pattern): a flat list of (row, column, position in storage order), so the
// expansion is a branch-free pass of all threads over a coalesced list.
//
// One persistent CTA per SM walks "units": a band and a run of its tiles.  A band cut into
// several units gives several partial results, which go to a workspace and are added in unit
// order by a second small kernel (results do not depend on timing).
//   warps 0-3   converters: the tile's 64 rows of `dense` from global memory (coalesced 128-bit
//               loads, one tile ahead in registers), split into hi / lo planes in the MN-major
//               layout tcgen05.mma reads (128-byte swizzle with 32-byte atomicity).
//   warps 4-11  expanders: each thread takes list entries of the tile (entry, position and value
//               fetched two tiles / one tile ahead), splits the value and stores hi and lo at
//               (row, column) of the A planes.  A stage's planes are all zero except for the
//               tile's entries; when the tensor core has released the stage, the same threads
//               first write zeros back over the entries of the tile before last (cheaper than
//               clearing 64 KB).  At the end of a unit they read the accumulator (tcgen05.ld)
//               and store the band's (partial) result.
//   warp 12     one thread issues the 24 tcgen05.mma.kind::tf32 (M = 128, N = n, K = 8) of a tile
//               and releases the stage with tcgen05.commit.
// Every mbarrier wait is bounded.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_prof.cuh"
#include "tile_plan.cuh"

namespace iex {
namespace spmm_tc {

using namespace iex::tc;

constexpr int TM = 128;            // rows per band (UMMA M)
constexpr int TK = 64;             // columns of the sparse matrix per tile (K of a stage)
constexpr int kConvWarps = 4;
constexpr int kFirstExpWarp = 4;   // warps 4..11: (warp & 3) = 0, 1, 2, 3, 0, 1, 2, 3
constexpr int kExpWarps = 8;
constexpr int kMmaWarp = 12;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr int kStages = 2;
constexpr int kEntriesInRegs = 4;  // list entries per expander thread kept in registers per tile
constexpr int kAtomBytesA = TM * 128;   // one 32-column K atom of a 128-row A plane
constexpr int kPlaneA = 2 * kAtomBytesA;  // hi or lo plane of a stage's A operand (64 columns)
constexpr int kAtomBytesB = TK * 128;   // one 32-float N atom of a 64-row B plane
constexpr int kBarBytes = 128;

struct Params {
  int m, k, n, nnz;
  const int* tile_ptr;
  const uint16_t* entry;
  const int* dest;
  const float* values;
  const float* dense;
  float* out;       // final result, written directly when a band is one unit
  float* partials;  // [unit][128][n] otherwise
  int tiles_per_band;
  int units, base_splits, bands_hi;
  int* status;
  IEX_PROF_FIELD
};

__device__ __forceinline__ void unit_of(int u, const Params& p, int& band, int& t0, int& t1, int& splits) {
  const int hi_units = p.bands_hi * (p.base_splits + 1);
  int s;
  if (u < hi_units) {
    splits = p.base_splits + 1;
    band = u / splits;
    s = u - band * splits;
  } else {
    splits = p.base_splits;
    const int v = u - hi_units;
    band = p.bands_hi + v / splits;
    s = v - (v / splits) * splits;
  }
  t0 = static_cast<int>(static_cast<long long>(s) * p.tiles_per_band / splits);
  t1 = static_cast<int>(static_cast<long long>(s + 1) * p.tiles_per_band / splits);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Byte offset of element (row, col) inside an A plane: [2 K atoms][128 rows][128 bytes], the
// 16-byte pieces of a row XOR-swizzled by (row & 7).
__device__ __forceinline__ uint32_t a_offset(uint32_t rc) {
  const uint32_t row = rc >> 7, col = rc & 63u;
  return (col >> 5) * kAtomBytesA + row * 128u + ((((col & 31u) >> 2) ^ (row & 7u)) << 4) + (col & 3u) * 4u;
}

// Shared-memory matrix descriptor for an MN-major operand of 32-bit elements: the only layout
// tcgen05 takes for it is the 128-byte swizzle with 32-byte atomicity (layout type 1): rows of
// 128 bytes (32 elements along N) per k, the four 32-byte pieces of a row XOR-ed with (k & 3),
// atoms of 4 k-rows.  lbo = bytes between 32-element groups along N, sbo = bytes between atoms
// of 4 k-rows.
__device__ __forceinline__ uint64_t smem_desc_mn32(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) |
         (static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (1ull << 61);
}

__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// NT = n / 32 (N atoms of the dense operand): 1 or 2.
template <int NT>
__global__ void __launch_bounds__(kThreads, 1) spmm_tc_kernel(const Params prm) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kPlaneB = NT * kAtomBytesB;
  constexpr uint32_t kStageBytes = 2u * kPlaneA + 2u * kPlaneB;
  constexpr int N = NT * 32;
  auto a_hi = [&](int s) { return smem_base + static_cast<uint32_t>(s) * kStageBytes; };
  auto b_hi = [&](int s) { return a_hi(s) + 2u * kPlaneA; };
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 16u + 8u * s; };
  const uint32_t acc_full = bar_base + 32u, acc_empty = bar_base + 40u, exp_bar = bar_base + 56u;
  const uint32_t tmem_slot = bar_base + 48u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_off = bar_base - smem_base;
  volatile uint32_t* tmem_ptr_generic = reinterpret_cast<volatile uint32_t*>(smem_aligned + bar_off + 48u);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_aligned + bar_off + 52u);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = N < 32 ? 32 : N;

  // the A planes start out all zero
  for (uint32_t i = threadIdx.x; i < kStages * 2u * kPlaneA / 16u; i += kThreads) {
    const uint32_t s = i / (2u * kPlaneA / 16u), o = i - s * (2u * kPlaneA / 16u);
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(a_hi(s) + 16u * o), "r"(0u) : "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), kConvWarps + kExpWarps);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kExpWarps);
    mbar_init(exp_bar, kExpWarps);
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

  const int T = prm.tiles_per_band;

  if (warp < kConvWarps) {
    // ------------------------------------------------------------------ converters (dense rows)
    constexpr int kv_shift = NT == 1 ? 3 : 4;            // log2(float4 per dense row)
    constexpr int NV = TK * NT * 8 / (kConvWarps * 32);  // float4 per thread per tile
    const int ct = threadIdx.x;
    uint32_t off[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = ct + j * (kConvWarps * 32);
      const int row = i >> kv_shift, c4 = i & ((1 << kv_shift) - 1);
      // [N atom of 32 floats][k row][128 bytes], 32-byte pieces XOR-ed with (k row & 3)
      off[j] = static_cast<uint32_t>((c4 >> 3) * kAtomBytesB + row * 128 + ((((c4 & 7) >> 1) ^ (row & 3)) << 5) +
                                     (c4 & 1) * 16);
    }
    auto load_tile = [&](float4(&v)[NV], int t) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = ct + j * (kConvWarps * 32);
        const int row = t * TK + (i >> kv_shift), c4 = i & ((1 << kv_shift) - 1);
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < prm.k) v[j] = __ldg(reinterpret_cast<const float4*>(prm.dense + static_cast<size_t>(row) * N) + c4);
      }
    };
    uint32_t it = 0;
    bool ok = true;
    IEX_PROF_BEGIN
    for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
      int band, t0, t1, splits;
      unit_of(u, prm, band, t0, t1, splits);
      float4 v[NV];
      load_tile(v, t0);
      IEX_LAP(0)  // unit start
      for (int t = t0; t < t1; ++t, ++it) {
        const int s = it & 1u;
        if (!mbar_wait(empty_bar(s), ((it >> 1) & 1u) ^ 1u, abort_flag, prm.status, 32)) { ok = false; break; }
        IEX_LAP(1)  // waiting for a free stage
        const uint32_t hi = b_hi(s), lo = hi + kPlaneB;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const float hx = tf32_round(v[j].x), hy = tf32_round(v[j].y), hz = tf32_round(v[j].z),
                      hw = tf32_round(v[j].w);
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(hi + off[j]), "f"(hx), "f"(hy), "f"(hz), "f"(hw)
                       : "memory");
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(lo + off[j]), "f"(v[j].x - hx),
                       "f"(v[j].y - hy), "f"(v[j].z - hz), "f"(v[j].w - hw)
                       : "memory");
        }
        IEX_LAP(2)  // split + store
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
        if (t + 1 < t1) load_tile(v, t + 1);
        IEX_LAP(3)  // fence, arrive, next loads issued
      }
    }
    IEX_PROF_DUMP(threadIdx.x == 0, 0)
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // D fp32, A tf32 K-major, B tf32 MN-major, N = n, M = 128
      constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) |
                                 (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(TM >> 4) << 24);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      IEX_PROF_BEGIN
      for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x, ++ui) {
        int band, t0, t1, splits;
        unit_of(u, prm, band, t0, t1, splits);
        if (!mbar_wait(acc_empty, (ui & 1u) ^ 1u, abort_flag, prm.status, 32)) { ok = false; break; }
        IEX_LAP(0)  // waiting for the accumulator
        for (int t = t0; t < t1; ++t, ++it) {
          const int s = it & 1u;
          if (!mbar_wait(full_bar(s), (it >> 1) & 1u, abort_flag, prm.status, 32)) { ok = false; break; }
          IEX_LAP(1)  // waiting for a filled stage
          tcgen05_fence_after();
          // small terms first: lo * hi', hi * lo', then hi * hi'
          const uint32_t a_plane[3] = {a_hi(s) + kPlaneA, a_hi(s), a_hi(s)};
          const uint32_t b_plane[3] = {b_hi(s), b_hi(s) + kPlaneB, b_hi(s)};
#pragma unroll
          for (int pr = 0; pr < 3; ++pr) {
#pragma unroll
            for (int kk = 0; kk < TK / 8; ++kk) {  // 8 columns of A = 8 rows of dense per instruction
              const uint64_t adesc = smem_desc(a_plane[pr] + (kk >> 2) * kAtomBytesA + (kk & 3) * 32, 16, 1024);
              const uint64_t bdesc = smem_desc_mn32(b_plane[pr] + kk * 1024, kAtomBytesB, 512);
              umma_tf32(tmem_base, adesc, bdesc, idesc, (t != t0 || pr != 0 || kk != 0) ? 1u : 0u);
            }
          }
          umma_commit(empty_bar(s));
          IEX_LAP(2)  // issuing
        }
        if (ok) umma_commit(acc_full);
      }
      IEX_PROF_DUMP(true, 8)
    }
  } else {
    // ------------------------------------------------------------------ expanders
    const int ew = warp - kFirstExpWarp;  // 0..7
    const int et = ew * 32 + lane;        // 0..255
    constexpr int kET = kExpWarps * 32;
    const int* __restrict__ tile_ptr = prm.tile_ptr;
    const uint16_t* __restrict__ entry = prm.entry;
    const int* __restrict__ dest = prm.dest;
    const float* __restrict__ values = prm.values;
    // entries of the tiles the two stages hold (to be zeroed when a stage is refilled), of the
    // tile being expanded, and of the next one
    uint32_t held[kStages][kEntriesInRegs];
    int held_beg[kStages], held_end[kStages];
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      held_beg[s] = held_end[s] = 0;
#pragma unroll
      for (int i = 0; i < kEntriesInRegs; ++i) held[s][i] = 0xffffffffu;
    }
    uint32_t it = 0, ui = 0, sync_it = 0;
    bool ok = true;
    IEX_PROF_BEGIN
    // all expander warps meet (bounded wait)
    auto exp_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(exp_bar);
      const bool done = mbar_wait(exp_bar, sync_it & 1u, abort_flag, prm.status, 20);
      ++sync_it;
      __syncwarp();
      return done;
    };
    for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x, ++ui) {
      int band, t0, t1, splits;
      unit_of(u, prm, band, t0, t1, splits);
      const int tile0 = band * T;
      // Start of the entry list of tile t0 + j (j <= nt) comes from lane (j & 31)'s window
      // register; the window is reloaded every 31 tiles.  Entries and positions are fetched two
      // tiles ahead and values one tile ahead, so that no load of the list sits on the path
      // between two tiles.
      const int nt = t1 - t0;
      int win_base = 0;
      int win = __ldg(tile_ptr + tile0 + t0 + min(lane, nt));
      auto list_start = [&](int j) {  // j in [win_base, win_base + 31]
        return __shfl_sync(0xffffffffu, win, j - win_base);
      };
      uint32_t rc0[kEntriesInRegs], rc1[kEntriesInRegs], rc2[kEntriesInRegs];
      float val0[kEntriesInRegs], val1[kEntriesInRegs];
      int de1[kEntriesInRegs], de2[kEntriesInRegs];
      auto fetch_entries = [&](uint32_t(&rc)[kEntriesInRegs], int(&de)[kEntriesInRegs], int beg, int end) {
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) {
          const int e = beg + et + i * kET;
          rc[i] = e < end ? __ldg(entry + e) : 0xffffffffu;
          de[i] = e < end ? __ldg(dest + e) : -1;
        }
      };
      auto fetch_values = [&](float(&val)[kEntriesInRegs], const int(&de)[kEntriesInRegs]) {
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) val[i] = de[i] >= 0 ? __ldg(values + de[i]) : 0.f;
      };
      int e_beg = list_start(0), e_end = list_start(1);
      int e1_end = nt > 1 ? list_start(2) : e_end;
      {
        int de0[kEntriesInRegs];
        fetch_entries(rc0, de0, e_beg, e_end);
        fetch_entries(rc1, de1, e_end, e1_end);
        fetch_values(val0, de0);
      }
      for (int t = t0; t < t1; ++t, ++it) {
        const int s = it & 1u;
        const int j = t - t0;
        if (j + 3 - win_base > 31) {  // slide the window of list starts
          win_base = j;
          win = __ldg(tile_ptr + tile0 + t0 + min(win_base + lane, nt));
        }
        // two tiles ahead: entries and positions; one tile ahead: values
        const int e2_end = j + 2 < nt ? list_start(j + 3) : e1_end;
        fetch_entries(rc2, de2, e1_end, e2_end);
        fetch_values(val1, de1);
        IEX_LAP(0)  // list loads issued
        if (!mbar_wait(empty_bar(s), ((it >> 1) & 1u) ^ 1u, abort_flag, prm.status, 32)) { ok = false; break; }
        IEX_LAP(1)  // waiting for a free stage
        const uint32_t hi = a_hi(s), lo = hi + kPlaneA;
        // zeros back over what the stage held
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i)
          if (held[s][i] != 0xffffffffu) {
            const uint32_t o = a_offset(held[s][i]);
            sts_f32(hi + o, 0.f);
            sts_f32(lo + o, 0.f);
          }
        for (int e = held_beg[s] + et + kEntriesInRegs * kET; e < held_end[s]; e += kET) {
          const uint32_t o = a_offset(__ldg(entry + e));
          sts_f32(hi + o, 0.f);
          sts_f32(lo + o, 0.f);
        }
        // an element may belong to the old tile through one thread and to the new one through
        // another: all zeros are in place before the first new value goes in
        IEX_LAP(2)  // zeros over the old entries
        if (!exp_sync()) { ok = false; break; }
        IEX_LAP(3)  // meeting
        // this tile's entries
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) {
          held[s][i] = rc0[i];
          if (rc0[i] != 0xffffffffu) {
            const uint32_t o = a_offset(rc0[i]);
            const float h = tf32_round(val0[i]);
            sts_f32(hi + o, h);
            sts_f32(lo + o, val0[i] - h);
          }
        }
        for (int e = e_beg + et + kEntriesInRegs * kET; e < e_end; e += kET) {
          const uint32_t o = a_offset(__ldg(entry + e));
          const float x = __ldg(values + __ldg(dest + e));
          const float h = tf32_round(x);
          sts_f32(hi + o, h);
          sts_f32(lo + o, x - h);
        }
        held_beg[s] = e_beg;
        held_end[s] = e_end;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
#pragma unroll
        for (int i = 0; i < kEntriesInRegs; ++i) {
          rc0[i] = rc1[i];
          val0[i] = val1[i];
          rc1[i] = rc2[i];
          de1[i] = de2[i];
        }
        e_beg = e_end;
        e_end = e1_end;
        e1_end = e2_end;
        IEX_LAP(4)  // new entries, fence, arrive
      }
      if (!ok) break;
      // ---- the band's (partial) result: TMEM -> global
      if (!mbar_wait(acc_full, ui & 1u, abort_flag, prm.status, 64)) { ok = false; break; }
      __syncwarp();
      IEX_LAP(5)  // waiting for the unit's last MMA
      tcgen05_fence_after();
      {
        const int q = warp & 3, half = ew >> 2;
        constexpr int kCols = N / 2;  // columns per warp: 16 or 32
        const int row_local = q * 32 + lane;
        const int row = band * TM + row_local;
        const uint32_t tacc = tmem_base + half * kCols + (static_cast<uint32_t>(q * 32) << 16);
        // straight to the result when no band of this launch is cut into several units
        const bool direct = prm.partials == nullptr;
        float* dst = direct ? prm.out + static_cast<size_t>(row) * N + half * kCols
                            : prm.partials + (static_cast<size_t>(u) * TM + row_local) * N + half * kCols;
        const bool store = !direct || row < prm.m;
        uint32_t r[32];
        if constexpr (kCols == 32) {
          tmem_ld32(tacc, r);
        } else {
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
              "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(tacc)
              : "memory");
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty);
        if (store) {
#pragma unroll
          for (int v4 = 0; v4 < kCols / 4; ++v4)
            reinterpret_cast<uint4*>(dst)[v4] = make_uint4(r[4 * v4], r[4 * v4 + 1], r[4 * v4 + 2], r[4 * v4 + 3]);
        }
      }
      IEX_LAP(6)  // result to global memory
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
  }
}

// out[band rows] = sum over the band's units, in unit order, of their partial tiles.
__global__ void __launch_bounds__(256) spmm_tc_reduce_kernel(const Params prm) {
  grid_dependency_wait();
  grid_launch_dependents();
  const int band = blockIdx.x;
  const int n4 = prm.n / 4;
  const int hi_units = prm.bands_hi * (prm.base_splits + 1);
  const int splits = band < prm.bands_hi ? prm.base_splits + 1 : prm.base_splits;
  const int u0 = band < prm.bands_hi ? band * splits : hi_units + (band - prm.bands_hi) * splits;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < TM * n4; f += gridDim.y * blockDim.x) {
    const int row_local = f / n4;
    const int row = band * TM + row_local;
    if (row >= prm.m) continue;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 t = __ldcg(reinterpret_cast<const float4*>(prm.partials + static_cast<size_t>(u0 + s) * TM * prm.n) + f);
      sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
    }
    reinterpret_cast<float4*>(prm.out + static_cast<size_t>(band) * TM * prm.n)[f] = sum;
  }
}

template <int NT>
int launch(const Params& prm, cudaStream_t stream) {
  constexpr size_t smem = 1024 + kStages * (2 * static_cast<size_t>(kPlaneA) + 2 * static_cast<size_t>(NT) * kAtomBytesB) + kBarBytes;
  auto kern = spmm_tc_kernel<NT>;
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
  const int grid = prm.units < sms ? prm.units : sms;
  int st = launch_overlapped(kern, dim3(grid), dim3(kThreads), smem, stream, prm);
  if (st == 0 && prm.partials != nullptr) {
    const int bands = (prm.m + TM - 1) / TM;
    const int slices = (TM * prm.n / 4 + 255) / 256;
    st = launch_overlapped(spmm_tc_reduce_kernel, dim3(bands, slices), dim3(256), 0, stream, prm);
  }
  return st;
}

// Unit decomposition of an m x k matrix: runs per band so that every SM gets a unit.
void decompose(int m, int k, int* base_splits, int* bands_hi, int* units) {
  const int bands = (m + TM - 1) / TM, T = (k + TK - 1) / TK;
  const int sms = sm_count();
  int base = bands >= sms ? 1 : sms / bands;
  int rem = bands >= sms ? 0 : sms % bands;
  if (base >= T) { base = T; rem = 0; }
  *base_splits = base;
  *bands_hi = rem;
  *units = rem * (base + 1) + (bands - rem) * base;
}

}  // namespace spmm_tc
}  // namespace iex

extern "C" int iex_spmm_f32_tc_supported(int m, int k, int n) {
  return (m > 0 && k > 0 && (n == 32 || n == 64)) ? 1 : 0;
}

extern "C" int iex_spmm_f32_prefers_tc(int m, int k, int n, int nnz) {
  if (!iex_spmm_f32_tc_supported(m, k, n)) return 0;
  // A K = 8 TF32 instruction is bound by the bandwidth of its shared-memory operands (about 75
  // cycles whatever n is), so this kernel's time follows m * k: it passes the gather-bound
  // CUDA-core kernels from about 8 % density on.
  const long long tiles = static_cast<long long>((m + 127) / 128) * ((k + 63) / 64);
  return tiles >= 128 && static_cast<long long>(nnz) * 12 >= static_cast<long long>(m) * k ? 1 : 0;
}

extern "C" size_t iex_spmm_f32_tc_workspace_bytes(int m, int k, int n) {
  using namespace iex::spmm_tc;
  if (!iex_spmm_f32_tc_supported(m, k, n)) return 0;
  int base, rem, units;
  decompose(m, k, &base, &rem, &units);
  if (base == 1 && rem == 0) return 0;
  return static_cast<size_t>(units) * TM * n * sizeof(float);
}

#ifdef IEX_TC_PROFILE
static long long* g_spmm_prof_buffer = nullptr;
extern "C" void iex_spmm_f32_tc_set_profile_buffer(long long* device_buffer) { g_spmm_prof_buffer = device_buffer; }
#endif

extern "C" int iex_spmm_f32_tc(int m, int k, int n, int nnz, const void* plan, const float* values,
                               const float* dense, float* out, void* workspace, size_t workspace_bytes,
                               void* stream) {
  using namespace iex;
  using namespace iex::spmm_tc;
  if (m < 0 || k < 0 || n < 0 || nnz < 0) return IEX_ERR_BAD_ARG;
  if (m == 0 || n == 0) return IEX_OK;
  if (!plan || !dense || !out || (nnz > 0 && !values) || !aligned16(plan)) return IEX_ERR_BAD_ARG;
  if (!iex_spmm_f32_tc_supported(m, k, n) || !aligned16(dense) || !aligned16(out)) return IEX_ERR_UNSUPPORTED;
  const tile_plan::Layout L = tile_plan::layout(m, k, nnz, TK);
  const uint8_t* base = static_cast<const uint8_t*>(plan);
  Params p{};
  p.m = m;
  p.k = k;
  p.n = n;
  p.nnz = nnz;
  p.tile_ptr = reinterpret_cast<const int*>(base + L.tile_ptr);
  p.entry = reinterpret_cast<const uint16_t*>(base + L.entry);
  p.dest = reinterpret_cast<const int*>(base + L.dest);
  p.values = values;
  p.dense = dense;
  p.out = out;
  p.tiles_per_band = L.tiles_per_band;
  p.status = tc::status_word();
#ifdef IEX_TC_PROFILE
  p.prof = g_spmm_prof_buffer;
#endif
  decompose(m, k, &p.base_splits, &p.bands_hi, &p.units);
  const size_t need = iex_spmm_f32_tc_workspace_bytes(m, k, n);
  p.partials = nullptr;
  if (need > 0) {
    if (!workspace || !aligned16(workspace)) return IEX_ERR_BAD_ARG;
    if (workspace_bytes < need) return IEX_ERR_TOO_LARGE;
    p.partials = static_cast<float*>(workspace);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return n == 32 ? launch<1>(p, s) : launch<2>(p, s);
}

#include "common.cuh"
#include "tile_plan.cuh"

namespace iex {
namespace tile_plan {

// Building a tile plan (tile_plan.cuh): a counting sort of the stored positions by tile that
// keeps the storage order inside a tile.  Three small kernels on the caller's stream:
//   count   one warp per row walks the row's indices and adds, per tile the row touches, the
//           number of its entries there into counts[tile][row in band]   (indices need not
//           ascend)
//   scan    one block: exclusive prefix sum over counts in (tile, row) order -> where each
//           (tile, row) run starts; tile_ptr[tile] = the start of its first row
//   fill    one warp per row again: every entry goes to its run, in storage order
// counts / starts live in the plan's own scratch part.
__global__ void __launch_bounds__(256) plan_count_kernel(int m, int T, int shift, const int* __restrict__ row_offsets,
                                                         const int* __restrict__ cols, int* __restrict__ cells) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= m) return;
  const int band = row >> 7, rl = row & 127;
  const int beg = __ldg(row_offsets + row), end = __ldg(row_offsets + row + 1);
  for (int p = beg + lane; p < end; p += 32) {
    const int t = __ldg(cols + p) >> shift;
    if (t >= 0 && t < T) atomicAdd(cells + (static_cast<size_t>(band) * T + t) * kBandRows + rl, 1);
  }
}

// cells[tile][row] : count -> exclusive start (in place); tile_ptr[tile]; one block of 1024.
__global__ void __launch_bounds__(1024) plan_scan_kernel(int ncells, int ntiles, int* __restrict__ cells,
                                                         int* __restrict__ tile_ptr) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < ncells; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < ncells ? cells[i] : 0;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int incl = x + (warp > 0 ? warp_sums[warp - 1] : 0) + carry_s;
    if (i < ncells) {
      cells[i] = incl - v;
      if ((i & (kBandRows - 1)) == 0) tile_ptr[i >> 7] = incl - v;
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) tile_ptr[ntiles] = carry_s;
}

__global__ void __launch_bounds__(256) plan_fill_kernel(int m, int T, int shift, const int* __restrict__ row_offsets,
                                                        const int* __restrict__ cols, int* __restrict__ cells,
                                                        uint16_t* __restrict__ entry, int* __restrict__ dest) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= m) return;
  const int band = row >> 7, rl = row & 127;
  const int beg = __ldg(row_offsets + row), end = __ldg(row_offsets + row + 1);
  // Entries of one row and one tile keep their storage order: within a pass of 32 entries a
  // lane's rank among the lanes of the same tile comes from a match mask, and the warp bumps
  // the cell's running start once per tile and pass.
  for (int p0 = beg; p0 < end; p0 += 32) {
    const int p = p0 + lane;
    const bool on = p < end;
    const int c = on ? __ldg(cols + p) : -1;
    const int t = c >> shift;
    const bool ok = on && t >= 0 && t < T;
    const unsigned peers = __match_any_sync(0xffffffffu, ok ? t : -1 - lane);
    if (ok) {
      int* cell = cells + (static_cast<size_t>(band) * T + t) * kBandRows + rl;
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int leader = __ffs(peers) - 1;
      int start = 0;
      if (lane == leader) {
        start = *cell;
        *cell = start + __popc(peers);
      }
      start = __shfl_sync(peers, start, leader);
      entry[start + rank] = static_cast<uint16_t>((rl << 7) | (c & ((1 << shift) - 1)));
      dest[start + rank] = p;
    }
  }
}

}  // namespace tile_plan
}  // namespace iex

extern "C" size_t iex_tile_plan_bytes(int m, int n, int nnz, int tile_cols) {
  if (m <= 0 || n <= 0 || nnz < 0 || (tile_cols != 64 && tile_cols != 128)) return 0;
  return iex::tile_plan::layout(m, n, nnz, tile_cols).total;
}

extern "C" int iex_tile_plan_build(int m, int n, int nnz, int tile_cols, const int32_t* row_offsets,
                                   const int32_t* column_indices, void* plan, size_t plan_bytes, void* stream) {
  using namespace iex;
  using namespace iex::tile_plan;
  if (m < 0 || n < 0 || nnz < 0 || (tile_cols != 64 && tile_cols != 128)) return IEX_ERR_BAD_ARG;
  if (m == 0 || n == 0) return IEX_OK;
  if (!row_offsets || !plan || (nnz > 0 && !column_indices) || !aligned16(plan)) return IEX_ERR_BAD_ARG;
  const Layout L = layout(m, n, nnz, tile_cols);
  if (plan_bytes < L.total) return IEX_ERR_TOO_LARGE;
  const int shift = tile_cols == 64 ? 6 : 7;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(plan);
  int* cells = reinterpret_cast<int*>(base + L.cells);
  cudaError_t e = cudaMemsetAsync(cells, 0, 4 * static_cast<size_t>(L.ntiles) * kBandRows, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int blocks = (m + 7) / 8;
  plan_count_kernel<<<blocks, 256, 0, s>>>(m, L.tiles_per_band, shift, row_offsets, column_indices, cells);
  int st = launch_status();
  if (st) return st;
  plan_scan_kernel<<<1, 1024, 0, s>>>(L.ntiles * kBandRows, L.ntiles, cells, reinterpret_cast<int*>(base + L.tile_ptr));
  st = launch_status();
  if (st) return st;
  plan_fill_kernel<<<blocks, 256, 0, s>>>(m, L.tiles_per_band, shift, row_offsets, column_indices, cells,
                                          reinterpret_cast<uint16_t*>(base + L.entry),
                                          reinterpret_cast<int*>(base + L.dest));
  return launch_status();
}

// The SDDMM's plan: 128-column tiles.
extern "C" size_t iex_sddmm_plan_bytes(int m, int n, int nnz) { return iex_tile_plan_bytes(m, n, nnz, 128); }

extern "C" int iex_sddmm_plan_build(int m, int n, int nnz, const int32_t* row_offsets,
                                    const int32_t* column_indices, void* plan, size_t plan_bytes,
                                    void* stream) {
  return iex_tile_plan_build(m, n, nnz, 128, row_offsets, column_indices, plan, plan_bytes, stream);
}

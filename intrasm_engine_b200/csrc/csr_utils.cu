// CSR <-> dense helpers on the device.
//   * csr_to_dense (fp16): where an activation CSR becomes the tile operand of the
//     tensor-core linear (ReLU-sparse FFN down projection).
//   * dense_to_csr (fp16 / fp32, optional ReLU): builds row_offsets, the row visiting order
//     (rows by decreasing nnz, ties in row order), values and ascending column indices of a
//     dense matrix in two calls: "count" (row lengths, offsets, row order) and, once the
//     caller has read nnz = row_offsets[m] and allocated the arrays, "fill".
#include "common.cuh"

namespace iex {
namespace {

__device__ __forceinline__ bool keeps(float v, bool relu) { return relu ? v > 0.f : v != 0.f; }

// One warp per row: number of stored elements of the row.
template <typename T>
__global__ void __launch_bounds__(256)
row_count_kernel(int m, int k, const T* __restrict__ dense, int relu, int* __restrict__ row_nnz) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < m; r += warps) {
    const T* row = dense + static_cast<size_t>(r) * k;
    int cnt = 0;
    for (int c0 = 0; c0 < k; c0 += 32) {
      const int c = c0 + lane;
      const bool on = c < k && keeps(to_float(row[c]), relu != 0);
      cnt += __popc(__ballot_sync(0xffffffffu, on));
    }
    if (lane == 0) row_nnz[r] = cnt;
  }
}

// One block: row_offsets[0..m] = exclusive prefix sum of row_nnz (chunks of 1024 rows).
__global__ void __launch_bounds__(1024) row_scan_kernel(int m, const int* __restrict__ row_nnz,
                                                        int* __restrict__ row_offsets) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { carry_s = 0; row_offsets[0] = 0; }
  __syncthreads();
  for (int base = 0; base < m; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < m ? row_nnz[i] : 0;
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
    if (i < m) row_offsets[i + 1] = incl;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = incl;
    __syncthreads();
  }
}

// Row visiting order: position of row r = number of rows with more nonzeros, plus the rows
// before r with as many (a stable descending sort, computed as a rank: every thread compares
// its row with all others, staged through shared memory in chunks).
__global__ void __launch_bounds__(256) row_rank_kernel(int m, const int* __restrict__ row_nnz,
                                                       int* __restrict__ row_indices) {
  __shared__ int chunk[1024];
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const int mine = r < m ? row_nnz[r] : 0;
  int rank = 0;
  for (int base = 0; base < m; base += 1024) {
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) chunk[i] = base + i < m ? row_nnz[base + i] : -1;
    __syncthreads();
    const int lim = min(1024, m - base);
    for (int i = 0; i < lim; ++i) {
      const int o = chunk[i];
      rank += (o > mine || (o == mine && base + i < r)) ? 1 : 0;
    }
    __syncthreads();
  }
  if (r < m) row_indices[rank] = r;
}

// One warp per row: stored elements and their column indices, in column order.
template <typename T, typename IT>
__global__ void __launch_bounds__(256)
row_fill_kernel(int m, int k, const T* __restrict__ dense, int relu, const int* __restrict__ row_offsets,
                T* __restrict__ values, IT* __restrict__ cols) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < m; r += warps) {
    const T* row = dense + static_cast<size_t>(r) * k;
    int pos = row_offsets[r];
    for (int c0 = 0; c0 < k; c0 += 32) {
      const int c = c0 + lane;
      const T v = c < k ? row[c] : T(0);
      const bool on = c < k && keeps(to_float(v), relu != 0);
      const unsigned b = __ballot_sync(0xffffffffu, on);
      if (on) {
        const int p = pos + __popc(b & ((1u << lane) - 1u));
        values[p] = v;
        cols[p] = static_cast<IT>(c);
      }
      pos += __popc(b);
    }
  }
}

// CTA (x, y) owns the columns [y * slice, (y + 1) * slice) of rows x, x + gridDim.x, ...: it
// clears its piece of the dense row with 128-bit stores and then writes the row's nonzeros
// that fall into it.  A few CTAs per row instead of one keep each CTA's work down to one or
// two instructions per thread, so the kernel is as long as its chain of three dependent memory
// round trips (row offsets, indices and values, stores) and no longer; the row's offsets and
// its first indices and values are requested before the clearing stores, not after.
template <typename IT>
__global__ void __launch_bounds__(256)
csr_to_dense_f16_kernel(int m, int k, int slice, const int* __restrict__ row_offsets, const IT* __restrict__ cols,
                        const __half* __restrict__ values, __half* __restrict__ out) {
  grid_dependency_wait();  // `out` may still be read by the kernel before this one
  grid_launch_dependents();
  const int c0 = blockIdx.y * slice;
  const int c1 = c0 + slice < k ? c0 + slice : k;
  const bool vec = (k & 7) == 0 && (slice & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  for (int r = blockIdx.x; r < m; r += gridDim.x) {
    __half* row = out + static_cast<size_t>(r) * k;
    const int beg = __ldg(row_offsets + r), end = __ldg(row_offsets + r + 1);
    int p = beg + threadIdx.x;
    int c = -1;
    __half v = __float2half(0.f);
    if (p < end) {
      c = to_index(__ldg(cols + p));
      v = __ldg(values + p);
    }
    if (vec) {
      uint4* row4 = reinterpret_cast<uint4*>(row);
      for (int i = (c0 >> 3) + threadIdx.x; i < (c1 >> 3); i += blockDim.x) row4[i] = make_uint4(0u, 0u, 0u, 0u);
    } else {
      for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) row[i] = __float2half(0.f);
    }
    __syncthreads();
    while (p < end) {
      if (c >= c0 && c < c1) row[c] = v;
      p += blockDim.x;
      if (p < end) {
        c = to_index(__ldg(cols + p));
        v = __ldg(values + p);
      }
    }
    __syncthreads();
  }
}

// CSR sanity check.  Threads stride over rows (offset rules, row order entries) and over
// nonzeros (column range, ascending order inside a row: position p belongs to a row boundary
// exactly when some offset equals p, which a binary search over row_offsets answers).
// Violations are OR-ed into one device word.
template <typename IT>
__global__ void __launch_bounds__(256)
csr_validate_kernel(int m, int k, int nnz, const int* __restrict__ row_offsets, const IT* __restrict__ cols,
                    const int* __restrict__ row_indices, int require_ascending, int* __restrict__ result) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const int nthreads = gridDim.x * blockDim.x;
  int bad = 0;
  if (tid == 0) {
    if (row_offsets[0] != 0) bad |= IEX_CSR_BAD_FIRST_OFFSET;
    if (row_offsets[m] != nnz) bad |= IEX_CSR_BAD_LAST_OFFSET;
  }
  for (int r = tid; r < m; r += nthreads) {
    const int a = row_offsets[r], b = row_offsets[r + 1];
    if (b < a || a < 0 || b > nnz) bad |= IEX_CSR_OFFSETS_NOT_MONOTONE;
    if (row_indices != nullptr) {
      const int v = row_indices[r];
      if (v < 0 || v >= m) bad |= IEX_CSR_BAD_ROW_INDEX;
    }
  }
  for (int p = tid; p < nnz; p += nthreads) {
    const int c = to_index(cols[p]);
    if (c < 0 || c >= k) bad |= IEX_CSR_COLUMN_OUT_OF_RANGE;
    if (require_ascending && p > 0) {
      // is p the first nonzero of a row?  largest r with row_offsets[r] <= p ...
      int lo = 0, hi = m;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (row_offsets[mid] <= p) lo = mid; else hi = mid - 1;
      }
      // ... starts the row holding p; p continues a row when that offset is below p
      if (row_offsets[lo] < p && to_index(cols[p - 1]) >= c) bad |= IEX_CSR_COLUMNS_NOT_ASCENDING;
    }
  }
  if (bad) atomicOr(result, bad);
}

}  // namespace
}  // namespace iex

extern "C" int iex_csr_validate(int m, int k, int nnz, const int32_t* row_offsets, const void* column_indices,
                                int index_bits, const int32_t* row_indices, int require_ascending,
                                int32_t* result, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || nnz < 0 || (index_bits != 16 && index_bits != 32)) return IEX_ERR_BAD_ARG;
  if (!row_offsets || !result || (nnz > 0 && !column_indices)) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(result, 0, sizeof(int32_t), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long work = static_cast<long long>(nnz) > m ? nnz : m;
  long long blocks = (work + 255) / 256;
  blocks = blocks < 1 ? 1 : (blocks > 8 * kNumSMs ? 8 * kNumSMs : blocks);
  if (index_bits == 16)
    csr_validate_kernel<uint16_t><<<static_cast<int>(blocks), 256, 0, s>>>(
        m, k, nnz, row_offsets, static_cast<const uint16_t*>(column_indices), row_indices, require_ascending,
        result);
  else
    csr_validate_kernel<int><<<static_cast<int>(blocks), 256, 0, s>>>(
        m, k, nnz, row_offsets, static_cast<const int*>(column_indices), row_indices, require_ascending, result);
  return launch_status();
}

extern "C" int iex_csr_to_dense_f16(int m, int k, const int32_t* row_offsets, const void* column_indices,
                                    int index_bits, const void* values, void* out, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || (index_bits != 16 && index_bits != 32)) return IEX_ERR_BAD_ARG;
  if (m == 0 || k == 0) return IEX_OK;
  if (!row_offsets || !out) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // about eight CTAs of 256 threads per SM in all: rows first, then up to eight column slices
  // (multiples of 8 columns) per row
  const int gx = m < 8 * kNumSMs ? m : 8 * kNumSMs;
  int slices = (8 * kNumSMs) / gx;
  slices = slices < 1 ? 1 : (slices > 8 ? 8 : slices);
  int slice = ((k + slices - 1) / slices + 7) & ~7;
  if (slice < 256) slice = 256 < k ? 256 : ((k + 7) & ~7);
  const int gy = (k + slice - 1) / slice;
  const dim3 grid(gx, gy);
  if (index_bits == 16)
    return launch_overlapped(csr_to_dense_f16_kernel<uint16_t>, grid, dim3(256), 0, s, m, k, slice, row_offsets,
                             static_cast<const uint16_t*>(column_indices), static_cast<const __half*>(values),
                             static_cast<__half*>(out));
  return launch_overlapped(csr_to_dense_f16_kernel<int>, grid, dim3(256), 0, s, m, k, slice, row_offsets,
                           static_cast<const int*>(column_indices), static_cast<const __half*>(values),
                           static_cast<__half*>(out));
}

extern "C" int iex_dense_to_csr_count(int m, int k, const void* dense, int value_bits, int relu,
                                      int32_t* row_offsets, int32_t* row_indices, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || (value_bits != 16 && value_bits != 32)) return IEX_ERR_BAD_ARG;
  if (!row_offsets || !row_indices || (m > 0 && k > 0 && !dense)) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the row lengths go to row_offsets[1..m], are ranked from there, then scanned in place
  int* lengths = row_offsets + 1;
  if (m > 0) {
    const int blocks = (m + 7) / 8 < 8 * kNumSMs ? (m + 7) / 8 : 8 * kNumSMs;
    if (value_bits == 16)
      row_count_kernel<__half><<<blocks, 256, 0, s>>>(m, k, static_cast<const __half*>(dense), relu, lengths);
    else
      row_count_kernel<float><<<blocks, 256, 0, s>>>(m, k, static_cast<const float*>(dense), relu, lengths);
    int st = launch_status();
    if (st) return st;
    row_rank_kernel<<<(m + 255) / 256, 256, 0, s>>>(m, lengths, row_indices);
    st = launch_status();
    if (st) return st;
  }
  row_scan_kernel<<<1, 1024, 0, s>>>(m, lengths, row_offsets);  // in place: reads [i+1], writes [i+1]
  return launch_status();
}

extern "C" int iex_dense_to_csr_fill(int m, int k, const void* dense, int value_bits, int relu,
                                     const int32_t* row_offsets, void* values, void* column_indices,
                                     int index_bits, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || (value_bits != 16 && value_bits != 32) || (index_bits != 16 && index_bits != 32))
    return IEX_ERR_BAD_ARG;
  if (index_bits == 16 && k > 65536) return IEX_ERR_UNSUPPORTED;
  if (m == 0 || k == 0) return IEX_OK;
  if (!dense || !row_offsets || !values || !column_indices) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = (m + 7) / 8 < 8 * kNumSMs ? (m + 7) / 8 : 8 * kNumSMs;
#define IEX_FILL(T, IT)                                                                              \
  row_fill_kernel<T, IT><<<blocks, 256, 0, s>>>(m, k, static_cast<const T*>(dense), relu, row_offsets, \
                                                static_cast<T*>(values), static_cast<IT*>(column_indices))
  if (value_bits == 16 && index_bits == 16) IEX_FILL(__half, uint16_t);
  else if (value_bits == 16) IEX_FILL(__half, int);
  else if (index_bits == 16) IEX_FILL(float, uint16_t);
  else IEX_FILL(float, int);
#undef IEX_FILL
  return launch_status();
}

// Sampled dense-dense matmul on CUDA cores (sm_100a):
//   out[p] = sum_z dot(lhs[z, row(p), :], rhs[z, col[p], :])   for every stored position p.
//
// Work decomposition
//   * A sub-warp of W lanes owns one row of the mask and walks its nonzeros in tiles of W.
//     The grid's y dimension splits long rows: sub-warp y takes tiles y, y+gridDim.y, ...
//     The grid is sized from nnz/m, not from the dense column count, so no CTA starts
//     only to find it has nothing to do.
//   * Lane i reads NV 128-bit vectors (4*NV consecutive k-values) of the lhs row and of each
//     gathered rhs row, so a rhs row is read as one coalesced segment.  Each lane keeps W
//     partial dot products (packed f32x2 FMAs), one per nonzero of the tile; all W gathers
//     of a tile are in flight together, and the next tile's column indices are fetched
//     while the current tile is computed.  Narrow sub-warps (8 lanes for k <= 64) put four
//     independent tiles in flight per warp: the kernel is bound by gather latency, so
//     memory-level parallelism is what counts.
//   * A butterfly exchange (W-1 shuffles instead of W*log2 W) leaves lane i with the full
//     dot product of nonzero i, and the tile's W results are stored as one coalesced row.
//   * Batch items are summed inside the kernel, in batch order: deterministic.
#include "common.cuh"

namespace iex {
namespace {

// NV = 128-bit vectors per lane per pass (0: scalar loads, any k / alignment).
template <int W, int NV>
__global__ void __launch_bounds__(128)
sddmm_rowtile_kernel(int m, int k, int n, const int* __restrict__ row_indices,
                     const int* __restrict__ row_offsets, const int* __restrict__ cols,
                     const float* __restrict__ lhs, const float* __restrict__ rhs,
                     float* __restrict__ out, int batch, int accumulate) {
  constexpr int KV = NV > 0 ? 4 * NV : 1;  // k-values per lane per pass
  constexpr int NVV = NV > 0 ? NV : 1;
  const int lane = threadIdx.x & 31;
  const int sub = lane / W;
  const int sl = lane % W;
  const unsigned submask = (W == 32) ? 0xffffffffu : (((1u << (W & 31)) - 1u) << (sub * W));
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int slot = warp * (32 / W) + sub;
  grid_dependency_wait();  // the kernel before this one may have written what is read below
  grid_launch_dependents();
  if (slot >= m) return;

  const int r = __ldg(row_indices + slot);
  const int beg = __ldg(row_offsets + r);
  const int end = __ldg(row_offsets + r + 1);

  int p0 = beg + blockIdx.y * W;
  int next_col = (p0 + sl < end) ? __ldg(cols + p0 + sl) : 0;
  for (; p0 < end; p0 += gridDim.y * W) {
    const int count = min(W, end - p0);
    const int my_col = next_col;
    {  // the next tile's indices travel while this tile is computed
      const int pn = p0 + gridDim.y * W + sl;
      next_col = (pn < end) ? __ldg(cols + pn) : 0;
    }

    float2 acc[W];
#pragma unroll
    for (int j = 0; j < W; ++j) acc[j] = make_float2(0.f, 0.f);

    for (int z = 0; z < batch; ++z) {
      const float* a_row = lhs + (static_cast<size_t>(z) * m + r) * k;
      const float* b_base = rhs + static_cast<size_t>(z) * n * k;
      for (int kc = 0; kc < k; kc += W * KV) {
        // Vector v of lane sl covers k-values [kc + v*4W + 4*sl, +4): the W lanes of one load
        // instruction read 16*W contiguous bytes, so every fetched 32-byte sector is used whole.
        const int kk = NV > 0 ? kc + sl * 4 : kc + sl;
        float4 a[NVV];
#pragma unroll
        for (int v = 0; v < NVV; ++v) {
          a[v] = make_float4(0.f, 0.f, 0.f, 0.f);
          if constexpr (NV > 0) {
            if (kk + 4 * W * v < k) a[v] = __ldg(reinterpret_cast<const float4*>(a_row + kk + 4 * W * v));
          } else {
            if (kk < k) a[v].x = __ldg(a_row + kk);
          }
        }
#pragma unroll
        for (int j = 0; j < W; ++j) {
          const int cj = __shfl_sync(submask, my_col, j, W);
          const float* b_row = b_base + static_cast<size_t>(cj) * k + kk;
#pragma unroll
          for (int v = 0; v < NVV; ++v) {
            if constexpr (NV > 0) {
              if (j < count && kk + 4 * W * v < k) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(b_row + 4 * W * v));
                acc[j] = ffma2(make_float2(a[v].x, a[v].y), make_float2(b.x, b.y), acc[j]);
                acc[j] = ffma2(make_float2(a[v].z, a[v].w), make_float2(b.z, b.w), acc[j]);
              }
            } else {
              if (j < count && kk < k) acc[j].x = fmaf(a[v].x, __ldg(b_row), acc[j].x);
            }
          }
        }
      }
    }

    // Butterfly: after the step with stride s a lane keeps the s partial sums whose
    // nonzero index agrees with its own lane index in bit s.
    float red[W];
#pragma unroll
    for (int j = 0; j < W; ++j) red[j] = acc[j].x + acc[j].y;
#pragma unroll
    for (int s = W / 2; s >= 1; s >>= 1) {
      const bool upper = (sl & s) != 0;
#pragma unroll
      for (int i = 0; i < s; ++i) {
        const float keep = upper ? red[i + s] : red[i];
        const float send = upper ? red[i] : red[i + s];
        red[i] = keep + __shfl_xor_sync(submask, send, s, W);
      }
    }
    if (sl < count) {
      if (accumulate) atomicAdd(out + p0 + sl, red[0]);
      else out[p0 + sl] = red[0];
    }
  }
}

template <int W, int NV>
int launch(int m, int k, int n, int nnz, const int* ri, const int* ro, const int* cols,
           const float* lhs, const float* rhs, float* out, int batch, int accumulate,
           cudaStream_t stream) {
  constexpr int kRowsPerBlock = 4 * (32 / W);
  // Split rows so that each sub-warp gets about two tiles of W nonzeros on average.
  const long long avg = m > 0 ? (static_cast<long long>(nnz) + m - 1) / m : 0;
  int split = static_cast<int>((avg + 2 * W - 1) / (2 * W));
  split = split < 1 ? 1 : (split > 64 ? 64 : split);
  dim3 grid((m + kRowsPerBlock - 1) / kRowsPerBlock, split, 1);
  return launch_overlapped(sddmm_rowtile_kernel<W, NV>, grid, dim3(128), 0, stream, m, k, n, ri, ro, cols, lhs, rhs,
                           out, batch, accumulate);
}


// fp16 operands, fp32 accumulation, fp16 result: the same decomposition with 8 k-values per
// 128-bit vector.  The reference declares this instantiation and leaves it commented out
// (sputnik_kernels.cpp:185-187); MySpMM's fp16 backward needs it, otherwise both operands
// would be converted to fp32 first.  NV = 0: scalar loads (any k / alignment).
template <typename IT, int W, int NV>
__global__ void __launch_bounds__(128)
sddmm_rowtile_half_kernel(int m, int k, int n, const int* __restrict__ row_indices,
                          const int* __restrict__ row_offsets, const IT* __restrict__ cols,
                          const __half* __restrict__ lhs, const __half* __restrict__ rhs,
                          __half* __restrict__ out, int batch) {
  constexpr int KV = NV > 0 ? 8 * NV : 1;
  constexpr int NVV = NV > 0 ? NV : 1;
  const int lane = threadIdx.x & 31;
  const int sub = lane / W;
  const int sl = lane % W;
  const unsigned submask = (W == 32) ? 0xffffffffu : (((1u << (W & 31)) - 1u) << (sub * W));
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int slot = warp * (32 / W) + sub;
  grid_dependency_wait();
  grid_launch_dependents();
  if (slot >= m) return;

  const int r = __ldg(row_indices + slot);
  const int beg = __ldg(row_offsets + r);
  const int end = __ldg(row_offsets + r + 1);

  int p0 = beg + blockIdx.y * W;
  int next_col = (p0 + sl < end) ? to_index(__ldg(cols + p0 + sl)) : 0;
  for (; p0 < end; p0 += gridDim.y * W) {
    const int count = min(W, end - p0);
    const int my_col = next_col;
    {
      const int pn = p0 + gridDim.y * W + sl;
      next_col = (pn < end) ? to_index(__ldg(cols + pn)) : 0;
    }
    float acc[W];
#pragma unroll
    for (int j = 0; j < W; ++j) acc[j] = 0.f;

    for (int z = 0; z < batch; ++z) {
      const __half* a_row = lhs + (static_cast<size_t>(z) * m + r) * k;
      const __half* b_base = rhs + static_cast<size_t>(z) * n * k;
      for (int kc = 0; kc < k; kc += W * KV) {
        const int kk = NV > 0 ? kc + sl * 8 : kc + sl;
        uint4 a[NVV];
#pragma unroll
        for (int v = 0; v < NVV; ++v) {
          a[v] = make_uint4(0u, 0u, 0u, 0u);
          if constexpr (NV > 0) {
            if (kk + 8 * W * v < k) a[v] = __ldg(reinterpret_cast<const uint4*>(a_row + kk + 8 * W * v));
          } else {
            if (kk < k) a[v].x = __half_as_ushort(__ldg(a_row + kk));
          }
        }
#pragma unroll
        for (int j = 0; j < W; ++j) {
          const int cj = __shfl_sync(submask, my_col, j, W);
          const __half* b_row = b_base + static_cast<size_t>(cj) * k + kk;
#pragma unroll
          for (int v = 0; v < NVV; ++v) {
            if constexpr (NV > 0) {
              if (j < count && kk + 8 * W * v < k) {
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(b_row + 8 * W * v));
                const __half2* ah = reinterpret_cast<const __half2*>(&a[v]);
                const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 af = __half22float2(ah[e]), bf = __half22float2(bh[e]);
                  acc[j] = fmaf(af.x, bf.x, acc[j]);
                  acc[j] = fmaf(af.y, bf.y, acc[j]);
                }
              }
            } else {
              if (j < count && kk < k)
                acc[j] = fmaf(__half2float(__ushort_as_half(static_cast<unsigned short>(a[v].x))),
                              __half2float(__ldg(b_row)), acc[j]);
            }
          }
        }
      }
    }
    // butterfly as in the fp32 kernel: lane i ends with the full sum of nonzero i
#pragma unroll
    for (int s = W / 2; s >= 1; s >>= 1) {
      const bool upper = (sl & s) != 0;
#pragma unroll
      for (int i = 0; i < s; ++i) {
        const float keep = upper ? acc[i + s] : acc[i];
        const float send = upper ? acc[i] : acc[i + s];
        acc[i] = keep + __shfl_xor_sync(submask, send, s, W);
      }
    }
    if (sl < count) out[p0 + sl] = __float2half_rn(acc[0]);
  }
}

template <typename IT, int W, int NV>
int launch_half(int m, int k, int n, int nnz, const int* ri, const int* ro, const IT* cols, const __half* lhs,
                const __half* rhs, __half* out, int batch, cudaStream_t stream) {
  constexpr int kRowsPerBlock = 4 * (32 / W);
  const long long avg = m > 0 ? (static_cast<long long>(nnz) + m - 1) / m : 0;
  int split = static_cast<int>((avg + 2 * W - 1) / (2 * W));
  split = split < 1 ? 1 : (split > 64 ? 64 : split);
  dim3 grid((m + kRowsPerBlock - 1) / kRowsPerBlock, split, 1);
  return launch_overlapped(sddmm_rowtile_half_kernel<IT, W, NV>, grid, dim3(128), 0, stream, m, k, n, ri, ro, cols,
                           lhs, rhs, out, batch);
}

template <typename IT>
int dispatch_half(int m, int k, int n, int nnz, const int* ri, const int* ro, const IT* cols, const __half* lhs,
                  const __half* rhs, __half* out, int batch, cudaStream_t s) {
  const bool vec = (k % 8 == 0) && aligned16(lhs) && aligned16(rhs);
  if (vec) {
    if (k <= 64) return launch_half<IT, 8, 1>(m, k, n, nnz, ri, ro, cols, lhs, rhs, out, batch, s);
    if (k <= 128) return launch_half<IT, 16, 1>(m, k, n, nnz, ri, ro, cols, lhs, rhs, out, batch, s);
    return launch_half<IT, 32, 1>(m, k, n, nnz, ri, ro, cols, lhs, rhs, out, batch, s);
  }
  if (k <= 8) return launch_half<IT, 8, 0>(m, k, n, nnz, ri, ro, cols, lhs, rhs, out, batch, s);
  if (k <= 16) return launch_half<IT, 16, 0>(m, k, n, nnz, ri, ro, cols, lhs, rhs, out, batch, s);
  return launch_half<IT, 32, 0>(m, k, n, nnz, ri, ro, cols, lhs, rhs, out, batch, s);
}

}  // namespace
}  // namespace iex

extern "C" int iex_sddmm_f32(int m, int k, int n, int nnz, const int32_t* row_indices,
                             const int32_t* row_offsets, const int32_t* column_indices,
                             const float* lhs, const float* rhs, float* out, int batch,
                             int accumulate, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || n < 0 || nnz < 0 || batch < 0) return IEX_ERR_BAD_ARG;
  if (m == 0 || nnz == 0) return IEX_OK;
  if (!row_indices || !row_offsets || !column_indices || !out) return IEX_ERR_BAD_ARG;
  if (batch > 0 && k > 0 && (!lhs || !rhs)) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = (k % 4 == 0) && aligned16(lhs) && aligned16(rhs);
#define IEX_GO(W, NV) \
  return launch<W, NV>(m, k, n, nnz, row_indices, row_offsets, column_indices, lhs, rhs, out, batch, accumulate, s)
  if (vec) {
    if (k <= 32) { IEX_GO(8, 1); }
    if (k <= 64) { IEX_GO(8, 2); }
    if (k <= 128) { IEX_GO(16, 2); }
    IEX_GO(32, 2);
  }
  if (k <= 8) { IEX_GO(8, 0); }
  if (k <= 16) { IEX_GO(16, 0); }
  IEX_GO(32, 0);
#undef IEX_GO
}

extern "C" int iex_sddmm_f16(int m, int k, int n, int nnz, const int32_t* row_indices,
                             const int32_t* row_offsets, const void* column_indices, int index_bits,
                             const void* lhs, const void* rhs, void* out, int batch, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || n < 0 || nnz < 0 || batch < 0 || (index_bits != 16 && index_bits != 32))
    return IEX_ERR_BAD_ARG;
  if (m == 0 || nnz == 0) return IEX_OK;
  if (!row_indices || !row_offsets || !column_indices || !out) return IEX_ERR_BAD_ARG;
  if (batch > 0 && k > 0 && (!lhs || !rhs)) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* a = static_cast<const __half*>(lhs);
  const __half* b = static_cast<const __half*>(rhs);
  __half* o = static_cast<__half*>(out);
  if (index_bits == 16)
    return dispatch_half<uint16_t>(m, k, n, nnz, row_indices, row_offsets,
                                   static_cast<const uint16_t*>(column_indices), a, b, o, batch, s);
  return dispatch_half<int>(m, k, n, nnz, row_indices, row_offsets, static_cast<const int*>(column_indices), a, b, o,
                            batch, s);
}

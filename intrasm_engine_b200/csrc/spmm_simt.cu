// CSR SpMM on CUDA cores (sm_100a): out[z, r, :] = sum_p values[p] * dense[z, col[p], :].
//
// The default for fp32 (spmm_tc.cu holds a TF32 head/tail tensor-core kernel that wins at
// densities of about 10 % and above) and for fp16 at high sparsity or small shapes; the
// moderate-sparsity fp16 case runs on the tensor-core kernel in tc_fused.cu.
//
// Work decomposition
//   * One sub-warp ("row group") of LPR lanes owns one row of A and one tile of
//     LPR * VD * NVEC output columns; a warp holds 32/LPR consecutive rows of the
//     swizzled order, which have similar length because that order is by decreasing nnz.
//   * The row's values and column indices are read with 128-bit loads, LPR*CHS nonzeros
//     per step (the row start is rounded down to a 16-byte boundary and the prefix is
//     skipped), and handed round the row group with warp shuffles — no shared memory, no
//     CTA barrier.
//   * For each nonzero the lanes read the gathered dense row with 128-bit loads
//     (coalesced across the row group) and accumulate in fp32 with packed f32x2 FMAs.
//   * Each output element is summed by exactly one lane, in storage order, so the result
//     does not depend on the launch shape.
#include "common.cuh"

namespace iex {
namespace {

template <typename VT> struct Elem;
template <> struct Elem<float> { static constexpr int kPerVec = 4; };
template <> struct Elem<__half> { static constexpr int kPerVec = 8; };

// Loads VD consecutive elements starting at p (16-byte aligned when VD > 1) as floats.
template <typename VT, int VD>
__device__ __forceinline__ void load_dense(const VT* __restrict__ p, float (&dst)[VD]) {
  if constexpr (VD == 1) {
    dst[0] = to_float(__ldg(p));
  } else if constexpr (sizeof(VT) == 4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
  } else {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      dst[2 * i] = f.x;
      dst[2 * i + 1] = f.y;
    }
  }
}

template <typename VT, int VD>
__device__ __forceinline__ void store_out(VT* __restrict__ p, const float (&src)[VD]) {
  if constexpr (VD == 1) {
    if constexpr (sizeof(VT) == 4) *p = src[0]; else *p = __float2half_rn(src[0]);
  } else if constexpr (sizeof(VT) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(src[0], src[1], src[2], src[3]);
  } else {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(src[2 * i], src[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  }
}

// Raw (unconverted) vector of VD dense elements, so that many gathers can be in flight
// without holding their fp32 expansion in registers.
template <typename VT, int VD> struct RawVec;
template <typename VT> struct RawVec<VT, 1> { VT x; };
template <> struct RawVec<float, 4> { float4 x; };
template <> struct RawVec<__half, 8> { uint4 x; };

template <typename VT, int VD>
__device__ __forceinline__ RawVec<VT, VD> load_raw(const VT* __restrict__ p) {
  RawVec<VT, VD> r;
  if constexpr (VD == 1) r.x = __ldg(p);
  else if constexpr (sizeof(VT) == 4) r.x = __ldg(reinterpret_cast<const float4*>(p));
  else r.x = __ldg(reinterpret_cast<const uint4*>(p));
  return r;
}
template <typename VT, int VD>
__device__ __forceinline__ void expand_raw(const RawVec<VT, VD>& r, float (&dst)[VD]) {
  if constexpr (VD == 1) {
    dst[0] = to_float(r.x);
  } else if constexpr (sizeof(VT) == 4) {
    dst[0] = r.x.x; dst[1] = r.x.y; dst[2] = r.x.z; dst[3] = r.x.w;
  } else {
    const __half2* h = reinterpret_cast<const __half2*>(&r.x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      dst[2 * i] = f.x;
      dst[2 * i + 1] = f.y;
    }
  }
}

// Loads CHS consecutive sparse values / indices starting at element p of the arrays.
template <typename VT, typename IT, int CHS>
__device__ __forceinline__ void load_sparse_chunk(const VT* __restrict__ values,
                                                  const IT* __restrict__ cols, int p,
                                                  int end, int nnz, float (&v)[CHS],
                                                  int (&c)[CHS]) {
#pragma unroll
  for (int e = 0; e < CHS; ++e) { v[e] = 0.f; c[e] = 0; }
  if (p >= end) return;
  bool vector_path = false;
  if constexpr (CHS > 1) {
    if (p + CHS <= nnz) {
      vector_path = true;
      // values: one 16-byte load; indices: CHS * sizeof(IT) bytes = 16 or 32.
      if constexpr (sizeof(VT) == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(values + p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      } else {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(values + p));
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
      }
      constexpr int kIdxVecs = CHS * sizeof(IT) / 16;
      constexpr int kPer = 16 / sizeof(IT);
#pragma unroll
      for (int q = 0; q < kIdxVecs; ++q) {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(cols + p) + q);
        const IT* s = reinterpret_cast<const IT*>(&t);
#pragma unroll
        for (int i = 0; i < kPer; ++i) c[q * kPer + i] = to_index(s[i]);
      }
    }
  }
  if (!vector_path) {
#pragma unroll
    for (int e = 0; e < CHS; ++e)
      if (p + e < end) {
        v[e] = to_float(__ldg(values + p + e));
        c[e] = to_index(__ldg(cols + p + e));
      }
  }
}

// LPR  lanes per row group (8, 16 or 32)     NVEC  dense vectors per lane
// VS   128-bit loads of the sparse arrays    VDN   128-bit loads/stores of dense/out
template <typename VT, typename IT, int LPR, int NVEC, bool VS, bool VDN>
__global__ void __launch_bounds__(128)
spmm_rowgroup_kernel(int m, int k, int n, int nnz, const int* __restrict__ row_indices,
                     const VT* __restrict__ values, long long values_batch_stride,
                     const int* __restrict__ row_offsets, const IT* __restrict__ cols,
                     const VT* __restrict__ dense, const float* __restrict__ bias,
                     VT* __restrict__ out, int accumulate) {
  constexpr int CHS = VS ? Elem<VT>::kPerVec : 1;
  constexpr int VD = VDN ? Elem<VT>::kPerVec : 1;
  constexpr int kTileCols = LPR * VD * NVEC;

  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int sl = lane % LPR;
  const unsigned submask =
      (LPR == 32) ? 0xffffffffu : (((1u << (LPR & 31)) - 1u) << (sub * LPR));
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int slot = warp * (32 / LPR) + sub;
  grid_dependency_wait();  // the kernel before this one may have written what is read below
  grid_launch_dependents();
  if (slot >= m) return;  // the whole row group leaves together

  const int r = __ldg(row_indices + slot);
  const int beg = __ldg(row_offsets + r);
  const int end = __ldg(row_offsets + r + 1);
  const int z = blockIdx.z;
  values += static_cast<size_t>(z) * static_cast<size_t>(values_batch_stride);
  dense += static_cast<size_t>(z) * k * n;
  out += static_cast<size_t>(z) * m * n;
  const int col0 = blockIdx.y * kTileCols + sl * VD;

  float2 acc2[NVEC][(VD + 1) / 2];
  float acc1[NVEC];  // VD == 1
#pragma unroll
  for (int v = 0; v < NVEC; ++v) {
    acc1[v] = 0.f;
#pragma unroll
    for (int i = 0; i < (VD + 1) / 2; ++i) acc2[v][i] = make_float2(0.f, 0.f);
  }

  // Memory-level parallelism: the next chunk of the row is loaded while the current one is
  // consumed, and the gathered dense rows of kJU source lanes (kJU * CHS nonzeros) are all
  // requested before the first FMA.  Loads are unconditional (padding lanes hold column 0,
  // a valid row); only the FMAs are predicated, and they run in storage order.
  constexpr int kWant = 16 / (CHS * NVEC) > 0 ? 16 / (CHS * NVEC) : 1;  // ~16 gathers in flight
  constexpr int kJU = kWant < LPR ? kWant : LPR;
  int base = VS ? (beg & ~(CHS - 1)) : beg;
  float v[CHS], vn[CHS];
  int c[CHS], cn[CHS];
  load_sparse_chunk<VT, IT, CHS>(values, cols, base + sl * CHS, end, nnz, v, c);
  for (; base < end; base += LPR * CHS) {
    load_sparse_chunk<VT, IT, CHS>(values, cols, base + LPR * CHS + sl * CHS, end, nnz, vn, cn);
    const int remaining = end - base;
    const int src_lanes = min(LPR, (remaining + CHS - 1) / CHS);
    for (int j0 = 0; j0 < src_lanes; j0 += kJU) {
      float vv[kJU][CHS];
      RawVec<VT, VD> b[kJU][CHS][NVEC];
#pragma unroll
      for (int jj = 0; jj < kJU; ++jj)
#pragma unroll
        for (int e = 0; e < CHS; ++e) {
          const int src = (j0 + jj) & (LPR - 1);
          vv[jj][e] = __shfl_sync(submask, v[e], src, LPR);
          const int cc = __shfl_sync(submask, c[e], src, LPR);
          const VT* brow = dense + static_cast<size_t>(cc) * n + col0;
#pragma unroll
          for (int q = 0; q < NVEC; ++q) {
            // columns past n are never stored; re-read the tile's first vector instead
            b[jj][e][q] = load_raw<VT, VD>(brow + ((col0 + q * LPR * VD < n) ? q * LPR * VD : 0));
          }
        }
#pragma unroll
      for (int jj = 0; jj < kJU; ++jj)
#pragma unroll
        for (int e = 0; e < CHS; ++e) {
          const int p = base + (j0 + jj) * CHS + e;
          if (j0 + jj < LPR && p >= beg && p < end) {  // uniform over the row group
#pragma unroll
            for (int q = 0; q < NVEC; ++q) {
              float bf[VD];
              expand_raw<VT, VD>(b[jj][e][q], bf);
              if constexpr (VD == 1) {
                acc1[q] = fmaf(vv[jj][e], bf[0], acc1[q]);
              } else {
#pragma unroll
                for (int i = 0; i < VD / 2; ++i)
                  acc2[q][i] = ffma2(make_float2(vv[jj][e], vv[jj][e]),
                                     make_float2(bf[2 * i], bf[2 * i + 1]), acc2[q][i]);
              }
            }
          }
        }
    }
#pragma unroll
    for (int e = 0; e < CHS; ++e) { v[e] = vn[e]; c[e] = cn[e]; }
  }

  const bool fuse_bias = bias != nullptr;
  const float bias_r = fuse_bias ? __ldg(bias + r) : 0.f;
#pragma unroll
  for (int q = 0; q < NVEC; ++q) {
    const int col = col0 + q * LPR * VD;
    if (col >= n) continue;
    float res[VD];
    if constexpr (VD == 1) {
      res[0] = acc1[q];
    } else {
#pragma unroll
      for (int i = 0; i < VD / 2; ++i) { res[2 * i] = acc2[q][i].x; res[2 * i + 1] = acc2[q][i].y; }
    }
    if (fuse_bias) {
#pragma unroll
      for (int i = 0; i < VD; ++i) { res[i] += bias_r; res[i] = res[i] > 0.f ? res[i] : 0.f; }
    }
    VT* dst = out + static_cast<size_t>(r) * n + col;
    if constexpr (sizeof(VT) == 4) {
      if (accumulate) {
#pragma unroll
        for (int i = 0; i < VD; ++i) atomicAdd(reinterpret_cast<float*>(dst) + i, res[i]);
        continue;
      }
    }
    store_out<VT, VD>(dst, res);
  }
}

template <typename VT, typename IT, int LPR, int NVEC, bool VS, bool VDN>
int launch(int m, int k, int n, int nnz, const int* row_indices, const VT* values,
           long long vstride, const int* row_offsets, const IT* cols, const VT* dense,
           const float* bias, VT* out, int batch, int accumulate, cudaStream_t stream) {
  constexpr int VD = VDN ? Elem<VT>::kPerVec : 1;
  constexpr int kTileCols = LPR * VD * NVEC;
  constexpr int kRowsPerBlock = 4 * (32 / LPR);
  const unsigned gy = (n + kTileCols - 1) / kTileCols;
  if (gy > 65535u) return IEX_ERR_UNSUPPORTED;
  dim3 grid((m + kRowsPerBlock - 1) / kRowsPerBlock, gy, batch);
  return launch_overlapped(spmm_rowgroup_kernel<VT, IT, LPR, NVEC, VS, VDN>, grid, dim3(128), 0, stream, m, k, n, nnz,
                           row_indices, values, vstride, row_offsets, cols, dense, bias, out, accumulate);
}

template <typename VT, typename IT, bool VS>
int dispatch_dense(int m, int k, int n, int nnz, const int* ri, const VT* values,
                   long long vstride, const int* ro, const IT* cols, const VT* dense,
                   const float* bias, VT* out, int batch, int accumulate,
                   cudaStream_t stream) {
  constexpr int VD = Elem<VT>::kPerVec;
  const bool vdn = (n % VD == 0) && aligned16(dense) && aligned16(out);
#define IEX_GO(LPR, NVEC, VDN)                                                          \
  return launch<VT, IT, LPR, NVEC, VS, VDN>(m, k, n, nnz, ri, values, vstride, ro, cols, \
                                            dense, bias, out, batch, accumulate, stream)
  if (!vdn) { IEX_GO(32, 1, false); }
  // Column tile = LPR * VD * NVEC.  Narrow n: fewer lanes per row so a warp carries
  // several rows; wide n: two vectors per lane so each shuffled nonzero feeds more FMAs.
  if (n <= 8 * VD) { IEX_GO(8, 1, true); }
  if (n <= 16 * VD) { IEX_GO(16, 1, true); }
  if (n <= 32 * VD) { IEX_GO(32, 1, true); }
  IEX_GO(32, 2, true);
#undef IEX_GO
}

template <typename VT, typename IT>
int spmm_entry(int m, int k, int n, int nnz, const int* ri, const VT* values,
               long long vstride, const int* ro, const IT* cols, const VT* dense,
               const float* bias, VT* out, int batch, int accumulate, void* stream) {
  if (m < 0 || k < 0 || n < 0 || nnz < 0 || batch < 0 || batch > 65535) return IEX_ERR_BAD_ARG;
  if (m == 0 || n == 0 || batch == 0) return IEX_OK;
  if (!ri || !ro || !out || (nnz > 0 && (!values || !cols || !dense))) return IEX_ERR_BAD_ARG;
  if (vstride != 0 && vstride < nnz) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 128-bit loads of the sparse arrays need 16-byte aligned bases for every batch item.
  const bool vs = aligned16(values) && aligned16(cols) &&
                  (vstride * static_cast<long long>(sizeof(VT))) % 16 == 0;
  if (vs)
    return dispatch_dense<VT, IT, true>(m, k, n, nnz, ri, values, vstride, ro, cols, dense,
                                        bias, out, batch, accumulate, s);
  return dispatch_dense<VT, IT, false>(m, k, n, nnz, ri, values, vstride, ro, cols, dense,
                                       bias, out, batch, accumulate, s);
}

}  // namespace
}  // namespace iex

extern "C" int iex_spmm_f32(int m, int k, int n, int nnz, const int32_t* row_indices,
                            const float* values, long long values_batch_stride,
                            const int32_t* row_offsets, const int32_t* column_indices,
                            const float* dense, const float* bias, float* out, int batch,
                            int accumulate, void* stream) {
  return iex::spmm_entry<float, int>(m, k, n, nnz, row_indices, values, values_batch_stride,
                                     row_offsets, column_indices, dense, bias, out, batch,
                                     accumulate, stream);
}

extern "C" int iex_spmm_f16_i16(int m, int k, int n, int nnz, const int32_t* row_indices,
                                const void* values, const int32_t* row_offsets,
                                const uint16_t* column_indices, const void* dense,
                                const float* bias, void* out, int batch, void* stream) {
  if (k > 65536) return IEX_ERR_UNSUPPORTED;
  return iex::spmm_entry<__half, uint16_t>(
      m, k, n, nnz, row_indices, static_cast<const __half*>(values), 0, row_offsets,
      column_indices, static_cast<const __half*>(dense), bias, static_cast<__half*>(out),
      batch, 0, stream);
}

extern "C" int iex_spmm_f16_i32(int m, int k, int n, int nnz, const int32_t* row_indices,
                                const void* values, const int32_t* row_offsets,
                                const int32_t* column_indices, const void* dense,
                                const float* bias, void* out, int batch, void* stream) {
  return iex::spmm_entry<__half, int>(
      m, k, n, nnz, row_indices, static_cast<const __half*>(values), 0, row_offsets,
      column_indices, static_cast<const __half*>(dense), bias, static_cast<__half*>(out),
      batch, 0, stream);
}

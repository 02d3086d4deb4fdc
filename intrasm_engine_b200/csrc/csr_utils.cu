// CSR <-> dense helpers on the device (fp16), used where an activation CSR becomes the
// tile operand of the tensor-core linear (ReLU-sparse FFN down projection).
#include "common.cuh"

namespace iex {
namespace {

// One CTA per row: clear the dense row with 128-bit stores, then scatter the row's nonzeros.
template <typename IT>
__global__ void __launch_bounds__(256)
csr_to_dense_f16_kernel(int m, int k, const int* __restrict__ row_offsets, const IT* __restrict__ cols,
                        const __half* __restrict__ values, __half* __restrict__ out) {
  for (int r = blockIdx.x; r < m; r += gridDim.x) {
    __half* row = out + static_cast<size_t>(r) * k;
    if ((k & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
      uint4* row4 = reinterpret_cast<uint4*>(row);
      for (int i = threadIdx.x; i < (k >> 3); i += blockDim.x) row4[i] = make_uint4(0u, 0u, 0u, 0u);
    } else {
      for (int i = threadIdx.x; i < k; i += blockDim.x) row[i] = __float2half(0.f);
    }
    __syncthreads();
    const int beg = __ldg(row_offsets + r), end = __ldg(row_offsets + r + 1);
    for (int p = beg + threadIdx.x; p < end; p += blockDim.x) {
      const int c = to_index(__ldg(cols + p));
      if (c < k) row[c] = __ldg(values + p);
    }
    __syncthreads();
  }
}

}  // namespace
}  // namespace iex

extern "C" int iex_csr_to_dense_f16(int m, int k, const int32_t* row_offsets, const void* column_indices,
                                    int index_bits, const void* values, void* out, void* stream) {
  using namespace iex;
  if (m < 0 || k < 0 || (index_bits != 16 && index_bits != 32)) return IEX_ERR_BAD_ARG;
  if (m == 0 || k == 0) return IEX_OK;
  if (!row_offsets || !out) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = m < 4 * kNumSMs ? m : 4 * kNumSMs;
  if (index_bits == 16)
    csr_to_dense_f16_kernel<uint16_t><<<grid, 256, 0, s>>>(m, k, row_offsets,
                                                          static_cast<const uint16_t*>(column_indices),
                                                          static_cast<const __half*>(values),
                                                          static_cast<__half*>(out));
  else
    csr_to_dense_f16_kernel<int><<<grid, 256, 0, s>>>(m, k, row_offsets, static_cast<const int*>(column_indices),
                                                      static_cast<const __half*>(values),
                                                      static_cast<__half*>(out));
  return launch_status();
}

/*
 * CPU oracle for the CSR SpMM / SDDMM / dense-linear hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the GPU kernels are compared
 * against; nothing in the shipped library links or calls it.
 *
 * PARITY STATUS: "parity unpinned" by the reference's own tests — the reference holds no
 * golden vector, known-answer test or fixture that evaluates SpMM or SDDMM
 * (tests/test_torch_load_library.py:15-19 only looks the ops up), and its device code
 * lives in an un-vendored submodule (.gitmodules:4-6, K-Wu/sputnik_experimental, no
 * pinned SHA), so it cannot be compiled.  The restatement below follows the arithmetic
 * that the reference's driver code states, and is pinned instead against fixtures made
 * with torch.sparse.mm / torch.sparse.sampled_addmm / torch.matmul on CPU (the path the
 * task names as the reference CPU path); see tests/golden/make_golden.py.
 *
 * Every function accumulates in fp32 with one fused multiply-add per term, in the order
 * in which the reference's thread that owns the output element visits the terms, so the
 * SpMM result is reproducible bit for bit by any implementation that keeps that order.
 * The *_f64 variants accumulate in double and are the ground truth for tolerance checks.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

/*
 * SpMM: out[z, r, :] = sum_{p in row r} values[p] * dense[z, col[p], :]  (+bias[r], ReLU)
 *
 * Follows intrasm_engine/pytorch/csrc/extensions/sputnik_spmm.cu.inc:101-294:
 *   - rows are visited through the swizzle map row_indices (:114); every row of
 *     row_indices is computed exactly once, rows absent from it are left untouched;
 *   - the row's extent comes from row_offsets[r], row_offsets[r+1] (:127-128);
 *   - accumulators are fp32 and start at zero (:187); terms are added in storage order;
 *   - optional bias[r] then ReLU (:273-282);
 *   - values are shared by all batch items (values_batch_stride == 0, the
 *     "reuse_weight" stamp, :160-164) or per batch item (stride == nnz, the "atomic"
 *     stamp);  dense and out advance by k*n and m*n per batch item (:176-181, :285).
 * accumulate != 0 adds the result onto out (the atomic-store stamp, :287-290) instead of
 * overwriting it.
 */
void iex_oracle_spmm_f32(int m, int k, int n, int nnz, int batch,
                         const int32_t* row_indices, const float* values,
                         long values_batch_stride, const int32_t* row_offsets,
                         const int32_t* column_indices, const float* dense,
                         const float* bias, float* out, int accumulate) {
  (void)nnz;
  for (int z = 0; z < batch; ++z) {
    const float* vals = values + (size_t)z * (size_t)values_batch_stride;
    const float* b = dense + (size_t)z * (size_t)k * (size_t)n;
    float* o = out + (size_t)z * (size_t)m * (size_t)n;
    for (int i = 0; i < m; ++i) {
      const int r = row_indices[i];
      const int beg = row_offsets[r], end = row_offsets[r + 1];
      for (int c = 0; c < n; ++c) {
        float acc = 0.0f;
        for (int p = beg; p < end; ++p)
          acc = fmaf(vals[p], b[(size_t)column_indices[p] * (size_t)n + c], acc);
        if (bias) {
          acc += bias[r];
          acc = acc > 0.0f ? acc : 0.0f;
        }
        if (accumulate)
          o[(size_t)r * n + c] += acc;
        else
          o[(size_t)r * n + c] = acc;
      }
    }
  }
}

/* Same sum in double; no bias, no accumulate.  Ground truth for tolerance checks. */
void iex_oracle_spmm_f64(int m, int k, int n, int batch, const int32_t* row_indices,
                         const float* values, long values_batch_stride,
                         const int32_t* row_offsets, const int32_t* column_indices,
                         const float* dense, double* out) {
  for (int z = 0; z < batch; ++z) {
    const float* vals = values + (size_t)z * (size_t)values_batch_stride;
    const float* b = dense + (size_t)z * (size_t)k * (size_t)n;
    double* o = out + (size_t)z * (size_t)m * (size_t)n;
    for (int i = 0; i < m; ++i) {
      const int r = row_indices[i];
      const int beg = row_offsets[r], end = row_offsets[r + 1];
      for (int c = 0; c < n; ++c) {
        double acc = 0.0;
        for (int p = beg; p < end; ++p)
          acc += (double)vals[p] * (double)b[(size_t)column_indices[p] * (size_t)n + c];
        o[(size_t)r * n + c] = acc;
      }
    }
  }
}

/*
 * SDDMM: out[p] (+)= sum_z sum_t lhs[z, row(p), t] * rhs[z, col[p], t]
 *
 * Follows intrasm_engine/pytorch/csrc/extensions/sputnik_sddmm.cu.inc:62-181: one output
 * per stored position p, written at row_offsets[row] + position, i.e. aligned with
 * column_indices (:122-130); the batch items all add into the same [nnz] vector (the
 * "atomic_upd_weight" stamp, :177-178).  accumulate == 0 starts from zero; the reference
 * op adds onto whatever its freshly allocated output holds
 * (sputnik_kernels.cpp:21-24), which is only meaningful when that is zero.
 */
void iex_oracle_sddmm_f32(int m, int k, int n, int nnz, int batch,
                          const int32_t* row_indices, const int32_t* row_offsets,
                          const int32_t* column_indices, const float* lhs,
                          const float* rhs, float* out, int accumulate) {
  (void)nnz;
  for (int i = 0; i < m; ++i) {
    const int r = row_indices[i];
    for (int p = row_offsets[r]; p < row_offsets[r + 1]; ++p) {
      float total = accumulate ? out[p] : 0.0f;
      for (int z = 0; z < batch; ++z) {
        const float* a = lhs + ((size_t)z * m + r) * (size_t)k;
        const float* b = rhs + ((size_t)z * n + column_indices[p]) * (size_t)k;
        float acc = 0.0f;
        for (int t = 0; t < k; ++t) acc = fmaf(a[t], b[t], acc);
        total += acc;
      }
      out[p] = total;
    }
  }
}

void iex_oracle_sddmm_f64(int m, int k, int n, int batch, const int32_t* row_indices,
                          const int32_t* row_offsets, const int32_t* column_indices,
                          const float* lhs, const float* rhs, double* out) {
  for (int i = 0; i < m; ++i) {
    const int r = row_indices[i];
    for (int p = row_offsets[r]; p < row_offsets[r + 1]; ++p) {
      double total = 0.0;
      for (int z = 0; z < batch; ++z) {
        const float* a = lhs + ((size_t)z * m + r) * (size_t)k;
        const float* b = rhs + ((size_t)z * n + column_indices[p]) * (size_t)k;
        for (int t = 0; t < k; ++t) total += (double)a[t] * (double)b[t];
      }
      out[p] = total;
    }
  }
}

/*
 * Dense branch: out[t, f] = sum_c input[t, c] * weight[f, c]   (input @ weight^T)
 * Follows intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/torch.py:17.
 * fp32 accumulate, sequential in c.
 */
void iex_oracle_linear_f32(int tokens, int in_features, int out_features,
                           const float* input, const float* weight, float* out) {
  for (int t = 0; t < tokens; ++t)
    for (int f = 0; f < out_features; ++f) {
      const float* x = input + (size_t)t * in_features;
      const float* w = weight + (size_t)f * in_features;
      float acc = 0.0f;
      for (int c = 0; c < in_features; ++c) acc = fmaf(x[c], w[c], acc);
      out[(size_t)t * out_features + f] = acc;
    }
}

/*
 * CSR validator: the invariants every launcher assumes (monotone offsets that start at
 * 0 and end at nnz, in-range columns, row_indices a permutation of [0, m)).
 * Returns 0 when valid, else a small positive code naming the first broken rule.
 */
int iex_oracle_validate_csr(int m, int k, int nnz, const int32_t* row_indices,
                            const int32_t* row_offsets, const int32_t* column_indices,
                            uint8_t* seen /* m bytes of scratch */) {
  if (row_offsets[0] != 0) return 1;
  if (row_offsets[m] != nnz) return 2;
  for (int r = 0; r < m; ++r)
    if (row_offsets[r + 1] < row_offsets[r]) return 3;
  for (int p = 0; p < nnz; ++p)
    if (column_indices[p] < 0 || column_indices[p] >= k) return 4;
  for (int r = 0; r < m; ++r) seen[r] = 0;
  for (int i = 0; i < m; ++i) {
    const int r = row_indices[i];
    if (r < 0 || r >= m || seen[r]) return 5;
    seen[r] = 1;
  }
  return 0;
}

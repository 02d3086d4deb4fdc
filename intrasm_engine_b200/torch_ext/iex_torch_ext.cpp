// torch.ops.iex_ops.* — the reference's operator boundary as a compiled torch extension.
//
// Schemas, argument checks, output shapes and stream choice follow
// intrasm_engine/pytorch/csrc/extensions/sputnik_kernels.cpp:32-193; every operator then calls
// the C ABI of libiex_b200.so (include/iex_b200.h) with raw pointers.  Outputs come from the
// torch caching allocator and kernels are enqueued on the current torch stream with no
// synchronisation, so every operator can be recorded by a stream capture, as the
// reference's callers do (layers_and_funcs/sputnik.py:59-66).
//
// Deliberate differences from the reference, all supersets:
//   * spmm_sputnik_reuse_weight_half is registered (the reference defines it at
//     sputnik_kernels.cpp:179-181 but leaves it out of its TORCH_LIBRARY block, :189-193); it
//     takes int16 or int32 column indices.
//   * The atomic variant zeroes its output before accumulating; the reference accumulates
//     onto an uninitialised at::empty tensor (sputnik_kernels.cpp:91).
//   * linear_fp16, spmm_tc_half, fused_spmm_linear_half and csr_to_dense_half are new
//     operators (dense branch, tensor-core SpMM, fused sparse||dense layer, CSR expansion);
//     the reference has no kernel of its own for them.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <algorithm>
#include <cstdlib>
#include <tuple>

#include "iex_b200.h"

namespace {

void* stream_of(const at::Tensor& t) {
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

void check_status(int st, const char* what) {
  TORCH_CHECK(st == 0, what, " failed with status ", st, ": ", iex_error_string(st));
}

void check_common(std::initializer_list<std::pair<const char*, const at::Tensor*>> named) {
  const at::Tensor* first = nullptr;
  for (const auto& [name, t] : named) {
    TORCH_CHECK(t->is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t->is_contiguous(), name, " must be a contiguous tensor");
    TORCH_CHECK(!t->is_sparse(), name, " must be a dense tensor");
    if (first == nullptr) first = t;
    TORCH_CHECK(t->device() == first->device(), name, " should be in the same device as the first argument");
  }
}

// CSR validation on the device (iex_csr_validate): returns 0 or the OR of IEX_CSR_* bits.
// Synchronises the stream, so it must not run during stream capture.
int64_t validate_csr_impl(const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m,
                          int64_t k, const at::Tensor* row_indices, bool require_ascending) {
  c10::cuda::CUDAGuard guard(row_offsets.device());
  const bool i16 = column_indices.scalar_type() == at::kShort;
  TORCH_CHECK(i16 || column_indices.scalar_type() == at::kInt, "column_indices must be int16 or int32");
  TORCH_CHECK(row_offsets.scalar_type() == at::kInt && row_offsets.numel() == m + 1,
              "row_offsets must be int32 with m + 1 entries");
  at::Tensor result = at::empty({1}, row_offsets.options());
  check_status(iex_csr_validate(m, k, column_indices.numel(), row_offsets.data_ptr<int>(),
                                column_indices.data_ptr(), i16 ? 16 : 32,
                                row_indices != nullptr ? row_indices->data_ptr<int>() : nullptr,
                                require_ascending ? 1 : 0, result.data_ptr<int>(), stream_of(row_offsets)),
               "iex_csr_validate");
  return result.item<int>();
}

// With IEX_VALIDATE_CSR=1 in the environment every sparse operator checks its CSR arguments
// on the device before launching (one extra kernel and a stream synchronisation per call: a
// debugging aid, off by default and skipped while the stream is being captured).
bool validation_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("IEX_VALIDATE_CSR");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return on;
}

void maybe_validate(const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m, int64_t k,
                    const at::Tensor* row_indices, bool require_ascending) {
  if (!validation_enabled()) return;
  if (iex_stream_is_capturing(stream_of(row_offsets))) return;
  const int64_t code = validate_csr_impl(row_offsets, column_indices, m, k, row_indices, require_ascending);
  TORCH_CHECK(code == 0, "malformed CSR argument (IEX_CSR_* bits ", code,
              "): 1 first offset, 2 last offset, 4 offsets not monotone, 8 column out of range, "
              "16 columns not ascending, 32 row index out of range");
}

void check_spmm(const at::Tensor& b, const at::Tensor& row_indices, const at::Tensor& values,
                const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m,
                bool per_batch_values) {
  TORCH_CHECK(b.dim() == 3, "b must be [batch, k, n]");
  if (per_batch_values) {
    TORCH_CHECK(values.dim() == 2, "values must be [batch, nnz]");
    TORCH_CHECK(b.size(0) == values.size(0), "values and b disagree on the batch size");
    TORCH_CHECK(values.size(1) == column_indices.size(0), "values and column_indices disagree on nnz");
  } else {
    TORCH_CHECK(values.dim() == 1, "values must be [nnz]");
    TORCH_CHECK(values.size(0) == column_indices.size(0), "values and column_indices disagree on nnz");
  }
  TORCH_CHECK(row_indices.dim() == 1 && row_offsets.dim() == 1 && column_indices.dim() == 1,
              "row_indices, row_offsets and column_indices must be 1-D");
  check_common({{"b", &b}, {"row_indices", &row_indices}, {"values", &values},
                {"row_offsets", &row_offsets}, {"column_indices", &column_indices}});
  TORCH_CHECK(row_indices.scalar_type() == at::kInt && row_offsets.scalar_type() == at::kInt,
              "row_indices and row_offsets must be int32");
  TORCH_CHECK(row_indices.size(0) == m && row_offsets.size(0) == m + 1,
              "row_indices must have m entries and row_offsets m + 1");
  TORCH_CHECK(b.size(0) == 1 || column_indices.size(0) % 4 == 0,
              "If batch size > 1 then number of nonzeros should be a multiple of 4");
}

at::Tensor spmm_f32(const at::Tensor& b, const at::Tensor& row_indices, const at::Tensor& values,
                    const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m,
                    bool per_batch_values) {
  check_spmm(b, row_indices, values, row_offsets, column_indices, m, per_batch_values);
  TORCH_CHECK(b.scalar_type() == at::kFloat && values.scalar_type() == at::kFloat,
              "b and values must be float32");
  TORCH_CHECK(column_indices.scalar_type() == at::kInt, "column_indices must be int32");
  c10::cuda::CUDAGuard guard(b.device());
  const int batch = b.size(0), k = b.size(1), n = b.size(2), nnz = column_indices.size(0);
  maybe_validate(row_offsets, column_indices, m, k, &row_indices, false);
  at::Tensor out = per_batch_values ? at::zeros({batch, m, n}, b.options()) : at::empty({batch, m, n}, b.options());
  check_status(iex_spmm_f32(m, k, n, nnz, row_indices.data_ptr<int>(), values.data_ptr<float>(),
                            per_batch_values ? nnz : 0, row_offsets.data_ptr<int>(),
                            column_indices.data_ptr<int>(), b.data_ptr<float>(), nullptr,
                            out.data_ptr<float>(), batch, per_batch_values ? 1 : 0, stream_of(b)),
               "iex_spmm_f32");
  return out;
}

// fp32, one values vector shared by the batch (sputnik_kernels.cpp:173-175)
at::Tensor spmm_sputnik_reuse_weight(const at::Tensor& b, const at::Tensor& row_indices,
                                     const at::Tensor& values, const at::Tensor& row_offsets,
                                     const at::Tensor& column_indices, int64_t m) {
  return spmm_f32(b, row_indices, values, row_offsets, column_indices, m, false);
}

// fp32, per-batch values, atomic accumulate (sputnik_kernels.cpp:170-172)
at::Tensor spmm_sputnik_atomic(const at::Tensor& b, const at::Tensor& row_indices,
                               const at::Tensor& values, const at::Tensor& row_offsets,
                               const at::Tensor& column_indices, int64_t m) {
  return spmm_f32(b, row_indices, values, row_offsets, column_indices, m, true);
}

// fp16 storage, fp32 accumulate, int16 or int32 column indices (sputnik_kernels.cpp:179-181)
at::Tensor spmm_sputnik_reuse_weight_half(const at::Tensor& b, const at::Tensor& row_indices,
                                          const at::Tensor& values, const at::Tensor& row_offsets,
                                          const at::Tensor& column_indices, int64_t m) {
  check_spmm(b, row_indices, values, row_offsets, column_indices, m, false);
  TORCH_CHECK(b.scalar_type() == at::kHalf && values.scalar_type() == at::kHalf,
              "b and values must be float16");
  const bool i16 = column_indices.scalar_type() == at::kShort;
  TORCH_CHECK(i16 || column_indices.scalar_type() == at::kInt, "column_indices must be int16 or int32");
  c10::cuda::CUDAGuard guard(b.device());
  const int batch = b.size(0), k = b.size(1), n = b.size(2), nnz = column_indices.size(0);
  maybe_validate(row_offsets, column_indices, m, k, &row_indices, false);
  at::Tensor out = at::empty({batch, m, n}, b.options());
  const int st = i16 ? iex_spmm_f16_i16(m, k, n, nnz, row_indices.data_ptr<int>(), values.data_ptr(),
                                        row_offsets.data_ptr<int>(),
                                        reinterpret_cast<const uint16_t*>(column_indices.data_ptr()),
                                        b.data_ptr(), nullptr, out.data_ptr(), batch, stream_of(b))
                     : iex_spmm_f16_i32(m, k, n, nnz, row_indices.data_ptr<int>(), values.data_ptr(),
                                        row_offsets.data_ptr<int>(), column_indices.data_ptr<int>(),
                                        b.data_ptr(), nullptr, out.data_ptr(), batch, stream_of(b));
  check_status(st, "iex_spmm_f16");
  return out;
}

// fp32 SDDMM, batch items summed into one [nnz] vector (sputnik_kernels.cpp:182-184)
at::Tensor sddmm_sputnik_atomic_upd_weight(const at::Tensor& a, const at::Tensor& b,
                                           const at::Tensor& row_indices, const at::Tensor& row_offsets,
                                           const at::Tensor& column_indices) {
  TORCH_CHECK(a.dim() == b.dim() && a.dim() == 3, "a and b must be [batch, rows, k]");
  TORCH_CHECK(a.size(0) == b.size(0), "a and b disagree on the batch size");
  TORCH_CHECK(a.size(2) == b.size(2), "a and b disagree on k");
  TORCH_CHECK(row_indices.dim() == 1 && row_offsets.dim() == 1 && column_indices.dim() == 1,
              "row_indices, row_offsets and column_indices must be 1-D");
  check_common({{"a", &a}, {"b", &b}, {"row_indices", &row_indices}, {"row_offsets", &row_offsets},
                {"column_indices", &column_indices}});
  TORCH_CHECK(a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat, "a and b must be float32");
  TORCH_CHECK(row_indices.scalar_type() == at::kInt && row_offsets.scalar_type() == at::kInt &&
                  column_indices.scalar_type() == at::kInt,
              "index tensors must be int32");
  const int batch = a.size(0), m = a.size(1), k = a.size(2), n = b.size(1);
  TORCH_CHECK(row_indices.size(0) == m && row_offsets.size(0) == m + 1,
              "row_indices must have m entries and row_offsets m + 1");
  const int nnz = column_indices.size(0);
  c10::cuda::CUDAGuard guard(a.device());
  maybe_validate(row_offsets, column_indices, m, n, &row_indices, false);
  at::Tensor out = at::empty({nnz}, a.options());
  check_status(iex_sddmm_f32(m, k, n, nnz, row_indices.data_ptr<int>(), row_offsets.data_ptr<int>(),
                             column_indices.data_ptr<int>(), a.data_ptr<float>(), b.data_ptr<float>(),
                             out.data_ptr<float>(), batch, 0, stream_of(a)),
               "iex_sddmm_f32");
  return out;
}

// fp16 SDDMM (the instantiation the reference leaves commented out, sputnik_kernels.cpp:185-187):
// a [batch, m, k] and b [batch, n, k] fp16 -> fp16 [nnz]; int16 or int32 column indices
at::Tensor sddmm_sputnik_half(const at::Tensor& a, const at::Tensor& b, const at::Tensor& row_indices,
                              const at::Tensor& row_offsets, const at::Tensor& column_indices) {
  TORCH_CHECK(a.dim() == b.dim() && a.dim() == 3, "a and b must be [batch, rows, k]");
  TORCH_CHECK(a.size(0) == b.size(0) && a.size(2) == b.size(2), "a and b disagree on batch size or k");
  check_common({{"a", &a}, {"b", &b}, {"row_indices", &row_indices}, {"row_offsets", &row_offsets},
                {"column_indices", &column_indices}});
  TORCH_CHECK(a.scalar_type() == at::kHalf && b.scalar_type() == at::kHalf, "a and b must be float16");
  TORCH_CHECK(row_indices.scalar_type() == at::kInt && row_offsets.scalar_type() == at::kInt,
              "row_indices and row_offsets must be int32");
  const bool i16 = column_indices.scalar_type() == at::kShort;
  TORCH_CHECK(i16 || column_indices.scalar_type() == at::kInt, "column_indices must be int16 or int32");
  const int batch = a.size(0), m = a.size(1), k = a.size(2), n = b.size(1);
  TORCH_CHECK(row_indices.size(0) == m && row_offsets.size(0) == m + 1,
              "row_indices must have m entries and row_offsets m + 1");
  const int nnz = column_indices.size(0);
  c10::cuda::CUDAGuard guard(a.device());
  maybe_validate(row_offsets, column_indices, m, n, &row_indices, false);
  at::Tensor out = at::empty({nnz}, a.options());
  check_status(iex_sddmm_f16(m, k, n, nnz, row_indices.data_ptr<int>(), row_offsets.data_ptr<int>(),
                             column_indices.data_ptr(), i16 ? 16 : 32, a.data_ptr(), b.data_ptr(),
                             out.data_ptr(), batch, stream_of(a)),
               "iex_sddmm_f16");
  return out;
}

// One block of at most 256 tokens (a multiple of 16) of the dense branch into `out` (a
// contiguous [tokens, out_features] block).
void linear_block(const at::Tensor& input, const at::Tensor& weight, at::Tensor out) {
  const int64_t tokens = input.size(0), out_features = weight.size(0);
  // A weight with few 128-row tiles would leave most SMs without work: split every tile's K
  // range over about 128 / tiles CTAs (measured optimum on B200: 32 tiles -> 4 parts,
  // 4 tiles -> 16).  The partial tiles live in a scratch tensor of the caching allocator.
  const int64_t tiles = (out_features + 127) / 128;
  const int parts = tiles > 0 ? static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(16, 128 / tiles))) : 1;
  if (parts > 1 && tokens % 32 == 0 && input.size(1) >= 128 * parts) {
    const size_t need = iex_tc_workspace_bytes(0, 1, static_cast<int>(out_features), parts,
                                               static_cast<int>(tokens));
    at::Tensor scratch = at::empty({static_cast<int64_t>(need)}, input.options().dtype(at::kByte));
    check_status(iex_linear_f16_splitk(tokens, input.size(1), out_features, input.data_ptr(),
                                       weight.data_ptr(), out.data_ptr(), parts, scratch.data_ptr(), need,
                                       stream_of(input)),
                 "iex_linear_f16_splitk");
    return;
  }
  check_status(iex_linear_f16(tokens, input.size(1), out_features, input.data_ptr(), weight.data_ptr(),
                              out.data_ptr(), stream_of(input)),
               "iex_linear_f16");
}

// Dense branch on tensor cores: input @ weight^T (layers_and_funcs/torch.py:17).  Any number
// of tokens: the kernel takes up to 256 at a time (a multiple of 16), so longer inputs run
// block after block into the rows of one output, and a ragged tail is padded with zero rows.
at::Tensor linear_fp16(const at::Tensor& input, const at::Tensor& weight) {
  TORCH_CHECK(input.dim() == 2 && weight.dim() == 2, "input and weight must be 2-D");
  TORCH_CHECK(input.size(1) == weight.size(1), "input and weight disagree on in_features");
  check_common({{"input", &input}, {"weight", &weight}});
  TORCH_CHECK(input.scalar_type() == at::kHalf && weight.scalar_type() == at::kHalf,
              "input and weight must be float16");
  c10::cuda::CUDAGuard guard(input.device());
  const int64_t tokens = input.size(0), out_features = weight.size(0), in_features = input.size(1);
  at::Tensor out = at::empty({tokens, out_features}, input.options());
  if (tokens == 0 || out_features == 0) return out;
  const int64_t whole = tokens / 16 * 16;
  for (int64_t t0 = 0; t0 < whole; t0 += 256) {
    const int64_t block = std::min<int64_t>(256, whole - t0);
    linear_block(input.narrow(0, t0, block), weight, out.narrow(0, t0, block));
  }
  if (whole < tokens) {  // ragged tail: 16 rows, the missing ones zero
    at::Tensor tail_in = at::zeros({16, in_features}, input.options());
    tail_in.narrow(0, 0, tokens - whole).copy_(input.narrow(0, whole, tokens - whole));
    at::Tensor tail_out = at::empty({16, out_features}, input.options());
    linear_block(tail_in, weight, tail_out);
    out.narrow(0, whole, tokens - whole).copy_(tail_out.narrow(0, 0, tokens - whole));
  }
  return out;
}

// dinput = grad @ weight (blocks of up to 256 tokens, a ragged tail padded with zero rows)
at::Tensor linear_fp16_dgrad(const at::Tensor& grad, const at::Tensor& weight) {
  TORCH_CHECK(grad.dim() == 2 && weight.dim() == 2 && grad.size(1) == weight.size(0),
              "grad must be [tokens, out_features] and weight [out_features, in_features]");
  check_common({{"grad", &grad}, {"weight", &weight}});
  TORCH_CHECK(grad.scalar_type() == at::kHalf && weight.scalar_type() == at::kHalf, "grad and weight must be float16");
  c10::cuda::CUDAGuard guard(grad.device());
  const int64_t tokens = grad.size(0), out_features = weight.size(0), in_features = weight.size(1);
  at::Tensor dinput = at::empty({tokens, in_features}, grad.options());
  if (tokens == 0 || in_features == 0) return dinput;
  auto block = [&](const at::Tensor& g, at::Tensor d) {
    check_status(iex_linear_f16_dgrad(g.size(0), in_features, out_features, g.data_ptr(), weight.data_ptr(),
                                      d.data_ptr(), stream_of(grad)),
                 "iex_linear_f16_dgrad");
  };
  const int64_t whole = tokens / 16 * 16;
  for (int64_t t0 = 0; t0 < whole; t0 += 256) {
    const int64_t rows = std::min<int64_t>(256, whole - t0);
    block(grad.narrow(0, t0, rows), dinput.narrow(0, t0, rows));
  }
  if (whole < tokens) {
    at::Tensor tail_in = at::zeros({16, out_features}, grad.options());
    tail_in.narrow(0, 0, tokens - whole).copy_(grad.narrow(0, whole, tokens - whole));
    at::Tensor tail_out = at::empty({16, in_features}, grad.options());
    block(tail_in, tail_out);
    dinput.narrow(0, whole, tokens - whole).copy_(tail_out.narrow(0, 0, tokens - whole));
  }
  return dinput;
}

// dweight = grad^T @ input (the token dimension is the contraction; padded to a multiple of 8)
at::Tensor linear_fp16_wgrad(const at::Tensor& grad, const at::Tensor& input) {
  TORCH_CHECK(grad.dim() == 2 && input.dim() == 2 && grad.size(0) == input.size(0),
              "grad must be [tokens, out_features] and input [tokens, in_features]");
  check_common({{"grad", &grad}, {"input", &input}});
  TORCH_CHECK(grad.scalar_type() == at::kHalf && input.scalar_type() == at::kHalf, "grad and input must be float16");
  c10::cuda::CUDAGuard guard(grad.device());
  const int64_t tokens = grad.size(0), out_features = grad.size(1), in_features = input.size(1);
  at::Tensor dweight = at::empty({out_features, in_features}, grad.options());
  if (out_features == 0 || in_features == 0) return dweight;
  at::Tensor g = grad, x = input;
  if (tokens % 8 != 0 || tokens == 0) {
    const int64_t padded = std::max<int64_t>(8, (tokens + 7) / 8 * 8);
    g = at::zeros({padded, out_features}, grad.options());
    x = at::zeros({padded, in_features}, input.options());
    if (tokens > 0) {
      g.narrow(0, 0, tokens).copy_(grad);
      x.narrow(0, 0, tokens).copy_(input);
    }
  }
  check_status(iex_linear_f16_wgrad(g.size(0), in_features, out_features, g.data_ptr(), x.data_ptr(),
                                    dweight.data_ptr(), stream_of(grad)),
               "iex_linear_f16_wgrad");
  return dweight;
}

int tc_sparse_checks(const at::Tensor& x, const at::Tensor& row_offsets, const at::Tensor& values,
                     const at::Tensor& column_indices, int64_t m) {
  TORCH_CHECK(x.dim() == 2, "x must be [k, n]");
  TORCH_CHECK(values.dim() == 1 && values.size(0) == column_indices.size(0),
              "values and column_indices must be 1-D with nnz entries");
  TORCH_CHECK(row_offsets.dim() == 1 && row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries");
  check_common({{"x", &x}, {"row_offsets", &row_offsets}, {"values", &values},
                {"column_indices", &column_indices}});
  TORCH_CHECK(x.scalar_type() == at::kHalf && values.scalar_type() == at::kHalf,
              "x and values must be float16");
  TORCH_CHECK(row_offsets.scalar_type() == at::kInt, "row_offsets must be int32");
  const bool i16 = column_indices.scalar_type() == at::kShort;
  TORCH_CHECK(i16 || column_indices.scalar_type() == at::kInt, "column_indices must be int16 or int32");
  return i16 ? 16 : 32;
}

// CSR SpMM on tensor cores: A [m, k] in CSR (ascending columns per row) times x [k, n]
at::Tensor spmm_tc_half(const at::Tensor& x, const at::Tensor& row_offsets, const at::Tensor& values,
                        const at::Tensor& column_indices, int64_t m) {
  const int bits = tc_sparse_checks(x, row_offsets, values, column_indices, m);
  c10::cuda::CUDAGuard guard(x.device());
  maybe_validate(row_offsets, column_indices, m, x.size(0), nullptr, true);
  at::Tensor out = at::empty({m, x.size(1)}, x.options());
  check_status(iex_spmm_f16_tc(m, x.size(0), x.size(1), column_indices.size(0), row_offsets.data_ptr<int>(),
                               column_indices.data_ptr(), bits, values.data_ptr(), x.data_ptr(),
                               out.data_ptr(), stream_of(x)),
               "iex_spmm_f16_tc");
  return out;
}

// Fused sparse || dense layer in ONE launch: (A_csr @ x [m, n], (weight @ x)^T [n, out_features])
std::tuple<at::Tensor, at::Tensor> fused_spmm_linear_half(const at::Tensor& x, const at::Tensor& row_offsets,
                                                          const at::Tensor& values,
                                                          const at::Tensor& column_indices, int64_t m,
                                                          const at::Tensor& weight) {
  const int bits = tc_sparse_checks(x, row_offsets, values, column_indices, m);
  TORCH_CHECK(weight.dim() == 2 && weight.size(1) == x.size(0), "weight must be [out_features, k]");
  check_common({{"x", &x}, {"weight", &weight}});
  TORCH_CHECK(weight.scalar_type() == at::kHalf, "weight must be float16");
  c10::cuda::CUDAGuard guard(x.device());
  maybe_validate(row_offsets, column_indices, m, x.size(0), nullptr, true);
  const int64_t n = x.size(1), md = weight.size(0);
  at::Tensor out_s = at::empty({m, n}, x.options());
  at::Tensor out_d = at::empty({n, md}, x.options());
  check_status(iex_fused_spmm_linear_f16(m, md, x.size(0), n, column_indices.size(0),
                                         row_offsets.data_ptr<int>(), column_indices.data_ptr(), bits,
                                         values.data_ptr(), weight.data_ptr(), x.data_ptr(), out_s.data_ptr(),
                                         out_d.data_ptr(), 1, stream_of(x)),
               "iex_fused_spmm_linear_f16");
  return {out_s, out_d};
}

// Dense fp16 [m, k] copy of a CSR matrix
at::Tensor csr_to_dense_half(const at::Tensor& row_offsets, const at::Tensor& values,
                             const at::Tensor& column_indices, int64_t m, int64_t k) {
  check_common({{"row_offsets", &row_offsets}, {"values", &values}, {"column_indices", &column_indices}});
  TORCH_CHECK(values.scalar_type() == at::kHalf && row_offsets.scalar_type() == at::kInt, "dtype mismatch");
  TORCH_CHECK(row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries");
  const bool i16 = column_indices.scalar_type() == at::kShort;
  TORCH_CHECK(i16 || column_indices.scalar_type() == at::kInt, "column_indices must be int16 or int32");
  c10::cuda::CUDAGuard guard(values.device());
  at::Tensor out = at::empty({m, k}, values.options());
  check_status(iex_csr_to_dense_f16(m, k, row_offsets.data_ptr<int>(), column_indices.data_ptr(),
                                    i16 ? 16 : 32, values.data_ptr(), out.data_ptr(), stream_of(values)),
               "iex_csr_to_dense_f16");
  return out;
}

// Plan of a sparsity pattern for the tensor-core SDDMM (pattern-only, like row_indices:
// build once per pattern, reuse for every product on it).  Returns an opaque uint8 tensor.
at::Tensor sddmm_plan(const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m, int64_t n) {
  check_common({{"row_offsets", &row_offsets}, {"column_indices", &column_indices}});
  TORCH_CHECK(row_offsets.scalar_type() == at::kInt && column_indices.scalar_type() == at::kInt,
              "index tensors must be int32");
  TORCH_CHECK(row_offsets.dim() == 1 && row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries");
  c10::cuda::CUDAGuard guard(row_offsets.device());
  const int64_t nnz = column_indices.numel();
  const size_t bytes = iex_sddmm_plan_bytes(m, n, nnz);
  at::Tensor plan = at::empty({static_cast<int64_t>(std::max<size_t>(bytes, 16))},
                              row_offsets.options().dtype(at::kByte));
  check_status(iex_sddmm_plan_build(m, n, nnz, row_offsets.data_ptr<int>(), column_indices.data_ptr<int>(),
                                    plan.data_ptr(), bytes, stream_of(row_offsets)),
               "iex_sddmm_plan_build");
  return plan;
}

// SDDMM on tensor cores with a plan from sddmm_plan: a [m, k] and b [n, k] fp32 -> [nnz] in
// storage order (the result contract of sddmm_sputnik_atomic_upd_weight with batch 1)
at::Tensor sddmm_tc_planned(const at::Tensor& a, const at::Tensor& b, const at::Tensor& plan, int64_t nnz) {
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "a must be [m, k] and b [n, k]");
  check_common({{"a", &a}, {"b", &b}, {"plan", &plan}});
  TORCH_CHECK(a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat, "a and b must be float32");
  TORCH_CHECK(plan.scalar_type() == at::kByte, "plan must come from sddmm_plan");
  const int64_t m = a.size(0), k = a.size(1), n = b.size(0);
  TORCH_CHECK(static_cast<size_t>(plan.numel()) >= iex_sddmm_plan_bytes(m, n, nnz),
              "plan was built for another pattern size");
  c10::cuda::CUDAGuard guard(a.device());
  at::Tensor out = at::empty({nnz}, a.options());
  check_status(iex_sddmm_f32_tc(m, k, n, nnz, plan.data_ptr(), a.data_ptr<float>(), b.data_ptr<float>(),
                                out.data_ptr<float>(), 0, stream_of(a)),
               "iex_sddmm_f32_tc");
  return out;
}

// Tile plan of a pattern with 64-column tiles, for spmm_tc_planned (k = A's column count).
at::Tensor spmm_plan(const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m, int64_t k) {
  check_common({{"row_offsets", &row_offsets}, {"column_indices", &column_indices}});
  TORCH_CHECK(row_offsets.scalar_type() == at::kInt && column_indices.scalar_type() == at::kInt,
              "index tensors must be int32");
  TORCH_CHECK(row_offsets.dim() == 1 && row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries");
  c10::cuda::CUDAGuard guard(row_offsets.device());
  const int64_t nnz = column_indices.numel();
  const size_t bytes = iex_tile_plan_bytes(m, k, nnz, 64);
  at::Tensor plan = at::empty({static_cast<int64_t>(std::max<size_t>(bytes, 16))},
                              row_offsets.options().dtype(at::kByte));
  check_status(iex_tile_plan_build(m, k, nnz, 64, row_offsets.data_ptr<int>(), column_indices.data_ptr<int>(),
                                   plan.data_ptr(), bytes, stream_of(row_offsets)),
               "iex_tile_plan_build");
  return plan;
}

// CSR SpMM on tensor cores with a plan from spmm_plan: A [m, k] (values in storage order) times
// b [k, n] fp32 -> [m, n]
at::Tensor spmm_tc_planned(const at::Tensor& b, const at::Tensor& values, const at::Tensor& plan, int64_t m) {
  TORCH_CHECK(b.dim() == 2 && values.dim() == 1, "b must be [k, n] and values [nnz]");
  check_common({{"b", &b}, {"values", &values}, {"plan", &plan}});
  TORCH_CHECK(b.scalar_type() == at::kFloat && values.scalar_type() == at::kFloat, "b and values must be float32");
  TORCH_CHECK(plan.scalar_type() == at::kByte, "plan must come from spmm_plan");
  const int64_t k = b.size(0), n = b.size(1), nnz = values.numel();
  TORCH_CHECK(static_cast<size_t>(plan.numel()) >= iex_tile_plan_bytes(m, k, nnz, 64),
              "plan was built for another pattern size");
  c10::cuda::CUDAGuard guard(b.device());
  at::Tensor out = at::empty({m, n}, b.options());
  const size_t need = iex_spmm_f32_tc_workspace_bytes(m, k, n);
  at::Tensor scratch = at::empty({static_cast<int64_t>(std::max<size_t>(need, 16))}, b.options().dtype(at::kByte));
  check_status(iex_spmm_f32_tc(m, k, n, nnz, plan.data_ptr(), values.data_ptr<float>(), b.data_ptr<float>(),
                               out.data_ptr<float>(), scratch.data_ptr(), need, stream_of(b)),
               "iex_spmm_f32_tc");
  return out;
}

// 0 when the CSR is well formed, else the OR of the IEX_CSR_* bits (include/iex_b200.h)
int64_t validate_csr(const at::Tensor& row_offsets, const at::Tensor& column_indices, int64_t m, int64_t k,
                     bool require_ascending) {
  check_common({{"row_offsets", &row_offsets}, {"column_indices", &column_indices}});
  return validate_csr_impl(row_offsets, column_indices, m, k, nullptr, require_ascending);
}

}  // namespace

TORCH_LIBRARY(iex_ops, m) {
  m.def("spmm_sputnik_atomic(Tensor b, Tensor row_indices, Tensor values, Tensor row_offsets, Tensor column_indices, int m) -> Tensor");
  m.def("spmm_sputnik_reuse_weight(Tensor b, Tensor row_indices, Tensor values, Tensor row_offsets, Tensor column_indices, int m) -> Tensor");
  m.def("spmm_sputnik_reuse_weight_half(Tensor b, Tensor row_indices, Tensor values, Tensor row_offsets, Tensor column_indices, int m) -> Tensor");
  m.def("sddmm_sputnik_atomic_upd_weight(Tensor a, Tensor b, Tensor row_indices, Tensor row_offsets, Tensor column_indices) -> Tensor");
  m.def("sddmm_sputnik_half(Tensor a, Tensor b, Tensor row_indices, Tensor row_offsets, Tensor column_indices) -> Tensor");
  m.def("linear_fp16(Tensor input, Tensor weight) -> Tensor");
  m.def("linear_fp16_dgrad(Tensor grad, Tensor weight) -> Tensor");
  m.def("linear_fp16_wgrad(Tensor grad, Tensor input) -> Tensor");
  m.def("spmm_tc_half(Tensor x, Tensor row_offsets, Tensor values, Tensor column_indices, int m) -> Tensor");
  m.def("fused_spmm_linear_half(Tensor x, Tensor row_offsets, Tensor values, Tensor column_indices, int m, Tensor weight) -> (Tensor, Tensor)");
  m.def("csr_to_dense_half(Tensor row_offsets, Tensor values, Tensor column_indices, int m, int k) -> Tensor");
  m.def("validate_csr(Tensor row_offsets, Tensor column_indices, int m, int k, bool require_ascending) -> int");
  m.def("sddmm_plan(Tensor row_offsets, Tensor column_indices, int m, int n) -> Tensor");
  m.def("sddmm_tc_planned(Tensor a, Tensor b, Tensor plan, int nnz) -> Tensor");
  m.def("spmm_plan(Tensor row_offsets, Tensor column_indices, int m, int k) -> Tensor");
  m.def("spmm_tc_planned(Tensor b, Tensor values, Tensor plan, int m) -> Tensor");
}

// CUDA dispatch key only: a CPU tensor reaches no implementation (there is no CPU path).
TORCH_LIBRARY_IMPL(iex_ops, CUDA, m) {
  m.impl("spmm_sputnik_atomic", &spmm_sputnik_atomic);
  m.impl("spmm_sputnik_reuse_weight", &spmm_sputnik_reuse_weight);
  m.impl("spmm_sputnik_reuse_weight_half", &spmm_sputnik_reuse_weight_half);
  m.impl("sddmm_sputnik_atomic_upd_weight", &sddmm_sputnik_atomic_upd_weight);
  m.impl("sddmm_sputnik_half", &sddmm_sputnik_half);
  m.impl("linear_fp16", &linear_fp16);
  m.impl("linear_fp16_dgrad", &linear_fp16_dgrad);
  m.impl("linear_fp16_wgrad", &linear_fp16_wgrad);
  m.impl("spmm_tc_half", &spmm_tc_half);
  m.impl("fused_spmm_linear_half", &fused_spmm_linear_half);
  m.impl("csr_to_dense_half", &csr_to_dense_half);
  m.impl("validate_csr", &validate_csr);
  m.impl("sddmm_plan", &sddmm_plan);
  m.impl("sddmm_tc_planned", &sddmm_tc_planned);
  m.impl("spmm_plan", &spmm_plan);
  m.impl("spmm_tc_planned", &spmm_tc_planned);
}

/*
 * iex_b200 — C ABI of the B200 (sm_100a) implementation of intrasm_engine's hot path:
 * CSR SpMM, SDDMM, the dense fp16 linear and the fused sparse||dense layer.
 *
 * Plain pointers and sizes only.  All pointers are device pointers unless a comment says
 * "host".  `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 * No entry point synchronises, allocates or frees unless its comment says so, so all of
 * them may be called while the stream is being captured into a CUDA graph — the
 * reference wraps these calls in capture_library_call_begin/end
 * (intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/sputnik.py:59-66).
 *
 * Return value: 0 on success; a positive value is the cudaError_t of the launch (the
 * reference's launchers return cudaGetLastError(),
 * intrasm_engine/pytorch/csrc/extensions/sputnik_spmm.cu.inc:359); a negative value is
 * one of IEX_ERR_* (argument rejected before any launch).
 */
#ifndef IEX_B200_H_
#define IEX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define IEX_API __attribute__((visibility("default")))
#else
#define IEX_API
#endif

#define IEX_OK 0
#define IEX_ERR_BAD_ARG (-1)      /* null pointer, negative size, batch out of range   */
#define IEX_ERR_UNSUPPORTED (-2)  /* shape outside what the kernel family implements   */
#define IEX_ERR_TOO_LARGE (-3)    /* exceeds a fixed-size resource named in the comment */
#define IEX_ERR_DRIVER (-4)       /* a driver entry point (tensor-map encode) failed   */
#define IEX_ERR_TIMEOUT (-5)      /* a bounded device-side wait gave up (status word)  */
#define IEX_ERR_BAD_CSR (-6)      /* malformed CSR argument (see iex_csr_validate)        */

/* Human-readable text for any return value above (static storage, never NULL). */
IEX_API const char* iex_error_string(int status);

/* Library version, and the SM architecture the kernels were compiled for (100). */
IEX_API int iex_version(void);
IEX_API int iex_compiled_sm(void);

/* ------------------------------------------------------------------------------------
 * CSR SpMM      out[z, r, :] = sum_{p in row r} values[p] * dense[z, col[p], :]
 *
 * Replaces my_sputnik::CudaSpmm2 / CudaSpmm3 / CudaSpmmBiasRelu{2,3}
 * (intrasm_engine/pytorch/csrc/extensions.h:10-17, :28-29;
 *  sputnik_spmm_host_func.cu.inc:118-218).
 *   row_indices  int32[m]    row visiting order (rows by decreasing nnz)
 *   row_offsets  int32[m+1]  column_indices int32[nnz]
 *   values       fp32, shared by the batch (values_batch_stride = 0, the "reuse_weight"
 *                stamp) or one vector per batch item (stride = nnz, the "atomic" stamp)
 *   dense [batch,k,n], out [batch,m,n], row-major contiguous
 *   bias  fp32[m] or NULL; when given, out = relu(sum + bias[r])
 *   accumulate != 0: the result is added onto `out` with atomic adds (the reference's
 *                atomic store, sputnik_spmm.cu.inc:287-290); 0: plain store.
 * Without `accumulate` every output element is summed by one thread in storage order
 * with fused multiply-adds, so results are deterministic and reproducible bit for bit.
 * ------------------------------------------------------------------------------------ */
IEX_API int iex_spmm_f32(int m, int k, int n, int nnz, const int32_t* row_indices,
                 const float* values, long long values_batch_stride,
                 const int32_t* row_offsets, const int32_t* column_indices,
                 const float* dense, const float* bias, float* out, int batch,
                 int accumulate, void* stream);

/* fp16 storage, fp32 accumulate.  Replaces my_sputnik::CudaSpmm5 / CudaSpmmBiasRelu5
 * (extensions.h:30; sputnik_spmm_host_func_half.cu.inc:3-63), whose column indices are
 * 16-bit (sputnik_kernels.cpp:179-181).  Unlike the reference kernel, odd n, odd row
 * lengths and odd row offsets are accepted.  `_i32` is the same kernel with 32-bit
 * column indices (k may exceed 65535). values/dense/out are IEEE binary16. */
IEX_API int iex_spmm_f16_i16(int m, int k, int n, int nnz, const int32_t* row_indices,
                     const void* values, const int32_t* row_offsets,
                     const uint16_t* column_indices, const void* dense, const float* bias,
                     void* out, int batch, void* stream);
IEX_API int iex_spmm_f16_i32(int m, int k, int n, int nnz, const int32_t* row_indices,
                     const void* values, const int32_t* row_offsets,
                     const int32_t* column_indices, const void* dense, const float* bias,
                     void* out, int batch, void* stream);

/* ------------------------------------------------------------------------------------
 * SDDMM     out[p] = sum_z dot(lhs[z, row(p), :], rhs[z, col[p], :])   for every stored p
 *
 * Replaces my_sputnik::CudaSddmm2 (extensions.h:19-26, :31;
 * sputnik_sddmm.cu.inc:186-233).  lhs [batch,m,k], rhs [batch,n,k], out fp32[nnz] in the
 * order of column_indices.  The batch items are summed inside the kernel (the reference
 * adds them with atomics into one vector, sputnik_sddmm.cu.inc:177-178).
 * accumulate != 0 adds onto `out` (atomic adds); 0 overwrites it.
 * ------------------------------------------------------------------------------------ */
IEX_API int iex_sddmm_f32(int m, int k, int n, int nnz, const int32_t* row_indices,
                  const int32_t* row_offsets, const int32_t* column_indices,
                  const float* lhs, const float* rhs, float* out, int batch,
                  int accumulate, void* stream);

/* The fp16 instantiation (fp16 operands and result, fp32 accumulation; 16- or 32-bit column
 * indices), which the reference declares and leaves commented out
 * (sputnik_kernels.cpp:185-187): the backward pass of an fp16 SpMM needs it.  Overwrites out. */
IEX_API int iex_sddmm_f16(int m, int k, int n, int nnz, const int32_t* row_indices,
                  const int32_t* row_offsets, const void* column_indices, int index_bits,
                  const void* lhs, const void* rhs, void* out, int batch, void* stream);

/* SDDMM on tensor cores (tcgen05.mma.kind::tf32 into TMEM), fp32 in and out; same result
 * contract as iex_sddmm_f32 with batch = 1 (replaces my_sputnik::CudaSddmm2,
 * extensions.h:19-26, :31).  The dense product of a 128-row band of lhs with 128 rows of
 * rhs is formed per tile -- each value split into a TF32 head and tail, three products per
 * tile, error below 2^-19 of sum |lhs||rhs| -- and only the stored positions are written,
 * out[] in storage order as always.
 *
 * Which positions a tile holds comes from a PLAN, a pattern-only argument like the
 * reference's row_indices (computed once per sparsity pattern, reused by every call on it):
 * the stored positions regrouped by 128 x 128 tile.
 *   iex_sddmm_plan_bytes   size of a plan for an m x n pattern with nnz stored positions
 *   iex_sddmm_plan_build   fills `plan` (device memory, 16-byte aligned, caller-owned) from
 *                          row_offsets / column_indices: a memset and three small kernels on
 *                          `stream`.  Column indices need not ascend; an index outside [0, n)
 *                          is left out of the plan (its out[] position is not written).
 *   iex_sddmm_f32_tc       the product; `plan` must have been built for the same m, n, nnz.
 * Limits: k = 32 or 64, lhs / rhs 16-byte aligned (else IEX_ERR_UNSUPPORTED).
 * iex_sddmm_f32_tc_supported tells whether a shape is inside the limits;
 * iex_sddmm_f32_prefers_tc whether this kernel is expected to beat the CUDA-core one
 * (its time follows m * n, the CUDA-core kernel's follows nnz). */
IEX_API size_t iex_sddmm_plan_bytes(int m, int n, int nnz);
IEX_API int iex_sddmm_plan_build(int m, int n, int nnz, const int32_t* row_offsets,
                                 const int32_t* column_indices, void* plan, size_t plan_bytes,
                                 void* stream);
IEX_API int iex_sddmm_f32_tc(int m, int k, int n, int nnz, const void* plan, const float* lhs,
                             const float* rhs, float* out, int accumulate, void* stream);

/* Several products of one shape (m, k, n) in ONE launch: problem i has its own lhs[i], rhs[i],
 * outs[i], nnz[i] and plans[i] (host arrays of `count` entries, count <= iex_sddmm_f32_tc_max_batch()).
 * The kernel's fixed costs (launch, the first lhs band, the last tile's read-out) are paid once
 * and a CTA loads its next unit's lhs band while the tensor core works on the current one:
 * the heads of a sparse attention layer, or the independent instances of a throughput job.
 * Results equal `count` calls of iex_sddmm_f32_tc bit for bit.  No counterpart in the
 * reference, whose batch dimension sums the products into one vector (sputnik_sddmm.cu.inc:177-178). */
IEX_API int iex_sddmm_f32_tc_batched(int count, int m, int k, int n, const int* nnz,
                                     const void* const* plans, const float* const* lhs,
                                     const float* const* rhs, float* const* outs, int accumulate,
                                     void* stream);
IEX_API int iex_sddmm_f32_tc_max_batch(void);
IEX_API int iex_sddmm_f32_tc_supported(int m, int k, int n, int batch);
IEX_API int iex_sddmm_f32_prefers_tc(int m, int k, int n, int nnz, int batch);

/* The plan in general: stored positions regrouped by tile of 128 rows x tile_cols columns
 * (tile_cols 64 or 128).  iex_sddmm_plan_* are these with tile_cols = 128; the tensor-core
 * SpMM below takes tile_cols = 64.  No counterpart in the reference beyond row_indices. */
IEX_API size_t iex_tile_plan_bytes(int m, int n, int nnz, int tile_cols);
IEX_API int iex_tile_plan_build(int m, int n, int nnz, int tile_cols, const int32_t* row_offsets,
                                const int32_t* column_indices, void* plan, size_t plan_bytes,
                                void* stream);

/* CSR SpMM on tensor cores, fp32 in and out: out [m, n] = A_csr [m, k] * dense [k, n]; same
 * result contract as iex_spmm_f32 with batch = 1, shared values, no bias (replaces
 * my_sputnik::CudaSpmm2 / CudaSpmm3, extensions.h:10-17).  A 128-row band of A is expanded, 64
 * columns at a time, into a dense shared-memory operand (TF32 head and tail planes) and
 * multiplied with the matching rows of `dense` by tcgen05.mma.kind::tf32; error below 2^-19 of
 * sum |a||b|, summation order fixed (results do not depend on timing).
 *   plan       a tile plan of A's pattern with tile_cols = 64 (iex_tile_plan_build(m, k, ...))
 *   workspace  device memory, 16-byte aligned, iex_spmm_f32_tc_workspace_bytes(m, k, n) bytes
 *              (0 for matrices of many bands): partial results of bands that are cut into
 *              several units; a second small kernel adds them in unit order.
 * Limits: n = 32 or 64; dense / out 16-byte aligned (else IEX_ERR_UNSUPPORTED).
 * iex_spmm_f32_prefers_tc: whether this kernel is expected to beat the CUDA-core one. */
IEX_API int iex_spmm_f32_tc(int m, int k, int n, int nnz, const void* plan, const float* values,
                            const float* dense, float* out, void* workspace, size_t workspace_bytes,
                            void* stream);
IEX_API size_t iex_spmm_f32_tc_workspace_bytes(int m, int k, int n);
IEX_API int iex_spmm_f32_tc_supported(int m, int k, int n);
IEX_API int iex_spmm_f32_prefers_tc(int m, int k, int n, int nnz);

/* ------------------------------------------------------------------------------------
 * Tensor-core (tcgen05 / TMEM / TMA) entry points, fp16 storage, fp32 accumulate.
 * Shared limits: n (tokens) a multiple of 16 (dense) / 64 (sparse, fused) and <= 256;
 * k a multiple of 8; operand base pointers 16-byte aligned.  Shapes outside these limits
 * return IEX_ERR_UNSUPPORTED (the CUDA-core entry points above take any shape).
 * A device-side wait that gives up leaves IEX_ERR_TIMEOUT in a status word that
 * iex_last_device_status() reads back (it synchronises the device; not capturable).
 * ------------------------------------------------------------------------------------ */

/* Dense branch: out[t, f] = sum_c input[t, c] * weight[f, c]  (input @ weight^T).
 * Replaces the cuBLAS call behind MyLinear.forward
 * (intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/torch.py:17) and the
 * CUTLASS-Python / Triton dense paths (intrasm_engine/common/cutlass_utils.py:106-204,
 * triton_utils.py:14-137).  input [tokens, in_features], weight [out_features,
 * in_features], out [tokens, out_features], all row-major fp16. */
IEX_API int iex_linear_f16(int tokens, int in_features, int out_features, const void* input,
                           const void* weight, void* out, void* stream);

/* Backward pass of the dense branch on the same tensor-core kernel (operands read in their
 * other major-ness straight from the forward's tensors, no transposed copies).  Replace the two
 * cuBLAS calls of MyLinear.backward
 * (intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/torch.py:20-31).
 *   dgrad  dinput [tokens, in_features] = grad [tokens, out_features] * weight [out_features, in_features]
 *          tokens a multiple of 16 and <= 256; in_features, out_features multiples of 8.
 *   wgrad  dweight [out_features, in_features] = grad^T * input, input [tokens, in_features]
 *          any number of tokens that is a multiple of 8; in_features, out_features multiples of 8.
 * All row-major fp16, 16-byte aligned; fp32 accumulation. */
IEX_API int iex_linear_f16_dgrad(int tokens, int in_features, int out_features, const void* grad,
                                 const void* weight, void* dinput, void* stream);
IEX_API int iex_linear_f16_wgrad(int tokens, int in_features, int out_features, const void* grad,
                                 const void* input, void* dweight, void* stream);

/* CSR SpMM on tensor cores: out[r, :] = sum_p values[p] * dense[col[p], :].
 * Same contract as iex_spmm_f16_i16 / _i32 with batch = 1 and no bias (replaces
 * my_sputnik::CudaSpmm5, extensions.h:30), plus one precondition: column indices ascend
 * inside each row.  Rows are taken in natural order in tiles of 128, so no row_indices
 * argument.  index_bits is 16 or 32.  Meant for moderate sparsity, where expanding a row
 * tile into a dense shared-memory operand costs less than gathering dense rows. */
IEX_API int iex_spmm_f16_tc(int m, int k, int n, int nnz, const int32_t* row_offsets,
                            const void* column_indices, int index_bits, const void* values,
                            const void* dense, void* out, void* stream);

/* The same with the reference's bias + ReLU epilogue (my_sputnik::CudaSpmmBiasRelu5,
 * extensions.h:30; sputnik_spmm.cu.inc:273-282): out[r, :] = relu(sum + bias[r]); bias fp32[m],
 * NULL for the plain product. */
IEX_API int iex_spmm_f16_tc_bias_relu(int m, int k, int n, int nnz, const int32_t* row_offsets,
                                      const void* column_indices, int index_bits, const void* values,
                                      const void* dense, const float* bias, void* out, void* stream);

/* Fused sparse || dense layer: ONE launch computes
 *     out_sparse[r, t] = sum_p values[p] * x[col[p], t]        (CSR W_sparse [m_sparse, k])
 *     out_dense        = weight [m_dense, k] times x           (dense)
 * with x [k, n] read by both branches.  This is the kernel behind the pair function of
 * MySpMM + MyLinear (intrasm_engine/pytorch/horizontal_rewriter.py:76-311), replacing the
 * two-stream graph interleaving of tests/test_interleaving.py:434-476.
 * out_dense is [n, m_dense] (tokens major, the MyLinear convention) when
 * dense_out_tokens_major != 0, else [m_dense, n]. */
IEX_API int iex_fused_spmm_linear_f16(int m_sparse, int m_dense, int k, int n, int nnz,
                                      const int32_t* row_offsets, const void* column_indices,
                                      int index_bits, const void* values, const void* weight,
                                      const void* x, void* out_sparse, void* out_dense,
                                      int dense_out_tokens_major, void* stream);

/* Split-K variants of the three tensor-core entry points.  Every 128-row tile's K range is
 * cut into `parts` runs handled by different CTAs, so that few-tile problems (a tall-skinny
 * weight, or 86 decoder-bound sparse tiles on 148 SMs) use the whole GPU.  The fp32 partial
 * tiles go through `workspace` (device memory, 256-byte aligned, at least
 * iex_tc_workspace_bytes(...) bytes, contents irrelevant); a second small kernel on the
 * same stream adds the parts in part order, so results do not depend on timing.  Two
 * launches that use one workspace must not overlap.  parts = 1 needs no workspace and is
 * identical to the plain entry point.  With parts > 1 the dense linear needs tokens to be a
 * multiple of 32.  These have no counterpart in the reference. */
IEX_API size_t iex_tc_workspace_bytes(int m_sparse, int sparse_parts, int m_dense, int dense_parts,
                                      int n);
IEX_API int iex_linear_f16_splitk(int tokens, int in_features, int out_features, const void* input,
                                  const void* weight, void* out, int parts, void* workspace,
                                  size_t workspace_bytes, void* stream);
IEX_API int iex_spmm_f16_tc_splitk(int m, int k, int n, int nnz, const int32_t* row_offsets,
                                   const void* column_indices, int index_bits, const void* values,
                                   const void* dense, void* out, int parts, void* workspace,
                                   size_t workspace_bytes, void* stream);
IEX_API int iex_fused_spmm_linear_f16_splitk(int m_sparse, int m_dense, int k, int n, int nnz,
                                             const int32_t* row_offsets, const void* column_indices,
                                             int index_bits, const void* values, const void* weight,
                                             const void* x, void* out_sparse, void* out_dense,
                                             int dense_out_tokens_major, int sparse_parts,
                                             int dense_parts, void* workspace, size_t workspace_bytes,
                                             void* stream);

/* iex_linear_f16_splitk for callers that cannot hand over a workspace because they may
 * not allocate device memory while running (a serving process or plugin host whose memory
 * budget is fixed at start-up and which bans later cudaMalloc calls, since those
 * synchronise the device and may fail under fragmentation).  No counterpart in the
 * reference.  Same arguments and results as iex_linear_f16_splitk minus the workspace: the
 * partial tiles go to a fixed array inside the library, iex_static_workspace_capacity()
 * bytes (8 MiB) on every GPU that loads the library, held until the process exits.  The
 * call allocates and frees nothing, neither directly nor through a library.  It returns
 * IEX_ERR_TOO_LARGE when ceil(out_features / 128) * parts * 128 * tokens * 4 bytes exceed
 * that capacity.  The first call on a device looks the array's address up (a runtime
 * query, once per device, with that device current); make that first call before any
 * stream capture.  All calls on a device share the one array and each overwrites what the
 * previous left (nothing in it has to start at zero): two calls that overlap on the GPU
 * race, so keep them on one stream or order them with events. */
IEX_API size_t iex_static_workspace_capacity(void);
IEX_API int iex_linear_f16_splitk_static(int tokens, int in_features, int out_features,
                                         const void* input, const void* weight, void* out,
                                         int parts, void* stream);

/* Column-sharded linear whose all-gather is done by the kernel's own stores.  Rank `rank` of
 * `world` GPUs of one box (<= 8) computes its [tokens, out_features] slab of a wider
 * [tokens, ld_out] result -- columns [col_offset, col_offset + out_features) -- and the
 * threads that produce it store it into EVERY rank's copy of the result: outs[r] (a host
 * array of `world` device pointers) is rank r's [tokens, ld_out] buffer, reachable from this
 * GPU (peer access over NVLink, e.g. CUDA IPC or symmetric memory).  This replaces the
 * per-layer NCCL all-gather of the column-sharded FFN down projection; the reference has no
 * multi-GPU code (layers_and_funcs/torch.py:34-36 is an empty MyLinearPartitioned).  Other
 * arguments as iex_linear_f16_splitk.  col_offset and ld_out must be multiples of 8.
 * The stores are plain global stores; follow the call with iex_peer_barrier() before any
 * rank reads the gathered result. */
IEX_API int iex_linear_f16_splitk_gather(int tokens, int in_features, int out_features,
                                         const void* input, const void* weight, void* const* outs,
                                         int world, int rank, long long ld_out, long long col_offset,
                                         int parts, void* workspace, size_t workspace_bytes,
                                         void* stream);

/* Barrier among the `world` GPUs of one box, enqueued on `stream`: one small kernel that
 * makes this GPU's earlier stores visible system-wide, publishes a new epoch in every
 * rank's signal array and waits until every rank's epoch has arrived here.  signals[r] (host
 * array of `world` device pointers) is rank r's array of world + 1 uint32 words, zeroed
 * once before the first barrier and reachable from every GPU.  Every rank must enqueue the
 * same sequence of barriers.  The wait is bounded (a fraction of a second); when it gives
 * up, IEX_ERR_TIMEOUT is left for iex_last_device_status() and the kernel returns.  No
 * counterpart in the reference. */
IEX_API int iex_peer_barrier(void* const* signals, int world, int rank, void* stream);

/* The same barrier with the caller's own limit on the wait: max_polls polls of about 100 ns
 * each (0 = the default, also the upper limit).  A rank that knows a peer may have left (a
 * host-side heartbeat went missing) can bound the damage to microseconds, and a test can make
 * the wait run out on purpose -- a signal word that nobody writes -- to see the failure path:
 * the kernel returns, IEX_ERR_TIMEOUT is left in the status word, and the context stays
 * usable.  No counterpart in the reference. */
IEX_API int iex_peer_barrier_bounded(void* const* signals, int world, int rank, unsigned max_polls,
                                     void* stream);

/* Dense fp16 copy of a CSR matrix: out [m, k] row-major, zeros where nothing is stored.
 * The device-side counterpart of the CSR <-> dense conversions the reference delegates to
 * xformers (intrasm_engine/pytorch/utils.py:143-153); used to hand an activation CSR to the
 * tensor-core linear as its dense tile operand.  index_bits is 16 or 32. */
IEX_API int iex_csr_to_dense_f16(int m, int k, const int32_t* row_offsets, const void* column_indices,
                                 int index_bits, const void* values, void* out, void* stream);

/* Dense matrix -> CSR on the device, in two calls, for the conversions the reference
 * delegates to xformers (_dense_to_sparse, intrasm_engine/pytorch/utils.py:143-153) and for
 * ReLU-sparse activations, which become a new CSR every layer.  dense [m, k] row-major,
 * fp16 (value_bits 16) or fp32 (32).  An element is stored when it is != 0, or, with
 * relu != 0, when it is > 0 (the CSR of relu(dense)).
 *   iex_dense_to_csr_count  writes row_offsets int32[m+1] and row_indices int32[m] (rows by
 *                           decreasing length, equal lengths in row order).  The caller then
 *                           reads nnz = row_offsets[m] (its own copy and synchronisation)
 *                           and allocates values[nnz] (same type as dense) and
 *                           column_indices[nnz] (index_bits 16 or 32).
 *   iex_dense_to_csr_fill   writes them, columns ascending inside each row.  */
IEX_API int iex_dense_to_csr_count(int m, int k, const void* dense, int value_bits, int relu,
                                   int32_t* row_offsets, int32_t* row_indices, void* stream);
IEX_API int iex_dense_to_csr_fill(int m, int k, const void* dense, int value_bits, int relu,
                                  const int32_t* row_offsets, void* values, void* column_indices,
                                  int index_bits, void* stream);

/* CSR sanity check on the device.  The reference's launchers trust their index arrays
 * (intrasm_engine/pytorch/csrc/extensions/sputnik_kernels.cpp:41-91 checks shapes and
 * dtypes only); the kernels here gather dense rows at column_indices unchecked, so a caller
 * that cannot vouch for its CSR runs this first.  Writes 0 to *result (a device word the
 * caller owns) when the matrix is well formed, else the OR of the IEX_CSR_* bits below.
 * row_indices may be NULL (not checked); require_ascending != 0 also demands strictly
 * ascending columns inside every row, the precondition of the tensor-core SpMM.  The call
 * enqueues a memset and one kernel on `stream`; the caller reads *result after its own
 * synchronisation.  Duplicate entries in row_indices are not detected. */
#define IEX_CSR_BAD_FIRST_OFFSET 1       /* row_offsets[0] != 0                        */
#define IEX_CSR_BAD_LAST_OFFSET 2        /* row_offsets[m] != nnz                      */
#define IEX_CSR_OFFSETS_NOT_MONOTONE 4   /* a row ends before it begins                */
#define IEX_CSR_COLUMN_OUT_OF_RANGE 8    /* a column index outside [0, k)              */
#define IEX_CSR_COLUMNS_NOT_ASCENDING 16 /* columns of a row not strictly ascending    */
#define IEX_CSR_BAD_ROW_INDEX 32         /* a row_indices entry outside [0, m)         */
IEX_API int iex_csr_validate(int m, int k, int nnz, const int32_t* row_offsets,
                             const void* column_indices, int index_bits,
                             const int32_t* row_indices, int require_ascending,
                             int32_t* result, void* stream);

/* 1 while `stream` is being captured into a CUDA graph, else 0.  Callers that want to
 * synchronise or read a result back (the CSR check above) ask this first. */
IEX_API int iex_stream_is_capturing(void* stream);

/* Last device-side failure recorded by any kernel of this library (0 = none).
 * Synchronises the device.  clear != 0 resets the word. */
IEX_API int iex_last_device_status(int clear);

/* ------------------------------------------------------------------------------------
 * CUDA-graph constructor: one graph assembled from work enqueued on several registered
 * streams, so that independent chains can be co-scheduled by the hardware.
 *
 * Replaces the pybind classes CUDAExperimentalGraphConstructor / CudaGraphWrapper
 * (intrasm_engine/pytorch/csrc/extensions/pybind.cu:529-615) and the native code under
 * them (intrasm_engine/common/include/helper_CUDAGraphConstructor.cu.h:106-166, :268-486;
 * helper_cuda_graph.cu.h:34-62).  Handles are opaque pointers; streams and events are
 * cudaStream_t / cudaEvent_t values, as the reference passes them (pybind.cu:367-399).
 * Host-only calls; a constructor must be used from one thread at a time.
 *   create / destroy                      CudaGraphWrapper ctor / dtor
 *   register_stream                       register_stream          (pybind.cu:553)
 *   add_event_record_node                 add_event_record_node
 *   add_stream_wait_event_node            add_stream_wait_event_node
 *   join                                  join
 *   capture_begin / capture_end           notify_before / notify_after_invoking_library_call
 *   instantiate / launch / exec_destroy   instantiate_graph_exec / execute_graph / destroy_graph_exec
 *   add_child / combine                   add_graph_as_child_node / combine_graphs
 *   dump / node_count                     dump_graph / print_graph
 * ------------------------------------------------------------------------------------ */
IEX_API void* iex_graph_create(void);
IEX_API int iex_graph_destroy(void* graph);
IEX_API int iex_graph_register_stream(void* graph, void* stream);
IEX_API int iex_graph_add_event_record_node(void* graph, void* event, void* stream);
IEX_API int iex_graph_add_stream_wait_event_node(void* graph, void* stream, void* event);
IEX_API int iex_graph_join(void* graph, void* const* streams, int count, void* dst_stream);
IEX_API int iex_graph_capture_begin(void* graph, void* stream);
IEX_API int iex_graph_capture_end(void* graph, void* stream);
IEX_API int iex_graph_instantiate(void* graph);
IEX_API int iex_graph_launch(void* graph, void* stream);
IEX_API int iex_graph_exec_destroy(void* graph);
IEX_API int iex_graph_node_count(void* graph, long long* nodes, long long* edges);
IEX_API int iex_graph_dump(void* graph, const char* path);
IEX_API int iex_graph_add_child(void* graph, void* child);
IEX_API void* iex_graph_combine(void* const* graphs, int count);

#ifdef __cplusplus
}
#endif
#endif /* IEX_B200_H_ */

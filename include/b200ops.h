/*
 * b200ops.h -- C ABI of libb200ops.so: hand-written sm_100a CUDA kernels for the aten
 * lowering hot path of torch-mojo-backend (torch.compile(backend=mojo_backend)).
 *
 * Contract shared by every entry point (it mirrors the contract of the reference's native
 * bridges, torch_mojo_backend/eager_kernels/bf16_matmul_ops.mojo:1-8,25-63 and
 * torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:1-6,20-61):
 *   - arguments are raw device pointers (storage offset already applied), sizes and strides
 *     in ELEMENTS, dtype enums, scalars, and the CUDA stream to enqueue on;
 *   - the caller owns every buffer, outputs and workspace included; nothing is allocated,
 *     nothing is synchronised and no tensor data is read on the host;
 *   - all validation happens before the first launch, so a failing call leaves no partial work;
 *   - the return value is B200_OK (0) or a negative status; no C++ exception crosses the ABI;
 *   - device-side waits are bounded: a kernel that gives up sets a bit in a per-device status
 *     word that b200_device_status() reads back.
 */
#ifndef B200OPS_H_
#define B200OPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

/* 2: b200_layer_norm_backward takes dx_add, dx_cast, dx_sum and dx_sum_dtype. */
#define B200_ABI_VERSION 2

/* status codes */
#define B200_OK 0
#define B200_ERR_INVALID_ARG (-1)   /* null pointer, negative size, bad enum */
#define B200_ERR_UNSUPPORTED (-2)   /* valid request that no kernel covers (dtype mix, head_dim...) */
#define B200_ERR_ALIGNMENT (-3)     /* pointer or stride not aligned as the chosen route needs */
#define B200_ERR_WORKSPACE (-4)     /* workspace missing or too small */
#define B200_ERR_CUDA (-5)          /* a CUDA runtime/driver call failed; see b200_last_error() */
#define B200_ERR_DEVICE_TIMEOUT (-6)/* a bounded device-side wait gave up (b200_device_status) */

/* element types */
#define B200_F32 0
#define B200_BF16 1

/* reductions for b200_reduce_lastdim */
#define B200_REDUCE_SUM 0
#define B200_REDUCE_MEAN 1
#define B200_REDUCE_AMAX 2

/* GEMM epilogue activation */
#define B200_EPILOGUE_NONE 0
#define B200_EPILOGUE_GELU_TANH 1
#define B200_EPILOGUE_GELU_ERF 2

/* kernel routes (args.route: request; b200_*_route(): answer) */
#define B200_ROUTE_AUTO 0
#define B200_ROUTE_SIMT 1     /* generic strided CUDA-core kernel, any layout */
#define B200_ROUTE_TCGEN05 2  /* TMA-fed tcgen05/TMEM tensor-core kernel */
#define B200_ROUTE_SKINNY 3   /* decode shapes, HBM bound: split-K small-M GEMM; split-KV attention for <= 16 query rows */
#define B200_ROUTE_SPLIT3 4   /* fp32 GEMM on the bf16 tensor cores: operands split into bf16 halves, three products
                                 accumulated in fp32 by one tensor-core launch (~2^-16 relative); needs workspace */

typedef void* b200_stream_t; /* cudaStream_t */

/* ---- library ------------------------------------------------------------------------ */

/* Replaces: the import-time handshake of the reference's lazily loaded CPython kernel
 * modules (torch_mojo_backend/eager_kernels/aten_fast.py:4495-4534). */
B200_API int32_t b200_abi_version(void);
B200_API const char* b200_status_string(int32_t status);
/* Thread-local detail text of the last non-OK status returned on this thread. */
B200_API const char* b200_last_error(void);
/* Reads (and clears) the current device's status word; *word == 0 means no kernel gave up.
 * Synchronises the device: test/debug use only. */
B200_API int32_t b200_device_status(uint32_t* word);

/* Test hook for the bounded waits: enqueues a one-warp kernel that waits, for at most limit_ns
 * (<= 100 ms), on a barrier nothing signals, and then gives up the way every kernel of the library
 * gives up a wait that ran out (CTA abort flag, bit 2 of the status word, normal return). Nothing
 * faults and nothing hangs; afterwards b200_device_status() reports B200_ERR_DEVICE_TIMEOUT once
 * and the device is as usable as before. No counterpart in the reference (its kernels trap or
 * spin); the production kernels use the same wait with a 2 s limit. */
B200_API int32_t b200_debug_wait_timeout(uint64_t limit_ns, b200_stream_t stream);

/* ---- row kernels (HBM bound) -------------------------------------------------------- */

/* LayerNorm over the last dim of x[rows, cols] (row stride x_row_stride, unit column
 * stride). y is contiguous [rows, cols]; mean/rstd (fp32 [rows]) may be NULL; gamma/beta may
 * be NULL. Two-pass centred variance in fp32, rstd = 1/sqrt(var + eps).
 * Replaces: aten_native_layer_norm (torch_mojo_backend/aten_functions.py:2828-2868) and
 * LayerNorm / _layer_norm_block_kernel (torch_mojo_backend/eager_kernels/nn_ops.mojo:208-326). */
B200_API int32_t b200_layer_norm(const void* x, const void* gamma, const void* beta, void* y,
                        float* mean, float* rstd, int64_t rows, int64_t cols,
                        int64_t x_row_stride, float eps, int32_t in_dtype,
                        int32_t param_dtype, int32_t out_dtype, b200_stream_t stream);

/* Row softmax of x[rows, cols] * scale along the last dim, optionally causal: with
 * causal != 0, row r attends to columns j <= r % q_len (top-left aligned) and masked
 * columns are written as exact 0.
 * Replaces: aten__softmax / aten_softmax (torch_mojo_backend/aten_functions.py:680-714) and
 * SoftmaxRows (torch_mojo_backend/eager_kernels/nn_ops.mojo:385-493). */
B200_API int32_t b200_softmax_lastdim(const void* x, void* y, int64_t rows, int64_t cols,
                             int64_t x_row_stride, float scale, int32_t causal, int64_t q_len,
                             int32_t in_dtype, int32_t out_dtype, b200_stream_t stream);

/* Row softmax of where(masked, fill, x * scale): the chain mul(scale) -> masked_fill(mask, fill)
 * -> _softmax of a decomposed attention in one pass over the scores. mask is bytes (torch.bool)
 * [mask_rows, cols] with row stride mask_row_stride; row r of x uses mask row r % mask_rows (a
 * [T, S] mask broadcast over batch and heads), and an element is masked where
 * (mask byte != 0) != (mask_invert != 0), so both masked_fill(mask, fill) and
 * where(keep, x, fill) map onto it. A row whose elements are all masked to -inf gives NaN, as torch.
 * Replaces: aten_masked_fill + aten__softmax (torch_mojo_backend/aten_functions.py:3965, 680-714)
 * with the fused contract of SoftmaxRows (torch_mojo_backend/eager_kernels/nn_ops.mojo:392-409),
 * generalised from its causal flag to an explicit mask. */
B200_API int32_t b200_softmax_masked(const void* x, const uint8_t* mask, void* y, int64_t rows,
                            int64_t cols, int64_t x_row_stride, int64_t mask_rows,
                            int64_t mask_row_stride, int32_t mask_invert, float fill, float scale,
                            int32_t in_dtype, int32_t out_dtype, b200_stream_t stream);

/* Elementwise GELU over numel contiguous elements; approximate_tanh selects the tanh form.
 * Replaces: aten_gelu (torch_mojo_backend/aten_functions.py:2062-2067) and
 * _gelu_forward_bf16_{exact,tanh}
 * (torch_mojo_backend/eager_kernels/activation_forward_kernels.mojo:22-56,137-154). */
B200_API int32_t b200_gelu(const void* x, void* y, int64_t numel, int32_t approximate_tanh,
                  int32_t dtype, b200_stream_t stream);

/* sum / mean / amax over the last dim of x[rows, cols] -> y[rows]; fp32 accumulation.
 * Replaces: aten_sum / aten_mean / aten_amax
 * (torch_mojo_backend/aten_functions.py:3310-3346, 2554-2603, 1001-1020) and
 * _reduce_block_kernel (torch_mojo_backend/eager_kernels/reduction_ops.mojo:161-263). */
B200_API int32_t b200_reduce_lastdim(const void* x, void* y, int64_t rows, int64_t cols,
                            int64_t x_row_stride, int32_t op, int32_t in_dtype,
                            int32_t out_dtype, b200_stream_t stream);

/* ---- backward of the row kernels (HBM bound) ------------------------------------------- */

/* dx = dy * gelu'(x) over numel contiguous elements, erf or tanh form; one dtype for all three.
 * Replaces: aten_gelu_backward (torch_mojo_backend/aten_functions.py:2070-2102) and
 * _gelu_backward_{exact,tanh}[_bf16]
 * (torch_mojo_backend/eager_kernels/activation_backward_ops.mojo:60-130). */
B200_API int32_t b200_gelu_backward(const void* dy, const void* x, void* dx, int64_t numel,
                           int32_t approximate_tanh, int32_t dtype, b200_stream_t stream);

/* dx[rows, cols] = scale * y * (dy - sum_j dy_j y_j) along the last dim: the backward of a row
 * softmax whose input had been multiplied by scale (aten._softmax_backward_data has scale 1).
 * dy and y have unit column stride and the given row strides; dx is contiguous.
 * Replaces: the softmax backward of the reference's decomposed attention
 * (torch_mojo_backend/eager_kernels/sdpa_backward_ops.mojo:28-78). */
B200_API int32_t b200_softmax_backward(const void* dy, const void* y, void* dx, int64_t rows,
                              int64_t cols, int64_t dy_row_stride, int64_t y_row_stride,
                              float scale, int32_t in_dtype, int32_t out_dtype,
                              b200_stream_t stream);

/* LayerNorm backward over x[rows, cols] with the forward's mean and rstd (fp32 [rows]):
 *   dx = rstd (g - mean_j g - xhat mean_j(g xhat)),  xhat = (x - mean) rstd,  g = dy gamma,
 *   dgamma = sum_rows dy xhat,  dbeta = sum_rows dy   (fp32 sums in a fixed order).
 * gamma may be NULL (ones); dgamma / dbeta may be NULL (not wanted) and are written in
 * param_dtype; dx is contiguous and has the dtype of dy, or fp32 when x is fp32 and dy bf16 (the
 * gradient a bf16 consumer sends back into an fp32 stream: no widening pass before the kernel).
 * dx_add may be NULL; otherwise it is a contiguous [rows, cols] tensor of dx's dtype that is added to
 * dx in the same pass (the gradient that reaches x along a residual branch). dx_cast may be NULL;
 * otherwise (dx fp32 only) it receives the same values rounded to bf16, contiguous: the operand of the
 * gradient GEMMs of the layer that produced x. dx_sum may be NULL; otherwise it receives, in
 * dx_sum_dtype, the column sums over the rows of dx_cast when that is given and of dx as stored
 * otherwise (that layer's bias gradient), fp32 accumulation in a fixed order. The workspace holds the
 * per-CTA column sums (b200_layer_norm_backward_workspace_bytes, 16-byte aligned).
 * Replaces: the decomposition of aten.native_layer_norm_backward
 * (torch_mojo_backend/aten_functions.py:2871) and the reference's eager kernels
 * _dx_warp_rows (torch_mojo_backend/eager_kernels/normalization_backward_dx.mojo:66-175) and
 * _partial_kernel / _final_kernel
 * (torch_mojo_backend/eager_kernels/normalization_backward_params.mojo:75-180). */
B200_API size_t b200_layer_norm_backward_workspace_bytes(int64_t rows, int64_t cols);
B200_API int32_t b200_layer_norm_backward(const void* dy, const void* x, const float* mean,
                                 const float* rstd, const void* gamma, const void* dx_add,
                                 void* dx, void* dgamma, void* dbeta, void* dx_cast, void* dx_sum,
                                 void* workspace, size_t workspace_bytes,
                                 int64_t rows, int64_t cols, int64_t dy_row_stride,
                                 int64_t x_row_stride, int32_t x_dtype, int32_t dy_dtype,
                                 int32_t param_dtype, int32_t dx_dtype, int32_t dx_sum_dtype,
                                 b200_stream_t stream);

/* y[cols] = sum over the rows of x[rows, cols] (unit column stride): the bias gradient of a linear
 * layer, aten.sum(dy, [0]). fp32 accumulation in a fixed order; workspace as above.
 * Replaces: aten_sum over a leading dim (torch_mojo_backend/aten_functions.py:3310-3346) and the
 * bias sum of aten_linear_backward (torch_mojo_backend/aten_functions.py:2323-2380). */
B200_API size_t b200_sum_rows_workspace_bytes(int64_t rows, int64_t cols, int32_t in_dtype);
B200_API int32_t b200_sum_rows(const void* x, void* y, void* workspace, size_t workspace_bytes,
                      int64_t rows, int64_t cols, int64_t x_row_stride, int32_t in_dtype,
                      int32_t out_dtype, b200_stream_t stream);

/* ---- index-driven row kernels (HBM bound) ---------------------------------------------- */

/* out[r, :] = table_a[idx_a[r], :] (+ table_b[idx_b[r % idx_b_len], :]) for r < rows: an embedding
 * gather, optionally summed with a second gather whose indices repeat with period idx_b_len (the
 * positional table of a [batch, seq] batch: idx_b = arange(seq)). Tables are [rows_x, cols] with the
 * given row strides and unit column stride; indices are int64; out is contiguous [rows, cols] in
 * out_dtype (bf16 tables may be widened to fp32 on the way out; the sum is taken in fp32). table_b
 * may be NULL. An index outside its table contributes zeros and sets bit 3 of the device status word.
 * Replaces: aten_embedding (torch_mojo_backend/aten_functions.py:1779-1831) and the add of the token
 * and positional embeddings that follows it in a GPT-2 graph (aten_add, :938). */
B200_API int32_t b200_embedding_sum(const void* table_a, const int64_t* idx_a, int64_t rows_a,
                           int64_t a_row_stride, const void* table_b, const int64_t* idx_b,
                           int64_t rows_b, int64_t b_row_stride, int64_t idx_b_len, void* out,
                           int64_t rows, int64_t cols, int32_t table_dtype, int32_t out_dtype,
                           b200_stream_t stream);

/* Index of the maximum over the last dim of x[rows, cols] -> out[rows] (int64). Ties go to the
 * smallest index, a NaN counts as the maximum (torch.argmax). Rows need no alignment (the 50257-wide
 * logits have a ragged pitch).
 * Replaces: aten_argmax (torch_mojo_backend/aten_functions.py:1108-1150), the step that turns the
 * LM head's logits into token ids. */
B200_API int32_t b200_argmax_lastdim(const void* x, int64_t* out, int64_t rows, int64_t cols,
                            int64_t x_row_stride, int32_t dtype, b200_stream_t stream);

/* dst[o, 0:inner] = src[o, 0:inner] for o < outer; rows are dst_row_stride / src_row_stride elements
 * of elem_bytes apart. One call per input writes a concatenation along any dim (outer = product of
 * the leading dims, inner = the input's extent along the dim times the trailing dims), and writing a
 * new token's K / V rows into a preallocated cache is the same copy with dst pointing at the slot.
 * Replaces: aten_cat (torch_mojo_backend/aten_functions.py:1432-1449). */
B200_API int32_t b200_copy_rows(void* dst, const void* src, int64_t outer, int64_t inner,
                       int64_t dst_row_stride, int64_t src_row_stride, int32_t elem_bytes,
                       b200_stream_t stream);

/* ---- GEMM ---------------------------------------------------------------------------- */

/* C[b] = act(alpha * A[b] @ B[b] + beta * bias) + residual, fp32 accumulation.
 * A is [m,k], B is [k,n], both with arbitrary element strides (a transposed view is just a
 * stride pair); C is [m,n] with unit column stride. fp32 operands: B200_ROUTE_AUTO takes the
 * split-precision tensor-core route for all but small problems (relative error ~2^-16, inside the
 * 1e-4 bar of the fp32 configurations); B200_ROUTE_SIMT is the exact fp32 CUDA-core kernel. bias is NULL, a 1-D [n] row
 * (bias_row_stride == 0) or a 2-D [m,n] matrix; residual is NULL or [m,n].
 * Replaces: aten_mm / aten_addmm / aten_bmm
 * (torch_mojo_backend/aten_functions.py:2631-2634, 970-992, 1414-1428) and the eager GEMM
 * bridges Bf16GemmBF16 / MatmulBiasSpec
 * (torch_mojo_backend/eager_kernels/bf16_matmul_ops.mojo:66-188,
 *  torch_mojo_backend/eager_kernels/matmul_ops.mojo:3500) and, for fp32 operands, the tensor-core
 * fp32 GEMM (torch_mojo_backend/eager_kernels/tf32_gemm_kernels.mojo:91,690,723). */
typedef struct b200_gemm_args {
  const void* a;
  const void* b;
  const void* bias;
  const void* residual;
  void* c;
  int64_t m, n, k, batch;
  int64_t a_row_stride, a_col_stride, a_batch_stride;
  int64_t b_row_stride, b_col_stride, b_batch_stride;
  int64_t c_row_stride, c_batch_stride;
  int64_t bias_row_stride;     /* 0: bias is a [n] row broadcast over m */
  int64_t residual_row_stride;
  float alpha, beta;
  int32_t in_dtype;            /* dtype of A and B */
  int32_t bias_dtype;
  int32_t residual_dtype;
  int32_t out_dtype;
  int32_t epilogue;            /* B200_EPILOGUE_* */
  int32_t route;               /* B200_ROUTE_AUTO or a forced route */
} b200_gemm_args;

/* The route B200_ROUTE_AUTO resolves to for these arguments (no launch), or a negative status. */
B200_API int32_t b200_gemm_route(const b200_gemm_args* args);
/* Bytes of workspace the resolved route needs (0 for most routes). */
B200_API size_t b200_gemm_workspace_bytes(const b200_gemm_args* args);
B200_API int32_t b200_gemm(const b200_gemm_args* args, void* workspace, size_t workspace_bytes,
                  b200_stream_t stream);

/* Small-M GEMM (the split-K route of b200_gemm) for callers that must not allocate device
 * memory and have no workspace to lend: a plugin running inside another engine's memory budget,
 * a serving loop that froze its memory pool after start-up, a host language whose binding can
 * only hand over the operand buffers it was given. The scratch for the partial sums is a static
 * array of B200_STATIC_SCRATCH_BYTES inside the library (every GPU that loads the library keeps
 * that much memory until the process exits). No cudaMalloc/cudaFree or other allocating call is
 * made.
 *  - Same arguments and result as b200_gemm; only problems that b200_gemm_route() resolves to
 *    B200_ROUTE_SKINNY are accepted (others: B200_ERR_UNSUPPORTED), and those that need more
 *    scratch than the array holds are refused with B200_ERR_WORKSPACE (use b200_gemm).
 *  - The first call on each device looks up the array's device address; make that first call
 *    before any stream capture is begun on that device.
 *  - All calls share the one array: two calls whose kernels may overlap on the GPU (different
 *    streams, or the same arguments from two threads) race on it. Serialise them on one stream.
 *    The array keeps the previous call's partial sums; every element a call reads it has first
 *    written itself, so no clearing is needed or done.
 * This entry point has no counterpart in the reference. */
#define B200_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
B200_API int32_t b200_gemm_small_m_static(const b200_gemm_args* args, b200_stream_t stream);

/* ---- attention ----------------------------------------------------------------------- */

/* softmax(scale * Q K^T [+ causal mask]) V per (batch, head); fp32 online softmax; writes
 * O (same dtype as Q) and, when lse != NULL, the natural-log LSE as fp32 [batch, heads, q_len].
 * Strides are in elements for the (batch, head, position) dims; head_dim is contiguous.
 * The causal mask is top-left aligned.
 * Routes: bf16 with head_dim 64 takes the tensor-core kernel; up to 16 query rows with
 * head_dim 32/64/128 and at most 32768 keys take the split-KV decode kernel (a cluster of eight
 * CTAs per row, merged through distributed shared memory); everything else the CUDA-core kernel.
 * Replaces: aten__scaled_dot_product_flash_attention
 * (torch_mojo_backend/aten_functions.py:539-677), the FA4 bridge
 * (torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:20-61,480-498) and the single-query
 * decode kernel (torch_mojo_backend/mojo_kernels/attention.mojo:27-191, gated at
 * torch_mojo_backend/aten_functions.py:3053-3074). */
typedef struct b200_sdpa_args {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  int64_t batch, heads, q_len, kv_len, head_dim;
  int64_t q_strides[3]; /* batch, head, position */
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t o_strides[3];
  float scale;
  int32_t causal;
  int32_t dtype;
  int32_t route; /* B200_ROUTE_AUTO / SIMT / TCGEN05 / SKINNY */
} b200_sdpa_args;

B200_API int32_t b200_sdpa_route(const b200_sdpa_args* args);
B200_API int32_t b200_sdpa_fwd(const b200_sdpa_args* args, b200_stream_t stream);

/* Gradients of b200_sdpa_fwd: dq, dk, dv ([batch, heads, len, head_dim] with the given element strides
 * and head_dim contiguous, dtype of q; a caller that wants them as [batch, len, heads * head_dim] passes
 * those strides and needs no transpose copy afterwards) from
 * d_out, the forward's output o and its natural-log LSE (fp32 [batch, heads, q_len], contiguous).
 * bf16 with head_dim 64 only (the tensor-core kernel); anything else is B200_ERR_UNSUPPORTED and the
 * caller composes the gradient from b200_gemm / b200_softmax_backward. Per 128-key tile one CTA keeps
 * dK and dV in tensor memory and walks the query tiles; the shares of dQ are written per key tile
 * to the workspace (b200_sdpa_bwd_workspace_bytes, 256-byte aligned) and added in tile order, so
 * the result does not depend on scheduling.
 * Replaces: aten._scaled_dot_product_flash_attention_backward through the FA4 backward bridge
 * (torch_mojo_backend/eager_flash_attention/fa4_bwd_kernel.mojo, fa4_bwd_launch.mojo). */
typedef struct b200_sdpa_bwd_args {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_out;
  const float* lse;
  void* dq;
  void* dk;
  void* dv;
  void* workspace;
  size_t workspace_bytes;
  int64_t batch, heads, q_len, kv_len, head_dim;
  int64_t q_strides[3]; /* batch, head, position */
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t o_strides[3];
  int64_t d_out_strides[3];
  int64_t dq_strides[3];
  int64_t dk_strides[3];
  int64_t dv_strides[3];
  float scale;
  int32_t causal;
  int32_t dtype;
} b200_sdpa_bwd_args;

B200_API size_t b200_sdpa_bwd_workspace_bytes(const b200_sdpa_bwd_args* args);
B200_API int32_t b200_sdpa_bwd(const b200_sdpa_bwd_args* args, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H_ */

// Index-driven row kernels on either side of the GEMMs of a language model forward: the embedding
// gather (token + positional table summed in one pass), the arg-max over the logits, and the copies
// that grow a KV cache. All HBM bound: 16-byte accesses, one warp or CTA per row.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kThreads = kWarpsPerCta * 32;

// ---- embedding (+ second table) --------------------------------------------------------------

// out[r, :] = A[ia[r], :] (+ B[ib[r % ib_len], :]), one warp per output row, 16-byte vectors of the
// table type. An index outside its table writes zeros for that term and raises a status bit.
template <typename Tt, typename Tout>
__global__ void __launch_bounds__(kThreads)
embedding_sum_kernel(const Tt* __restrict__ table_a, const int64_t* __restrict__ idx_a, int64_t rows_a,
                     const Tt* __restrict__ table_b, const int64_t* __restrict__ idx_b, int64_t rows_b,
                     int64_t idx_b_len, Tout* __restrict__ out, int64_t rows, int cols, int64_t a_row_stride,
                     int64_t b_row_stride, unsigned int* status) {
  constexpr int N = Elem<Tt>::kVec;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t ia = idx_a[row];
  const bool a_ok = ia >= 0 && ia < rows_a;
  int64_t ib = 0;
  bool b_ok = false;
  if (table_b != nullptr) {
    ib = idx_b[row % idx_b_len];
    b_ok = ib >= 0 && ib < rows_b;
  }
  if (lane == 0 && (!a_ok || (table_b != nullptr && !b_ok))) atomicOr(status, STATUS_INDEX_OUT_OF_RANGE);
  const Tt* ar = table_a + ia * a_row_stride;
  const Tt* br = table_b + ib * b_row_stride;
  Tout* orow = out + row * (int64_t)cols;
  const int nchunks = cols / N;
  for (int c = lane; c < nchunks; c += 32) {
    float v[N], w[N];
#pragma unroll
    for (int j = 0; j < N; ++j) { v[j] = 0.0f; w[j] = 0.0f; }
    if (a_ok) load16(ar + c * N, v);
    if (b_ok) load16(br + c * N, w);
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] += w[j];
    if constexpr (sizeof(Tout) * N == 16) {
      store16_stream(reinterpret_cast<Tout*>(orow) + c * N, reinterpret_cast<const float(&)[Elem<Tout>::kVec]>(v));
    } else {
      // fp32 output of bf16 tables: eight values, two 16-byte stores
      float lo[4] = {v[0], v[1], v[2], v[3]}, hi[4] = {v[N - 4], v[N - 3], v[N - 2], v[N - 1]};
      store16_stream(reinterpret_cast<float*>(orow) + c * N, lo);
      store16_stream(reinterpret_cast<float*>(orow) + c * N + 4, hi);
    }
  }
}

// Any layout: scalar accesses.
template <typename Tt, typename Tout>
__global__ void __launch_bounds__(kThreads)
embedding_sum_scalar_kernel(const Tt* __restrict__ table_a, const int64_t* __restrict__ idx_a, int64_t rows_a,
                            const Tt* __restrict__ table_b, const int64_t* __restrict__ idx_b, int64_t rows_b,
                            int64_t idx_b_len, Tout* __restrict__ out, int64_t rows, int64_t cols,
                            int64_t a_row_stride, int64_t b_row_stride, unsigned int* status) {
  const int64_t row = blockIdx.x;
  const int64_t ia = idx_a[row];
  const bool a_ok = ia >= 0 && ia < rows_a;
  int64_t ib = 0;
  bool b_ok = false;
  if (table_b != nullptr) {
    ib = idx_b[row % idx_b_len];
    b_ok = ib >= 0 && ib < rows_b;
  }
  if (threadIdx.x == 0 && (!a_ok || (table_b != nullptr && !b_ok))) atomicOr(status, STATUS_INDEX_OUT_OF_RANGE);
  for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
    float v = a_ok ? Elem<Tt>::to_f32(table_a[ia * a_row_stride + j]) : 0.0f;
    if (b_ok) v += Elem<Tt>::to_f32(table_b[ib * b_row_stride + j]);
    out[row * cols + j] = Elem<Tout>::from_f32(v);
  }
}

template <typename Tt, typename Tout>
int32_t launch_embedding_sum(const void* table_a, const int64_t* idx_a, int64_t rows_a, const void* table_b,
                             const int64_t* idx_b, int64_t rows_b, int64_t idx_b_len, void* out, int64_t rows,
                             int64_t cols, int64_t a_row_stride, int64_t b_row_stride, cudaStream_t stream) {
  constexpr int N = Elem<Tt>::kVec;
  unsigned int* status = device_status_ptr();
  B200_REQUIRE(status != nullptr, B200_ERR_CUDA, "embedding: device status word unavailable");
  const Tt* ta = static_cast<const Tt*>(table_a);
  const Tt* tb = static_cast<const Tt*>(table_b);
  Tout* o = static_cast<Tout*>(out);
  const bool vec_ok = cols % N == 0 && a_row_stride % N == 0 && aligned_to(table_a, 16) && aligned_to(out, 16) &&
                      (table_b == nullptr || (b_row_stride % N == 0 && aligned_to(table_b, 16))) &&
                      cols <= INT32_MAX && rows <= (int64_t)INT32_MAX * kWarpsPerCta;
  if (vec_ok) {
    const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
    embedding_sum_kernel<Tt, Tout><<<grid, kThreads, 0, stream>>>(ta, idx_a, rows_a, tb, idx_b, rows_b, idx_b_len, o,
                                                                  rows, (int)cols, a_row_stride, b_row_stride, status);
  } else {
    B200_REQUIRE(rows <= INT32_MAX, B200_ERR_UNSUPPORTED, "embedding: too many rows");
    embedding_sum_scalar_kernel<Tt, Tout><<<(unsigned)rows, kThreads, 0, stream>>>(
        ta, idx_a, rows_a, tb, idx_b, rows_b, idx_b_len, o, rows, cols, a_row_stride, b_row_stride, status);
  }
  B200_CHECK_LAUNCH("embedding");
  return B200_OK;
}

// ---- arg-max over the last dim ----------------------------------------------------------------

struct MaxAt {
  float v;
  int64_t i;
};

// Larger value wins, a NaN beats every number, ties go to the smaller index (torch.argmax).
__device__ __forceinline__ MaxAt better(MaxAt a, MaxAt b) {
  const bool a_nan = a.v != a.v, b_nan = b.v != b.v;
  bool take_b;
  if (a_nan || b_nan) take_b = b_nan && (!a_nan || b.i < a.i);
  else take_b = b.v > a.v || (b.v == a.v && b.i < a.i);
  return take_b ? b : a;
}

__device__ __forceinline__ MaxAt warp_best(MaxAt m) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxAt other;
    other.v = __shfl_xor_sync(0xffffffffu, m.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, m.i, o);
    m = better(m, other);
  }
  return m;
}

// One CTA per row: every thread walks 16-byte chunks of the row (scalar head and tail where the
// row does not start or end on a 16-byte boundary), then a warp and a CTA reduction.
template <typename T>
__global__ void __launch_bounds__(256)
argmax_row_kernel(const T* __restrict__ x, int64_t* __restrict__ out, int64_t cols, int64_t x_row_stride) {
  constexpr int N = Elem<T>::kVec;
  __shared__ float sv[8];
  __shared__ int64_t si[8];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * x_row_stride;
  MaxAt best = {-INFINITY, INT64_MAX};
  // elements before the first 16-byte boundary
  const uintptr_t addr = reinterpret_cast<uintptr_t>(xr);
  int64_t head = ((16 - (addr & 15)) & 15) / sizeof(T);
  if (head > cols) head = cols;
  for (int64_t j = threadIdx.x; j < head; j += blockDim.x) best = better(best, MaxAt{Elem<T>::to_f32(xr[j]), j});
  const int64_t nchunks = (cols - head) / N;
  const T* xa = xr + head;
  for (int64_t c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float v[N];
    load16_stream(xa + c * N, v);
#pragma unroll
    for (int j = 0; j < N; ++j) best = better(best, MaxAt{v[j], head + c * N + j});
  }
  for (int64_t j = head + nchunks * N + threadIdx.x; j < cols; j += blockDim.x)
    best = better(best, MaxAt{Elem<T>::to_f32(xr[j]), j});
  best = warp_best(best);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
  __syncthreads();
  if (warp == 0) {
    MaxAt m = lane < (int)(blockDim.x >> 5) ? MaxAt{sv[lane], si[lane]} : MaxAt{-INFINITY, INT64_MAX};
    m = warp_best(m);
    if (lane == 0) out[row] = m.i == INT64_MAX ? 0 : m.i;  // a row of -inf only: index 0, as torch
  }
}

// ---- strided block copy (concatenation, cache append) ------------------------------------------

// dst[o, j] = src[o, j] for o < outer, j < inner (elements of `esize` bytes moved as bytes), rows
// dst_stride / src_stride elements apart. 16-byte vectors when everything is aligned.
__global__ void __launch_bounds__(256)
copy_rows_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int64_t outer, int64_t inner_bytes,
                 int64_t dst_stride_bytes, int64_t src_stride_bytes, int vec) {
  if (vec) {
    const int64_t per_row = inner_bytes >> 4;
    const int64_t total = outer * per_row;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
      const int64_t o = t / per_row, j = t - o * per_row;
      const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src + o * src_stride_bytes) + j);
      reinterpret_cast<uint4*>(dst + o * dst_stride_bytes)[j] = v;
    }
  } else {
    const int64_t total = outer * inner_bytes;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
      const int64_t o = t / inner_bytes, j = t - o * inner_bytes;
      dst[o * dst_stride_bytes + j] = src[o * src_stride_bytes + j];
    }
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" B200_API int32_t b200_embedding_sum(const void* table_a, const int64_t* idx_a, int64_t rows_a,
                                               int64_t a_row_stride, const void* table_b, const int64_t* idx_b,
                                               int64_t rows_b, int64_t b_row_stride, int64_t idx_b_len, void* out,
                                               int64_t rows, int64_t cols, int32_t table_dtype, int32_t out_dtype,
                                               b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(rows >= 0 && cols >= 0 && rows_a >= 0, B200_ERR_INVALID_ARG, "embedding: negative extent");
  B200_REQUIRE(valid_dtype(table_dtype) && valid_dtype(out_dtype), B200_ERR_INVALID_ARG, "embedding: bad dtype enum");
  if (rows == 0 || cols == 0) return B200_OK;
  B200_REQUIRE(table_a != nullptr && idx_a != nullptr && out != nullptr, B200_ERR_INVALID_ARG, "embedding: null pointer");
  B200_REQUIRE(table_b == nullptr || (idx_b != nullptr && idx_b_len > 0 && rows_b >= 0), B200_ERR_INVALID_ARG,
               "embedding: second table without indices");
  B200_REQUIRE(a_row_stride >= cols && (table_b == nullptr || b_row_stride >= cols), B200_ERR_INVALID_ARG,
               "embedding: table row stride smaller than a row");
  B200_REQUIRE(aligned_to(table_a, dtype_size(table_dtype)) && aligned_to(out, dtype_size(out_dtype)) &&
                   aligned_to(idx_a, 8) && (table_b == nullptr || (aligned_to(table_b, dtype_size(table_dtype)) && aligned_to(idx_b, 8))),
               B200_ERR_ALIGNMENT, "embedding: pointer not element aligned");
  B200_REQUIRE(!(table_dtype == B200_F32 && out_dtype == B200_BF16), B200_ERR_UNSUPPORTED,
               "embedding: fp32 table with bf16 output is not supported");
#define EMB_LAUNCH(Tt, Tout) \
  launch_embedding_sum<Tt, Tout>(table_a, idx_a, rows_a, table_b, idx_b, rows_b, idx_b_len, out, rows, cols, a_row_stride, b_row_stride, stream)
  if (table_dtype == B200_F32) return EMB_LAUNCH(float, float);
  if (out_dtype == B200_BF16) return EMB_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  return EMB_LAUNCH(__nv_bfloat16, float);
#undef EMB_LAUNCH
}

extern "C" B200_API int32_t b200_argmax_lastdim(const void* x, int64_t* out, int64_t rows, int64_t cols,
                                                int64_t x_row_stride, int32_t dtype, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(rows >= 0 && cols > 0, B200_ERR_INVALID_ARG, "argmax: needs at least one column");
  B200_REQUIRE(valid_dtype(dtype), B200_ERR_INVALID_ARG, "argmax: bad dtype enum");
  if (rows == 0) return B200_OK;
  B200_REQUIRE(x != nullptr && out != nullptr, B200_ERR_INVALID_ARG, "argmax: null pointer");
  B200_REQUIRE(x_row_stride >= cols || rows == 1, B200_ERR_INVALID_ARG, "argmax: row stride smaller than a row");
  B200_REQUIRE(aligned_to(x, dtype_size(dtype)) && aligned_to(out, 8), B200_ERR_ALIGNMENT, "argmax: pointer not element aligned");
  B200_REQUIRE(rows <= INT32_MAX, B200_ERR_UNSUPPORTED, "argmax: too many rows");
  const int threads = cols >= 2048 ? 256 : 64;
  if (dtype == B200_F32)
    argmax_row_kernel<float><<<(unsigned)rows, threads, 0, stream>>>(static_cast<const float*>(x), out, cols, x_row_stride);
  else
    argmax_row_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), out, cols, x_row_stride);
  B200_CHECK_LAUNCH("argmax");
  return B200_OK;
}

extern "C" B200_API int32_t b200_copy_rows(void* dst, const void* src, int64_t outer, int64_t inner,
                                           int64_t dst_row_stride, int64_t src_row_stride, int32_t elem_bytes,
                                           b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(outer >= 0 && inner >= 0, B200_ERR_INVALID_ARG, "copy_rows: negative extent");
  B200_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8, B200_ERR_INVALID_ARG,
               "copy_rows: element size must be 1, 2, 4 or 8 bytes");
  if (outer == 0 || inner == 0) return B200_OK;
  B200_REQUIRE(dst != nullptr && src != nullptr, B200_ERR_INVALID_ARG, "copy_rows: null pointer");
  B200_REQUIRE((dst_row_stride >= inner && src_row_stride >= inner) || outer == 1, B200_ERR_INVALID_ARG,
               "copy_rows: row stride smaller than a row");
  B200_REQUIRE(aligned_to(dst, elem_bytes) && aligned_to(src, elem_bytes), B200_ERR_ALIGNMENT,
               "copy_rows: pointer not element aligned");
  const int64_t inner_b = inner * elem_bytes, ds = dst_row_stride * elem_bytes, ss = src_row_stride * elem_bytes;
  const int vec = aligned_to(dst, 16) && aligned_to(src, 16) && inner_b % 16 == 0 && ds % 16 == 0 && ss % 16 == 0;
  const int64_t work = vec ? outer * (inner_b >> 4) : outer * inner_b;
  int64_t blocks = (work + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  copy_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), outer,
                                                        inner_b, ds, ss, vec);
  B200_CHECK_LAUNCH("copy_rows");
  return B200_OK;
}

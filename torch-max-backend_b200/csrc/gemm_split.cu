// fp32 GEMM on the bf16 tensor cores, to fp32 accuracy.
//
// Every fp32 operand element x is written as x = hi + lo with hi = bf16(x) and lo = bf16(x - hi)
// (16 significant bits together), and the product is accumulated in fp32 as
//     A B ~= A_hi B_lo + A_lo B_hi + A_hi B_hi
// (the dropped A_lo B_lo term is ~2^-16 of a product; the three kept terms are exact products of
// bf16 numbers accumulated in fp32). A split kernel writes each operand once as a K-major bf16 matrix
// [rows, 2 * Kp] = [hi | lo] (Kp = K rounded up to the 64-element k-block, zero padded), and ONE launch
// of the tensor-core GEMM walks K three times with per-pass k offsets into those halves: no
// intermediate C passes through memory, the epilogue (alpha, bias, activation, residual, dtype) runs
// once on the final accumulator, and because both split operands are K-major the CTA-pair kernel
// applies whatever the layout of the original fp32 B was.
//
// The scratch for the split operands is the caller's workspace (b200_gemm_workspace_bytes).
#include "gemm_internal.cuh"

namespace b200 {
namespace {

constexpr int kSplitThreads = 256;

__device__ __forceinline__ void split_one(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

// Source rows are K-contiguous: row r is src[r * row_stride + k], k < K. One warp per output row,
// four consecutive k per lane and step (16-byte loads when aligned, 8-byte stores).
__global__ void __launch_bounds__(kSplitThreads)
split_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t rows, int64_t K,
                  int64_t Kp, int64_t row_stride, int vec) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kSplitThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* s = src + row * row_stride;
  __nv_bfloat16* d = dst + row * 2 * Kp;
  for (int64_t k = lane * 4; k < Kp; k += 128) {
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (vec && k + 4 <= K) {
      const float4 t = __ldcs(reinterpret_cast<const float4*>(s + k));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (k + j < K) v[j] = s[k + j];
    }
    __nv_bfloat16 hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) split_one(v[j], hi[j], lo[j]);
    *reinterpret_cast<uint2*>(d + k) = *reinterpret_cast<const uint2*>(hi);
    *reinterpret_cast<uint2*>(d + Kp + k) = *reinterpret_cast<const uint2*>(lo);
  }
}

// Source is MN-contiguous: element (r, k) is src[k * k_stride + r * r_stride] with r_stride == 1 in
// the fast case (a contiguous [K, N] weight). 32 x 32 tiles go through shared memory so that both the
// reads (along r) and the writes (along k) are coalesced.
__global__ void __launch_bounds__(kSplitThreads)
split_transposed_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t rows, int64_t K,
                        int64_t Kp, int64_t k_stride, int64_t r_stride) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t r0 = (int64_t)blockIdx.x * 32, k0 = (int64_t)blockIdx.y * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t k = k0 + ty + 8 * i, r = r0 + tx;
    tile[ty + 8 * i][tx] = (k < K && r < rows) ? src[k * k_stride + r * r_stride] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = r0 + ty + 8 * i, k = k0 + tx;
    if (r < rows && k < Kp) {
      __nv_bfloat16 hi, lo;
      split_one(tile[tx][ty + 8 * i], hi, lo);
      dst[r * 2 * Kp + k] = hi;
      dst[r * 2 * Kp + Kp + k] = lo;
    }
  }
}

int64_t padded_k(int64_t k) { return (k + 63) / 64 * 64; }

// rows x K source with strides (r_stride, k_stride) -> dst [rows, 2 * Kp]
int32_t launch_split(const float* src, __nv_bfloat16* dst, int64_t rows, int64_t K, int64_t r_stride,
                     int64_t k_stride, cudaStream_t stream) {
  const int64_t Kp = padded_k(K);
  if (k_stride == 1) {
    const int vec = aligned_to(src, 16) && r_stride % 4 == 0;
    const int64_t blocks = (rows + kSplitThreads / 32 - 1) / (kSplitThreads / 32);
    B200_REQUIRE(blocks <= INT32_MAX, B200_ERR_UNSUPPORTED, "gemm(split): too many rows");
    split_rows_kernel<<<(unsigned)blocks, kSplitThreads, 0, stream>>>(src, dst, rows, K, Kp, r_stride, vec);
  } else {
    const int64_t bx = (rows + 31) / 32, by = Kp / 32;
    B200_REQUIRE(bx <= INT32_MAX && by <= 65535, B200_ERR_UNSUPPORTED, "gemm(split): operand too large");
    split_transposed_kernel<<<dim3((unsigned)bx, (unsigned)by), kSplitThreads, 0, stream>>>(src, dst, rows, K, Kp,
                                                                                            k_stride, r_stride);
  }
  B200_CHECK_LAUNCH("gemm(split operands)");
  return B200_OK;
}

}  // namespace

const char* gemm_split_ineligible(const b200_gemm_args& g) {
  if (g.in_dtype != B200_F32) return "operands are not fp32";
  if (g.batch != 1) return "batched";
  if (g.k <= 0) return "k is zero";
  if (g.m > INT32_MAX - 256 || g.n > INT32_MAX - 256 || g.k > (INT32_MAX - 256) / 2) return "extent exceeds TMA coordinate range";
  if (g.a_row_stride < 0 || g.a_col_stride < 0 || g.b_row_stride < 0 || g.b_col_stride < 0) return "negative stride";
  return nullptr;
}

size_t gemm_split_scratch_bytes(const b200_gemm_args& g) {
  if (gemm_split_ineligible(g) != nullptr) return 0;
  const size_t Kp = (size_t)padded_k(g.k);
  const size_t a_bytes = ((size_t)g.m * 2 * Kp * 2 + 255) / 256 * 256;
  const size_t b_bytes = ((size_t)g.n * 2 * Kp * 2 + 255) / 256 * 256;
  return a_bytes + b_bytes;
}

int32_t launch_gemm_split(const b200_gemm_args& g, void* scratch, size_t scratch_bytes, cudaStream_t stream) {
  const char* why = gemm_split_ineligible(g);
  B200_REQUIRE(why == nullptr, B200_ERR_UNSUPPORTED, "gemm(split): %s", why);
  const size_t need = gemm_split_scratch_bytes(g);
  B200_REQUIRE(scratch != nullptr && scratch_bytes >= need, B200_ERR_WORKSPACE,
               "gemm(split): scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  B200_REQUIRE(aligned_to(scratch, 256), B200_ERR_ALIGNMENT, "gemm(split): scratch not 256-byte aligned");
  const int64_t Kp = padded_k(g.k);
  __nv_bfloat16* a2 = static_cast<__nv_bfloat16*>(scratch);
  const size_t a_bytes = ((size_t)g.m * 2 * Kp * 2 + 255) / 256 * 256;
  __nv_bfloat16* b2 = reinterpret_cast<__nv_bfloat16*>(static_cast<unsigned char*>(scratch) + a_bytes);

  // A is [m, k]: rows m. B is [k, n]: the K-major split of B has rows n.
  int32_t st = launch_split(static_cast<const float*>(g.a), a2, g.m, g.k, g.a_row_stride, g.a_col_stride, stream);
  if (st != B200_OK) return st;
  st = launch_split(static_cast<const float*>(g.b), b2, g.n, g.k, g.b_col_stride, g.b_row_stride, stream);
  if (st != B200_OK) return st;

  b200_gemm_args t = g;
  t.a = a2;
  t.b = b2;
  t.in_dtype = B200_BF16;
  t.k = Kp;  // per pass; the zero padding contributes nothing
  t.a_row_stride = 2 * Kp; t.a_col_stride = 1; t.a_batch_stride = 0;
  t.b_row_stride = 1; t.b_col_stride = 2 * Kp; t.b_batch_stride = 0;  // B^T rows are K-major
  t.route = B200_ROUTE_TCGEN05;
  why = gemm_tcgen05_ineligible(t);
  B200_REQUIRE(why == nullptr, B200_ERR_UNSUPPORTED, "gemm(split): split operands not eligible: %s", why);
  GemmKParts kp;
  kp.parts = 3;
  kp.k_storage = 2 * Kp;
  // smallest terms first: a_hi b_lo, a_lo b_hi, a_hi b_hi
  kp.a_off[0] = 0;          kp.b_off[0] = (int32_t)Kp;
  kp.a_off[1] = (int32_t)Kp; kp.b_off[1] = 0;
  kp.a_off[2] = 0;          kp.b_off[2] = 0;
  return launch_gemm_tcgen05(t, stream, &kp);
}

}  // namespace b200

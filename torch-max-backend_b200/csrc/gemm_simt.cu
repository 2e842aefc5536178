// Generic strided GEMM on CUDA cores: any layout (strides in elements), fp32 or bf16
// operands, fp32 accumulation, fused epilogue. It is the exact-fp32 route and the route for
// shapes/layouts the TMA-fed tensor-core kernel cannot describe (odd strides, unaligned
// pointers, K not a multiple of 8).
//
// Tile 128x128x16 per 256-thread CTA, 8x8 outputs per thread split as 2x2 groups of 4x4 so
// that shared-memory reads are 16-byte vectors without bank conflicts; the next k-slab is
// fetched into registers while the current one is multiplied.
#include "common.cuh"
#include "gemm_internal.cuh"

namespace b200 {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, PAD = 4, THREADS = 256;

template <typename T>
__device__ __forceinline__ float ld_elem(const T* p) { return Elem<T>::to_f32(__ldg(p)); }

struct EpilogueParams {
  const void* bias;
  const void* residual;
  int64_t bias_row_stride, residual_row_stride;
  float alpha, beta;
  int32_t bias_dtype, residual_dtype, epilogue;
};

__device__ __forceinline__ float load_any(const void* p, int64_t idx, int32_t dtype) {
  return dtype == B200_F32 ? __ldg(static_cast<const float*>(p) + idx)
                           : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

__device__ __forceinline__ float apply_epilogue(float acc, int64_t row, int64_t col,
                                                const EpilogueParams& ep) {
  float v = ep.alpha * acc;
  if (ep.bias != nullptr) v += ep.beta * load_any(ep.bias, row * ep.bias_row_stride + col, ep.bias_dtype);
  if (ep.epilogue == B200_EPILOGUE_GELU_TANH) v = gelu_tanh_f32(v);
  else if (ep.epilogue == B200_EPILOGUE_GELU_ERF) v = gelu_erf_f32(v);
  if (ep.residual != nullptr) v += load_any(ep.residual, row * ep.residual_row_stride + col, ep.residual_dtype);
  return v;
}

// A_KFAST: consecutive threads walk k when loading A (use when a_col_stride == 1).
// B_NFAST: consecutive threads walk n when loading B (use when b_col_stride == 1).
template <typename Tin, typename Tout, bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const Tin* __restrict__ A, const Tin* __restrict__ B, Tout* __restrict__ C,
                 int64_t M, int64_t N, int64_t K, int64_t a_rs, int64_t a_cs, int64_t a_bs,
                 int64_t b_rs, int64_t b_cs, int64_t b_bs, int64_t c_rs, int64_t c_bs,
                 EpilogueParams ep) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];

  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int64_t batch = blockIdx.z;
  A += batch * a_bs;
  B += batch * b_bs;
  C += batch * c_bs;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  float ra[8], rb[8];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int m, k;
      if (A_KFAST) { k = t & 15; m = (t >> 4) + 16 * i; }
      else { m = t & 127; k = (t >> 7) + 2 * i; }
      const int64_t gm = m0 + m, gk = k0 + k;
      ra[i] = (gm < M && gk < K) ? ld_elem(A + gm * a_rs + gk * a_cs) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int n, k;
      if (B_NFAST) { n = t & 127; k = (t >> 7) + 2 * i; }
      else { k = t & 15; n = (t >> 4) + 16 * i; }
      const int64_t gn = n0 + n, gk = k0 + k;
      rb[i] = (gn < N && gk < K) ? ld_elem(B + gk * b_rs + gn * b_cs) : 0.0f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int m, k;
      if (A_KFAST) { k = t & 15; m = (t >> 4) + 16 * i; }
      else { m = t & 127; k = (t >> 7) + 2 * i; }
      As[k][m] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int n, k;
      if (B_NFAST) { n = t & 127; k = (t >> 7) + 2 * i; }
      else { k = t & 15; n = (t >> 4) + 16 * i; }
      Bs[k][n] = rb[i];
    }
  };

  fetch(0);
  for (int64_t k0 = 0; k0 < K; k0 += BK) {
    __syncthreads();
    stash();
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (row >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (col >= N) continue;
      C[row * c_rs + col] = Elem<Tout>::from_f32(apply_epilogue(acc[i][j], row, col, ep));
    }
  }
}

template <typename Tin, typename Tout>
int32_t launch(const b200_gemm_args& g, cudaStream_t stream) {
  const int64_t gx = (g.n + BN - 1) / BN, gy = (g.m + BM - 1) / BM;
  B200_REQUIRE(gy <= 65535 && g.batch <= 65535 && gx <= INT32_MAX, B200_ERR_UNSUPPORTED,
               "gemm(simt): grid too large (m=%lld n=%lld batch=%lld)", (long long)g.m,
               (long long)g.n, (long long)g.batch);
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch);
  EpilogueParams ep{g.bias, g.residual, g.bias_row_stride, g.residual_row_stride, g.alpha,
                    g.beta, g.bias_dtype, g.residual_dtype, g.epilogue};
  const bool a_kfast = g.a_col_stride == 1;
  const bool b_nfast = g.b_col_stride == 1;
#define SIMT_LAUNCH(AK, BNF)                                                                   \
  gemm_simt_kernel<Tin, Tout, AK, BNF><<<grid, THREADS, 0, stream>>>(                           \
      static_cast<const Tin*>(g.a), static_cast<const Tin*>(g.b), static_cast<Tout*>(g.c), g.m,  \
      g.n, g.k, g.a_row_stride, g.a_col_stride, g.a_batch_stride, g.b_row_stride,               \
      g.b_col_stride, g.b_batch_stride, g.c_row_stride, g.c_batch_stride, ep)
  if (a_kfast && b_nfast) SIMT_LAUNCH(true, true);
  else if (a_kfast) SIMT_LAUNCH(true, false);
  else if (b_nfast) SIMT_LAUNCH(false, true);
  else SIMT_LAUNCH(false, false);
#undef SIMT_LAUNCH
  B200_CHECK_LAUNCH("gemm(simt)");
  return B200_OK;
}

}  // namespace

int32_t launch_gemm_simt(const b200_gemm_args& g, cudaStream_t stream) {
  if (g.in_dtype == B200_F32)
    return g.out_dtype == B200_F32 ? launch<float, float>(g, stream)
                                   : launch<float, __nv_bfloat16>(g, stream);
  return g.out_dtype == B200_F32 ? launch<__nv_bfloat16, float>(g, stream)
                                 : launch<__nv_bfloat16, __nv_bfloat16>(g, stream);
}

}  // namespace b200

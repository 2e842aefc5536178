// Very small M (decode: one to eight rows of bf16, up to 64 rows of fp32 operands): the weights are read once and the
// arithmetic is a handful of FMAs per weight, so the only question is how many SMs pull on them.
// Stage 1 splits the work over (column block, K slice) CTAs that stream their part of B with 16-byte
// loads, keep M x columns fp32 accumulators in registers and write fp32 partial sums [slices, m, n]
// into scratch; stage 2 (the split-K reduce of gemm_skinny.cu) adds the slices in a fixed order and
// applies the epilogue. Exact fp32 products and fp32 accumulation: for fp32 operands this is also
// the accurate route, and it replaces a 128 x 128-tile kernel that left 127 of 128 rows idle.
//
// With a K-contiguous B and at most eight K slices the two stages are ONE launch: the CTAs of a
// column block's slices form a thread-block cluster, leave their partial sums in shared memory, and
// the cluster's first CTA adds them in slice order out of its peers' shared memory (mapa +
// ld.shared::cluster between two cluster barriers) and applies the epilogue -- no scratch in HBM
// and no second launch, whose latency was a third of the time of a 20 MB weight.
//
// Two stage-1 kernels, by the layout of B:
//   K-contiguous (t() view of an [N, K] weight): a warp owns NW columns, its lanes walk K in 16-byte
//     chunks (so each column is one contiguous stream), A chunks are re-used across the NW columns.
//   N-contiguous ([K, N] weight): a thread owns one 16-byte chunk of columns, a warp 32 of them (512
//     contiguous bytes per k row), the warps of a CTA take alternate k rows and meet in shared memory.
#include "gemm_internal.cuh"
#include "ptx.cuh"

#include <cstdlib>

namespace b200 {
namespace {

constexpr int kMaxRowsBf16 = 8;    // more bf16 rows take the tensor-core split-K stage 1
constexpr int kMaxRowsF32 = 64;    // in row tiles of 16 (B is re-read per tile, from L2 mostly)
constexpr int kRowTile = 16;
constexpr int kThreads = 256;
constexpr int kMaxClusterSlices = 8;  // the portable cluster size

template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ static void load_keep(const float* p, float (&v)[4]) { load16(p, v); }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) { load16_stream(p, v); }
  __device__ static void load_keep(const __nv_bfloat16* p, float (&v)[8]) { load16(p, v); }
};

// What the fused form applies to the summed slices: the arguments of the epilogue.
struct GemvEpilogue {
  const void* bias;
  const void* residual;
  int64_t c_rs, bias_rs, residual_rs;
  float alpha, beta;
  int32_t bias_dtype, residual_dtype, epilogue;
};

__device__ __forceinline__ float ld_any_dtype(const void* p, int64_t idx, int32_t dtype) {
  return dtype == B200_F32 ? __ldg(static_cast<const float*>(p) + idx)
                           : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// ---- B K-contiguous -----------------------------------------------------------------------------
// grid (column groups / warps per CTA, slices, row tiles of M). Requires K % N_vec == 0, 16-byte
// aligned rows. Rows m_total .. of the last row tile are computed on row 0's data and not stored.
// FUSED: the slices of a column block are a cluster (1, slices, 1); the partial sums stay in shared
// memory and the cluster's first CTA writes C. Otherwise they go to `partial` [slices, m, n].
template <typename T, int M, int NW, bool FUSED, typename Tout>
__global__ void __launch_bounds__(kThreads)
gemv_kmajor_kernel(const T* __restrict__ A, const T* __restrict__ B, float* __restrict__ partial, Tout* __restrict__ C,
                   GemvEpilogue e, int64_t n, int64_t k, int64_t a_rs, int64_t b_cs, int64_t k_per_slice, int m_total,
                   int slices) {
  constexpr int V = Vec<T>::N;
  constexpr int kCols = (kThreads / 32) * NW;  // columns of a CTA
  __shared__ float sums[FUSED ? M : 1][FUSED ? kCols : 1];
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.z * M;
  const int m_live = min(M, m_total - m0);
  A += (int64_t)m0 * a_rs;
  const int64_t group = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t n0 = group * NW;
  if (!FUSED && n0 >= n) return;  // (the fused form needs every thread at the cluster barriers)
  const int64_t k_begin = (int64_t)blockIdx.y * k_per_slice;
  const int64_t k_end = n0 < n ? min(k, k_begin + k_per_slice) : k_begin;
  float acc[M][NW];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int c = 0; c < NW; ++c) acc[m][c] = 0.0f;
  for (int64_t kk = k_begin + lane * V; kk < k_end; kk += 32 * V) {
    float b[NW][V];
#pragma unroll
    for (int c = 0; c < NW; ++c) {
      if (n0 + c < n) {
        Vec<T>::load(B + (n0 + c) * b_cs + kk, b[c]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) b[c][j] = 0.0f;
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float a[V];
      Vec<T>::load_keep(A + (m < m_live ? m : 0) * a_rs + kk, a);
#pragma unroll
      for (int c = 0; c < NW; ++c)
#pragma unroll
        for (int j = 0; j < V; ++j) acc[m][c] = fmaf(a[j], b[c][j], acc[m][c]);
    }
  }
  if constexpr (!FUSED) {
    float* out = partial + ((int64_t)blockIdx.y * m_total + m0) * n;
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int c = 0; c < NW; ++c) {
        const float s = warp_sum(acc[m][c]);
        if (lane == 0 && m < m_live && n0 + c < n) out[(int64_t)m * n + n0 + c] = s;
      }
  } else {
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int c = 0; c < NW; ++c) {
        const float s = warp_sum(acc[m][c]);
        if (lane == 0) sums[m][warp * NW + c] = s;
      }
    ptx::cluster_sync();  // every slice's sums are written (release / acquire at cluster scope)
    if (ptx::cluster_ctarank() == 0) {
      // one thread per output element of the column block; slices added in index order, then the
      // epilogue in the order of the two-launch form: alpha, bias, activation, residual
      for (int idx = threadIdx.x; idx < M * kCols; idx += kThreads) {
        const int m = idx / kCols, c = idx - m * kCols;
        const int64_t col = (int64_t)blockIdx.x * kCols + c, row = m0 + m;
        if (m >= m_live || col >= n) continue;
        const uint32_t mine = ptx::smem_u32(&sums[m][c]);
        float total = 0.0f;
        for (int r = 0; r < slices; ++r) total += ld_cluster_f32(ptx::mapa(mine, (uint32_t)r));
        float v = e.alpha * total;
        if (e.bias != nullptr) v += e.beta * ld_any_dtype(e.bias, row * e.bias_rs + col, e.bias_dtype);
        if (e.epilogue == B200_EPILOGUE_GELU_TANH) v = gelu_tanh_f32(v);
        else if (e.epilogue == B200_EPILOGUE_GELU_ERF) v = gelu_erf_f32(v);
        if (e.residual != nullptr) v += ld_any_dtype(e.residual, row * e.residual_rs + col, e.residual_dtype);
        C[row * e.c_rs + col] = Elem<Tout>::from_f32(v);
      }
    }
    ptx::cluster_sync();  // the peers keep their shared memory alive until it has been read
  }
}

// ---- B N-contiguous -----------------------------------------------------------------------------
// grid (column blocks of 32 * V, slices); 8 warps take k rows k_begin + warp, + 8, ... Requires
// n % V == 0 and 16-byte aligned rows of B; A may have any strides.
template <typename T, int M>
__global__ void __launch_bounds__(kThreads)
gemv_nmajor_kernel(const T* __restrict__ A, const T* __restrict__ B, float* __restrict__ partial, int64_t n,
                   int64_t k, int64_t a_rs, int64_t a_cs, int64_t b_rs, int64_t k_per_slice, int m_total) {
  constexpr int V = Vec<T>::N;
  constexpr int kWarps = kThreads / 32;
  extern __shared__ float red[];  // [kWarps][M][32 * V]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m0 = blockIdx.z * M;
  const int m_live = min(M, m_total - m0);
  A += (int64_t)m0 * a_rs;
  const int64_t col = ((int64_t)blockIdx.x * 32 + lane) * V;
  const int64_t k_begin = (int64_t)blockIdx.y * k_per_slice;
  const int64_t k_end = min(k, k_begin + k_per_slice);
  float acc[M][V];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int j = 0; j < V; ++j) acc[m][j] = 0.0f;
  if (col < n) {
    int64_t kk = k_begin + warp;
    // four rows in flight per thread
    for (; kk + 3 * kWarps < k_end; kk += 4 * kWarps) {
      float b[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u) Vec<T>::load(B + (kk + u * kWarps) * b_rs + col, b[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float a = Elem<T>::to_f32(A[(m < m_live ? m : 0) * a_rs + (kk + u * kWarps) * a_cs]);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[m][j] = fmaf(a, b[u][j], acc[m][j]);
        }
    }
    for (; kk < k_end; kk += kWarps) {
      float b[V];
      Vec<T>::load(B + kk * b_rs + col, b);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float a = Elem<T>::to_f32(A[(m < m_live ? m : 0) * a_rs + kk * a_cs]);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[m][j] = fmaf(a, b[j], acc[m][j]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int j = 0; j < V; ++j) red[(warp * M + m) * (32 * V) + lane * V + j] = acc[m][j];
  __syncthreads();
  // warps added in index order: deterministic
  float* out = partial + ((int64_t)blockIdx.y * m_total + m0) * n;
  for (int idx = threadIdx.x; idx < M * 32 * V; idx += kThreads) {
    const int m = idx / (32 * V), c = idx - m * (32 * V);
    const int64_t gc = (int64_t)blockIdx.x * 32 * V + c;
    if (gc >= n || m >= m_live) continue;
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += red[(w * M + m) * (32 * V) + c];
    out[(int64_t)m * n + gc] = s;
  }
}

bool k_contiguous_b(const b200_gemm_args& g) { return g.b_row_stride == 1; }

template <typename T>
const char* ineligible_t(const b200_gemm_args& g) {
  constexpr int V = Vec<T>::N;
  if (k_contiguous_b(g)) {
    if (g.a_col_stride != 1) return "A is not K-contiguous";
    if (g.k % V != 0 || (g.n > 1 && g.b_col_stride % V != 0) || (g.m > 1 && g.a_row_stride % V != 0))
      return "K or a pitch is not a multiple of 16 bytes";
    if (!aligned_to(g.a, 16) || !aligned_to(g.b, 16)) return "operand pointer not 16-byte aligned";
    return nullptr;
  }
  if (g.b_col_stride != 1) return "B has no unit stride";
  // (measured: past one row tile the N-contiguous kernel, which fetches A element by element,
  // loses to the split-precision tensor-core route)
  if (g.m > kRowTile) return "more than 16 rows with an N-contiguous B";
  if (g.n % V != 0 || g.b_row_stride % V != 0) return "N or B's row pitch is not a multiple of 16 bytes";
  if (!aligned_to(g.b, 16)) return "B pointer not 16-byte aligned";
  return nullptr;
}

template <typename T, int M>
int32_t launch_m(const b200_gemm_args& g, float* partial, int slices, cudaStream_t stream) {
  constexpr int V = Vec<T>::N;
  const T* A = static_cast<const T*>(g.a);
  const T* B = static_cast<const T*>(g.b);
  const unsigned row_tiles = (unsigned)((g.m + M - 1) / M);
  if (k_contiguous_b(g)) {
    constexpr int NW = M <= 2 ? 2 : 4;  // A chunks are re-used across NW columns
    const int64_t groups = (g.n + NW - 1) / NW;
    const int64_t gx = (groups + kThreads / 32 - 1) / (kThreads / 32);
    // slices end on a warp-stride boundary so that every lane's chunks stay inside its slice
    int64_t per = (g.k + slices - 1) / slices;
    per = (per + 32 * V - 1) / (32 * V) * (32 * V);
    gemv_kmajor_kernel<T, M, NW, false, float><<<dim3((unsigned)gx, (unsigned)slices, row_tiles), kThreads, 0, stream>>>(
        A, B, partial, nullptr, GemvEpilogue{}, g.n, g.k, g.a_row_stride, g.b_col_stride, per, (int)g.m, slices);
  } else {
    const int64_t gx = (g.n + 32 * V - 1) / (32 * V);
    const int64_t per = (g.k + slices - 1) / slices;
    const size_t smem = (size_t)(kThreads / 32) * M * 32 * V * sizeof(float);
    auto kernel = gemv_nmajor_kernel<T, M>;
    if (smem > 48 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) B200_FAIL(B200_ERR_CUDA, "gemm(gemv): cannot opt in to %zu bytes of shared memory", smem);
    }
    kernel<<<dim3((unsigned)gx, (unsigned)slices, row_tiles), kThreads, smem, stream>>>(
        A, B, partial, g.n, g.k, g.a_row_stride, g.a_col_stride, g.b_row_stride, per, (int)g.m);
  }
  B200_CHECK_LAUNCH("gemm(gemv)");
  return B200_OK;
}

// The one-launch form: grid (column blocks, slices, row tiles) in clusters of (1, slices, 1).
template <typename T, int M, typename Tout>
int32_t launch_fused_m(const b200_gemm_args& g, int slices, cudaStream_t stream) {
  constexpr int V = Vec<T>::N;
  constexpr int NW = M <= 2 ? 2 : 4;
  const int64_t groups = (g.n + NW - 1) / NW;
  const int64_t gx = (groups + kThreads / 32 - 1) / (kThreads / 32);
  int64_t per = (g.k + slices - 1) / slices;
  per = (per + 32 * V - 1) / (32 * V) * (32 * V);
  GemvEpilogue e;
  e.bias = g.bias; e.residual = g.residual;
  e.c_rs = g.c_row_stride; e.bias_rs = g.bias_row_stride; e.residual_rs = g.residual_row_stride;
  e.alpha = g.alpha; e.beta = g.beta;
  e.bias_dtype = g.bias_dtype; e.residual_dtype = g.residual_dtype; e.epilogue = g.epilogue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)gx, (unsigned)slices, (unsigned)((g.m + M - 1) / M));
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)slices;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(
      &cfg, gemv_kmajor_kernel<T, M, NW, true, Tout>, static_cast<const T*>(g.a), static_cast<const T*>(g.b),
      static_cast<float*>(nullptr), static_cast<Tout*>(g.c), e, g.n, g.k, g.a_row_stride, g.b_col_stride, per, (int)g.m,
      slices);
  if (err != cudaSuccess) B200_FAIL(B200_ERR_CUDA, "gemm(gemv, one launch): launch failed: %s", cudaGetErrorString(err));
  return B200_OK;
}

template <typename T, typename Tout>
int32_t launch_fused_t(const b200_gemm_args& g, int slices, cudaStream_t stream) {
  if (g.m <= 1) return launch_fused_m<T, 1, Tout>(g, slices, stream);
  if (g.m <= 2) return launch_fused_m<T, 2, Tout>(g, slices, stream);
  if (g.m <= 4) return launch_fused_m<T, 4, Tout>(g, slices, stream);
  if (g.m <= 8 || sizeof(T) == 2) return launch_fused_m<T, 8, Tout>(g, slices, stream);
  if constexpr (sizeof(T) == 4) return launch_fused_m<T, kRowTile, Tout>(g, slices, stream);
  return B200_ERR_UNSUPPORTED;
}

// Row tile: the smallest of 1, 2, 4, 8 (and 16 for fp32) that holds m, else tiles of the largest.
template <typename T>
int32_t launch_t(const b200_gemm_args& g, float* partial, int slices, cudaStream_t stream) {
  if (g.m <= 1) return launch_m<T, 1>(g, partial, slices, stream);
  if (g.m <= 2) return launch_m<T, 2>(g, partial, slices, stream);
  if (g.m <= 4) return launch_m<T, 4>(g, partial, slices, stream);
  if (g.m <= 8 || sizeof(T) == 2) return launch_m<T, 8>(g, partial, slices, stream);
  if constexpr (sizeof(T) == 4) return launch_m<T, kRowTile>(g, partial, slices, stream);
  return B200_ERR_UNSUPPORTED;
}

}  // namespace

const char* gemm_gemv_ineligible(const b200_gemm_args& g) {
  if (g.batch != 1) return "batched";
  if (g.m <= 0 || g.m > (g.in_dtype == B200_F32 ? kMaxRowsF32 : kMaxRowsBf16))
    return g.in_dtype == B200_F32 ? "more than 64 rows" : "more than 8 rows";
  if (g.k <= 0) return "k is zero";
  return g.in_dtype == B200_F32 ? ineligible_t<float>(g) : ineligible_t<__nv_bfloat16>(g);
}

// K slices: enough CTAs to put a few on every SM, never slices shorter than 256 elements of K.
int gemm_gemv_slices(const b200_gemm_args& g) {
  const int vec = g.in_dtype == B200_F32 ? 4 : 8;
  int64_t ctas_x, by_k;
  if (g.b_row_stride == 1) {
    const int nw = g.m <= 2 ? 2 : 4;
    ctas_x = ((g.n + nw - 1) / nw + 7) / 8;
    by_k = g.k / (32 * vec);  // a warp covers 32 chunks of K per step
  } else {
    ctas_x = (g.n + 32 * vec - 1) / (32 * vec);
    by_k = g.k / 32;          // the 8 warps of a CTA take alternate k rows, four in flight each
  }
  ctas_x *= (g.m + kRowTile - 1) / kRowTile;
  const int64_t want = 4 * (int64_t)sm_count();
  int64_t s = (want + ctas_x - 1) / ctas_x;
  if (s > by_k) s = by_k;
  if (s > 64) s = 64;
  if (g.b_row_stride == 1 && s > kMaxClusterSlices) s = kMaxClusterSlices;  // the one-launch form: a portable cluster
  if (s < 1) s = 1;
  return (int)s;
}

// A K-contiguous B takes the one-launch form (no scratch) while its grid is about one wave of CTAs:
// measured 1.1 - 1.5 us faster than two launches on weights of 1 - 15 MB (3.2 - 4.5 us instead of
// 4.7 - 5.5), equal around 20 - 40 MB, and slower once clusters queue for a second wave (bf16
// 1 x 1600 x 6400, 800 CTAs: 11.8 against 9.3 us), where the two launches stay.
// (B200_GEMV_ONE_LAUNCH=0, read once, keeps the two-launch form everywhere: for measurements.)
bool gemm_gemv_one_launch(const b200_gemm_args& g) {
  static const bool enabled = [] {
    const char* v = getenv("B200_GEMV_ONE_LAUNCH");
    return v == nullptr || atoi(v) != 0;
  }();
  if (!enabled || g.b_row_stride != 1) return false;
  const int nw = g.m <= 2 ? 2 : 4;
  const int64_t column_blocks = ((g.n + nw - 1) / nw + kThreads / 32 - 1) / (kThreads / 32);
  const int64_t row_tiles = g.in_dtype == B200_F32 && g.m > 8 ? (g.m + kRowTile - 1) / kRowTile : 1;
  return column_blocks * gemm_gemv_slices(g) * row_tiles <= 5 * (int64_t)sm_count();
}

size_t gemm_gemv_scratch_bytes(const b200_gemm_args& g) {
  if (gemm_gemv_one_launch(g)) return 0;
  return (size_t)gemm_gemv_slices(g) * (size_t)g.m * (size_t)g.n * sizeof(float);
}

int32_t launch_gemm_gemv_one_launch(const b200_gemm_args& g, cudaStream_t stream) {
  const int slices = gemm_gemv_slices(g);
  const bool f32_out = g.out_dtype == B200_F32;
  if (g.in_dtype == B200_F32)
    return f32_out ? launch_fused_t<float, float>(g, slices, stream) : launch_fused_t<float, __nv_bfloat16>(g, slices, stream);
  return f32_out ? launch_fused_t<__nv_bfloat16, float>(g, slices, stream)
                 : launch_fused_t<__nv_bfloat16, __nv_bfloat16>(g, slices, stream);
}

int32_t launch_gemm_gemv_partials(const b200_gemm_args& g, float* partial, int slices, cudaStream_t stream) {
  return g.in_dtype == B200_F32 ? launch_t<float>(g, partial, slices, stream)
                                : launch_t<__nv_bfloat16>(g, partial, slices, stream);
}

}  // namespace b200

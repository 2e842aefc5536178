// Bandwidth-bound row kernels: LayerNorm, row softmax, GELU, trailing-dim reductions.
//
// Fast paths keep one row per warp in registers (one HBM read, one HBM write per element),
// move data as 16-byte vectors and reduce with warp shuffles. Rows that do not fit the
// register budget, or whose pointers/strides are not 16-byte friendly, take a CTA-per-row
// kernel with scalar accesses.
#include "common.cuh"

#include <cstdlib>

namespace b200 {
namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kRowThreads = kWarpsPerCta * 32;

// ---- chunk load/store: N consecutive elements of T <-> N fp32 lanes ----------------------
template <typename T, int N>
struct Chunk;

template <>
struct Chunk<float, 4> {
  __device__ static void load(const float* p, float (&v)[4]) { load16_stream(p, v); }
  __device__ static void load_keep(const float* p, float (&v)[4]) { load16(p, v); }
  __device__ static void store(float* p, const float (&v)[4]) { store16_stream(p, v); }
};

template <>
struct Chunk<float, 8> {
  __device__ static void load(const float* p, float (&v)[8]) {
    float a[4], b[4];
    load16_stream(p, a);
    load16_stream(p + 4, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[i] = a[i]; v[4 + i] = b[i]; }
  }
  __device__ static void load_keep(const float* p, float (&v)[8]) {
    float a[4], b[4];
    load16(p, a);
    load16(p + 4, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[i] = a[i]; v[4 + i] = b[i]; }
  }
  __device__ static void store(float* p, const float (&v)[8]) {
    float a[4] = {v[0], v[1], v[2], v[3]}, b[4] = {v[4], v[5], v[6], v[7]};
    store16_stream(p, a);
    store16_stream(p + 4, b);
  }
};

template <>
struct Chunk<__nv_bfloat16, 8> {
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) { load16_stream(p, v); }
  __device__ static void load_keep(const __nv_bfloat16* p, float (&v)[8]) { load16(p, v); }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) { store16_stream(p, v); }
};

template <>
struct Chunk<__nv_bfloat16, 4> {
  __device__ static void load(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  }
  __device__ static void load_keep(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 t;
    t.x = pack_bf16x2(v[0], v[1]);
    t.y = pack_bf16x2(v[2], v[3]);
    __stcs(reinterpret_cast<uint2*>(p), t);
  }
};

// CTA-wide reductions for the generic kernels (blockDim.x <= 1024, a multiple of 32).
__device__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? smem[lane] : 0.0f;
  return warp_sum(t);
}

__device__ float block_max(float v, float* smem) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? smem[lane] : -INFINITY;
  return warp_max(t);
}

// =========================================================================================
// LayerNorm
// =========================================================================================

// 16 raw bytes of a row (N elements of Tin) -> N fp32 values.
template <typename Tin, int N>
__device__ __forceinline__ void unpack_raw(const uint4& t, float (&v)[N]) {
  if constexpr (sizeof(Tin) == 2) {
    static_assert(sizeof(Tin) != 2 || N == 8, "16 bytes of bf16");
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
    static_assert(sizeof(Tin) != 4 || N == 4, "16 bytes of fp32");
    v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y);
    v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
  }
}

// CTAs of a warp-per-row kernel whose warps walk rows with a grid stride and prefetch their next
// row: one row per warp while that fills the GPU less than 32 CTAs per SM deep, then up to
// rows_per_warp rows per warp so that the prefetch has something to overlap.
unsigned prefetching_grid(int64_t rows, int rows_per_warp) {
  const int64_t ctas_1 = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  const int64_t ctas_r = (ctas_1 + rows_per_warp - 1) / rows_per_warp;
  const int64_t floor_ctas = (int64_t)sm_count() * 32;
  return (unsigned)(ctas_1 <= floor_ctas ? ctas_1 : (ctas_r > floor_ctas ? ctas_r : floor_ctas));
}

// One warp per row; the row lives in registers between the three uses (mean, variance,
// normalise). N = elements per chunk (16 bytes of Tin), MAXC = chunks per lane. A warp walks rows
// with a grid stride and issues the 16-byte loads of its NEXT row as soon as the current one is
// unpacked, so the loads overlap the two reductions and the stores.
template <typename Tin, typename Tp, typename Tout, int N, int MAXC>
__global__ void __launch_bounds__(kRowThreads)
layer_norm_warp_kernel(const Tin* __restrict__ x, const Tp* __restrict__ gamma,
                       const Tp* __restrict__ beta, Tout* __restrict__ y,
                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows,
                       int cols, int64_t x_row_stride, float eps) {
  static_assert(N * sizeof(Tin) == 16, "one chunk is one 16-byte load");
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerCta;
  int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nchunks = cols / N;
  uint4 raw[MAXC];
  auto fetch = [&](int64_t r) {
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunks) raw[i] = __ldcs(reinterpret_cast<const uint4*>(x + r * x_row_stride + c * N));
    }
  };
  fetch(row);
  while (true) {
  // The three uses of the row run on packed fp32 instructions (two elements per add / mul /
  // fma): at power-capped clocks the narrow-type variants are bound by instruction issue, not HBM.
  float v[MAXC][N];
  float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunks) {
      unpack_raw<Tin, N>(raw[i], v[i]);
#pragma unroll
      for (int j = 0; j < N; j += 2) sum2 = __fadd2_rn(sum2, make_float2(v[i][j], v[i][j + 1]));
    }
  }
  const int64_t next = row + stride;
  if (next < rows) fetch(next);
  const float mean = warp_sum(sum2.x + sum2.y) / (float)cols;
  const float2 neg_mean2 = make_float2(-mean, -mean);
  float2 sq2 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunks) {
#pragma unroll
      for (int j = 0; j < N; j += 2) {
        const float2 d = __fadd2_rn(make_float2(v[i][j], v[i][j + 1]), neg_mean2);
        v[i][j] = d.x;  // keep the centred value: the last pass starts from it
        v[i][j + 1] = d.y;
        sq2 = __ffma2_rn(d, d, sq2);
      }
    }
  }
  const float var = warp_sum(sq2.x + sq2.y) / (float)cols;
  const float rstd = 1.0f / sqrtf(var + eps);
  const float2 rstd2 = make_float2(rstd, rstd);

  Tout* yr = y + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunks) {
      float g[N], b[N], o[N];
      if (gamma != nullptr) {
        Chunk<Tp, N>::load_keep(gamma + c * N, g);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) g[j] = 1.0f;
      }
      if (beta != nullptr) {
        Chunk<Tp, N>::load_keep(beta + c * N, b);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) b[j] = 0.0f;
      }
#pragma unroll
      for (int j = 0; j < N; j += 2) {
        const float2 t = __fmul2_rn(make_float2(v[i][j], v[i][j + 1]), rstd2);
        const float2 r = __ffma2_rn(t, make_float2(g[j], g[j + 1]), make_float2(b[j], b[j + 1]));
        o[j] = r.x;
        o[j + 1] = r.y;
      }
      Chunk<Tout, N>::store(yr + c * N, o);
    }
  }
  if (lane == 0) {
    if (mean_out != nullptr) mean_out[row] = mean;
    if (rstd_out != nullptr) rstd_out[row] = rstd;
  }
  if (next >= rows) break;
  row = next;
  }
}

// The same computation with WPR warps per row: each lane keeps 1/WPR of the chunks (fewer registers
// per thread, more resident warps, and the loads of a row are spread over more warps) and the partial
// sums of a row's warps meet in shared memory. The loop over row groups is there for grids smaller
// than the number of groups; launching one CTA per group measured faster than a persistent grid
// (fresh CTAs overlap one group's loads with another's arithmetic, a looping CTA serialises them).
constexpr int kLnWarps = 8;
template <typename Tin, typename Tp, typename Tout, int N, int MAXC, int WPR>
__global__ void __launch_bounds__(kLnWarps * 32)
layer_norm_rows_kernel(const Tin* __restrict__ x, const Tp* __restrict__ gamma,
                       const Tp* __restrict__ beta, Tout* __restrict__ y,
                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows,
                       int cols, int64_t x_row_stride, float eps) {
  constexpr int kRowsPerCta = kLnWarps / WPR;
  __shared__ float part[2][kLnWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = warp % WPR;        // which share of the row this warp holds
  const int slot = warp / WPR;       // which of the CTA's rows
  const int nchunks = cols / N;
  const int64_t groups = (rows + kRowsPerCta - 1) / kRowsPerCta;
  for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int64_t row = grp * kRowsPerCta + slot;
    const bool live = row < rows;
    const Tin* xr = x + (live ? row : 0) * x_row_stride;
    float v[MAXC][N];
    float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * (sub + WPR * i);
      if (live && c < nchunks) {
        Chunk<Tin, N>::load(xr + c * N, v[i]);
#pragma unroll
        for (int j = 0; j < N; j += 2) sum2 = __fadd2_rn(sum2, make_float2(v[i][j], v[i][j + 1]));
      }
    }
    float total = warp_sum(sum2.x + sum2.y);
    if (WPR > 1) {
      if (lane == 0) part[0][warp] = total;
      __syncthreads();
      total = 0.0f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) total += part[0][slot * WPR + w];
    }
    const float mean = total / (float)cols;
    const float2 neg_mean2 = make_float2(-mean, -mean);
    float2 sq2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * (sub + WPR * i);
      if (live && c < nchunks) {
#pragma unroll
        for (int j = 0; j < N; j += 2) {
          const float2 d = __fadd2_rn(make_float2(v[i][j], v[i][j + 1]), neg_mean2);
          v[i][j] = d.x;
          v[i][j + 1] = d.y;
          sq2 = __ffma2_rn(d, d, sq2);
        }
      }
    }
    float sq = warp_sum(sq2.x + sq2.y);
    if (WPR > 1) {
      if (lane == 0) part[1][warp] = sq;
      __syncthreads();  // also orders this row's reads of part[0] before the next row's writes
      sq = 0.0f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) sq += part[1][slot * WPR + w];
    }
    const float rstd = 1.0f / sqrtf(sq / (float)cols + eps);
    const float2 rstd2 = make_float2(rstd, rstd);
    Tout* yr = y + (live ? row : 0) * (int64_t)cols;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * (sub + WPR * i);
      if (live && c < nchunks) {
        float g[N], b[N], o[N];
        if (gamma != nullptr) {
          Chunk<Tp, N>::load_keep(gamma + c * N, g);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) g[j] = 1.0f;
        }
        if (beta != nullptr) {
          Chunk<Tp, N>::load_keep(beta + c * N, b);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) b[j] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < N; j += 2) {
          const float2 t = __fmul2_rn(make_float2(v[i][j], v[i][j + 1]), rstd2);
          const float2 r = __ffma2_rn(t, make_float2(g[j], g[j + 1]), make_float2(b[j], b[j + 1]));
          o[j] = r.x;
          o[j + 1] = r.y;
        }
        Chunk<Tout, N>::store(yr + c * N, o);
      }
    }
    if (live && lane == 0 && sub == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      if (rstd_out != nullptr) rstd_out[row] = rstd;
    }
    if (WPR > 1) __syncthreads();  // part[1] is read before the next row overwrites it
  }
}

// Generic: one CTA per row, scalar accesses, three passes over the row (L1/L2 serve the
// re-reads).
template <typename Tin, typename Tp, typename Tout>
__global__ void layer_norm_block_kernel(const Tin* __restrict__ x, const Tp* __restrict__ gamma,
                                        const Tp* __restrict__ beta, Tout* __restrict__ y,
                                        float* __restrict__ mean_out,
                                        float* __restrict__ rstd_out, int64_t cols,
                                        int64_t x_row_stride, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const Tin* xr = x + row * x_row_stride;
  float s = 0.0f;
  for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) s += Elem<Tin>::to_f32(xr[j]);
  const float mean = block_sum(s, red) / (float)cols;
  float sq = 0.0f;
  for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
    const float d = Elem<Tin>::to_f32(xr[j]) - mean;
    sq += d * d;
  }
  const float var = block_sum(sq, red) / (float)cols;
  const float rstd = 1.0f / sqrtf(var + eps);
  Tout* yr = y + row * cols;
  for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
    const float g = gamma != nullptr ? Elem<Tp>::to_f32(gamma[j]) : 1.0f;
    const float b = beta != nullptr ? Elem<Tp>::to_f32(beta[j]) : 0.0f;
    yr[j] = Elem<Tout>::from_f32((Elem<Tin>::to_f32(xr[j]) - mean) * rstd * g + b);
  }
  if (threadIdx.x == 0) {
    if (mean_out != nullptr) mean_out[row] = mean;
    if (rstd_out != nullptr) rstd_out[row] = rstd;
  }
}

template <typename Tin, typename Tp, typename Tout>
int32_t launch_layer_norm(const void* x, const void* gamma, const void* beta, void* y,
                          float* mean, float* rstd, int64_t rows, int64_t cols,
                          int64_t x_row_stride, float eps, cudaStream_t stream) {
  constexpr int N = Elem<Tin>::kVec;
  const Tin* xp = static_cast<const Tin*>(x);
  const Tp* gp = static_cast<const Tp*>(gamma);
  const Tp* bp = static_cast<const Tp*>(beta);
  Tout* yp = static_cast<Tout*>(y);
  const size_t out_align = N * sizeof(Tout) > 16 ? 16 : N * sizeof(Tout);
  const size_t p_align = N * sizeof(Tp) > 16 ? 16 : N * sizeof(Tp);
  const bool vec_ok = cols % N == 0 && x_row_stride % N == 0 && aligned_to(x, 16) &&
                      aligned_to(y, out_align) && (gamma == nullptr || aligned_to(gamma, p_align)) &&
                      (beta == nullptr || aligned_to(beta, p_align)) && cols <= 32 * N * 16 &&
                      rows <= (int64_t)INT32_MAX * kWarpsPerCta;
  if (vec_ok) {
    const int per_lane = (int)((cols / N + 31) / 32);
    if (per_lane > 8) {
      // Wide rows (more than 8 chunks per lane, e.g. 1600 fp32 columns): two warps per row. Measured
      // on [65536, 1600] fp32 -> bf16: 1.00 of the copy bandwidth against 0.90 with one warp per row
      // (half the registers per thread, twice the resident warps); narrower rows measured no gain.
      constexpr int kRowsPerCta = kLnWarps / 2;
      const int64_t groups = (rows + kRowsPerCta - 1) / kRowsPerCta;
      B200_REQUIRE(groups <= INT32_MAX, B200_ERR_UNSUPPORTED, "layer_norm: too many rows");
      const unsigned grid2 = (unsigned)groups;
      const int share = (per_lane + 1) / 2;
#define LNR(MAXC) layer_norm_rows_kernel<Tin, Tp, Tout, N, MAXC, 2><<<grid2, kLnWarps * 32, 0, stream>>>( \
      xp, gp, bp, yp, mean, rstd, rows, (int)cols, x_row_stride, eps)
      if (share <= 5) LNR(5); else if (share <= 7) LNR(7); else LNR(8);
#undef LNR
      B200_CHECK_LAUNCH("layer_norm");
      return B200_OK;
    }
    const unsigned grid = prefetching_grid(rows, 4);
#define LN_LAUNCH(MAXC)                                                                   \
  layer_norm_warp_kernel<Tin, Tp, Tout, N, MAXC><<<grid, kRowThreads, 0, stream>>>(         \
      xp, gp, bp, yp, mean, rstd, rows, (int)cols, x_row_stride, eps)
    if (per_lane <= 1) LN_LAUNCH(1);
    else if (per_lane <= 2) LN_LAUNCH(2);
    else if (per_lane <= 4) LN_LAUNCH(4);
    else if (per_lane <= 8) LN_LAUNCH(8);
    else LN_LAUNCH(16);
#undef LN_LAUNCH
  } else {
    B200_REQUIRE(rows <= INT32_MAX, B200_ERR_UNSUPPORTED, "layer_norm: too many rows");
    const int threads = cols >= 1024 ? 512 : 128;
    layer_norm_block_kernel<Tin, Tp, Tout><<<(unsigned)rows, threads, 0, stream>>>(
        xp, gp, bp, yp, mean, rstd, cols, x_row_stride, eps);
  }
  B200_CHECK_LAUNCH("layer_norm");
  return B200_OK;
}

// =========================================================================================
// Softmax over the last dim
// =========================================================================================

// Optional element mask of the fused scale + masked_fill + softmax form: row r of x uses mask row
// r % rows (a [T, S] mask broadcast over batch and heads); an element is replaced by `fill`
// where (mask byte != 0) != invert. ptr == nullptr: no mask.
struct RowMask {
  const uint8_t* ptr;
  int64_t rows, stride;
  int invert;
  float fill;
};

// One warp per row, the row in registers; a warp walks rows with a grid stride and issues the
// 16-byte loads of its NEXT row before it reduces the current one, so every resident warp keeps a
// row of loads in flight through its arithmetic and store phases (without that the kernel waits
// on memory latency at half the copy bandwidth). Values are moved to the base-2 exponent domain
// when they are unpacked (x * scale * log2(e)), so each element costs one subtract and one ex2
// between the two reductions; masking is decided per 16-byte chunk and only chunks that straddle
// the causal limit (or rows that carry an explicit mask) look at single elements. A masked element
// is -inf, which the exponential turns into an exact 0; a row with nothing visible gives NaN like
// torch.
// Registers that hold row data: the fp32 row, the raw next row and its mask bytes. The launch bound
// asks for as many resident CTAs as leave those plus ~30 working registers per thread.
constexpr int softmax_min_ctas(int n, int maxc, bool has_mask) {
  const int live = maxc * n + maxc * 4 + (has_mask ? maxc * 2 : 0);
  return live < 56 ? 6 : (live <= 72 ? 5 : 3);
}

template <typename Tin, typename Tout, int N, int MAXC, bool HAS_MASK>
__global__ void __launch_bounds__(kRowThreads, softmax_min_ctas(N, MAXC, HAS_MASK))
softmax_warp_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, int64_t rows, int cols,
                    int64_t x_row_stride, float scale, int causal, int64_t q_len, RowMask mask) {
  static_assert(N * sizeof(Tin) == 16, "one chunk is one 16-byte load");
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerCta;
  int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nchunks = cols / N;
  constexpr float kLog2e = 1.4426950408889634f;
  const float sl = scale * kLog2e;
  const float fill2 = mask.fill * kLog2e;
  constexpr bool has_mask = HAS_MASK;

  uint4 raw[MAXC];
  uint64_t mraw[HAS_MASK ? MAXC : 1];
  auto limit_of = [&](int64_t r) {
    if (!causal) return cols;
    const int64_t a = r % q_len + 1;
    return a < cols ? (int)a : cols;
  };
  // Chunks entirely past the causal limit are never read.
  auto fetch = [&](int64_t r, int allowed) {
    const Tin* xr = x + r * x_row_stride;
    const uint8_t* mr = has_mask ? mask.ptr + (r % mask.rows) * mask.stride : nullptr;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunks && c * N < allowed) {
        raw[i] = __ldcs(reinterpret_cast<const uint4*>(xr + c * N));
        // N mask bytes of this chunk (the launcher guarantees N-byte alignment of every chunk)
        if constexpr (has_mask)
          mraw[i] = N == 8 ? *reinterpret_cast<const uint64_t*>(mr + c * N)
                           : (uint64_t) * reinterpret_cast<const uint32_t*>(mr + c * N);
      }
    }
  };

  int allowed = limit_of(row);
  fetch(row, allowed);
  while (true) {
    float v[MAXC][N];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunks && c * N < allowed) {
        unpack_raw<Tin, N>(raw[i], v[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) v[i][j] *= sl;
        if (c * N + N > allowed) {  // the chunk that straddles the limit
#pragma unroll
          for (int j = 0; j < N; ++j)
            if (c * N + j >= allowed) v[i][j] = -INFINITY;
        }
        if constexpr (has_mask) {
          const uint64_t mbits = mraw[i];
#pragma unroll
          for (int j = 0; j < N; ++j)
            if ((((mbits >> (8 * j)) & 0xffu) != 0) != (mask.invert != 0)) v[i][j] = fill2;
        }
#pragma unroll
        for (int j = 0; j < N; ++j) m = nan_max(m, v[i][j]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[i][j] = -INFINITY;
      }
    }
    const int64_t next = row + stride;
    const int next_allowed = next < rows ? limit_of(next) : 0;
    if (next < rows) fetch(next, next_allowed);

    m = warp_max(m);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        float e;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v[i][j] - m));
        v[i][j] = e;
        s += e;
      }
    }
    s = warp_sum(s);
    const float inv = 1.0f / s;
    Tout* yr = y + row * (int64_t)cols;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunks) {
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = v[i][j] * inv;
        Chunk<Tout, N>::store(yr + c * N, o);
      }
    }
    if (next >= rows) break;
    row = next;
    allowed = next_allowed;
  }
}

template <typename Tin, typename Tout>
__global__ void softmax_block_kernel(const Tin* __restrict__ x, Tout* __restrict__ y,
                                     int64_t cols, int64_t x_row_stride, float scale, int causal,
                                     int64_t q_len, RowMask mask) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  int64_t allowed = cols;
  if (causal) {
    const int64_t a = row % q_len + 1;
    allowed = a < cols ? a : cols;
  }
  const Tin* xr = x + row * x_row_stride;
  const uint8_t* mr = mask.ptr != nullptr ? mask.ptr + (row % mask.rows) * mask.stride : nullptr;
  auto value = [&](int64_t j) {
    if (mr != nullptr && (mr[j] != 0) != (mask.invert != 0)) return mask.fill;
    return Elem<Tin>::to_f32(xr[j]) * scale;
  };
  float m = -INFINITY;
  for (int64_t j = threadIdx.x; j < allowed; j += blockDim.x) m = nan_max(m, value(j));
  m = block_max(m, red);
  float s = 0.0f;
  for (int64_t j = threadIdx.x; j < allowed; j += blockDim.x) s += expf(value(j) - m);
  s = block_sum(s, red);
  const float inv = 1.0f / s;
  Tout* yr = y + row * cols;
  for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
    const float o = j < allowed ? expf(value(j) - m) * inv : 0.0f;
    yr[j] = Elem<Tout>::from_f32(o);
  }
}

int softmax_rows_per_warp() {
  static const int r = [] {
    const char* e = std::getenv("B200_SOFTMAX_ROWS_PER_WARP");
    const int v = e != nullptr ? std::atoi(e) : 0;
    return v >= 1 && v <= 64 ? v : 4;
  }();
  return r;
}

template <typename Tin, typename Tout>
int32_t launch_softmax(const void* x, void* y, int64_t rows, int64_t cols, int64_t x_row_stride,
                       float scale, int causal, int64_t q_len, RowMask mask, cudaStream_t stream) {
  constexpr int N = Elem<Tin>::kVec;
  const Tin* xp = static_cast<const Tin*>(x);
  Tout* yp = static_cast<Tout*>(y);
  const size_t out_align = N * sizeof(Tout) > 16 ? 16 : N * sizeof(Tout);
  const bool vec_ok = cols % N == 0 && x_row_stride % N == 0 && aligned_to(x, 16) &&
                      aligned_to(y, out_align) && cols <= 32 * N * 8 &&
                      rows <= (int64_t)INT32_MAX * kWarpsPerCta &&
                      (mask.ptr == nullptr || (aligned_to(mask.ptr, N) && mask.stride % N == 0));
  if (vec_ok) {
    const int per_lane = (int)((cols / N + 31) / 32);
    const unsigned grid = prefetching_grid(rows, softmax_rows_per_warp());
#define SM_LAUNCH(MAXC)                                                                      \
  do {                                                                                       \
    if (mask.ptr != nullptr)                                                                 \
      softmax_warp_kernel<Tin, Tout, N, MAXC, true><<<grid, kRowThreads, 0, stream>>>(       \
          xp, yp, rows, (int)cols, x_row_stride, scale, causal, q_len, mask);                \
    else                                                                                     \
      softmax_warp_kernel<Tin, Tout, N, MAXC, false><<<grid, kRowThreads, 0, stream>>>(      \
          xp, yp, rows, (int)cols, x_row_stride, scale, causal, q_len, mask);                \
  } while (0)
    if (per_lane <= 1) SM_LAUNCH(1);
    else if (per_lane <= 2) SM_LAUNCH(2);
    else if (per_lane <= 4) SM_LAUNCH(4);
    else SM_LAUNCH(8);
#undef SM_LAUNCH
  } else {
    B200_REQUIRE(rows <= INT32_MAX, B200_ERR_UNSUPPORTED, "softmax: too many rows");
    const int threads = cols >= 2048 ? 1024 : (cols >= 512 ? 256 : 128);
    softmax_block_kernel<Tin, Tout><<<(unsigned)rows, threads, 0, stream>>>(
        xp, yp, cols, x_row_stride, scale, causal, q_len, mask);
  }
  B200_CHECK_LAUNCH("softmax_lastdim");
  return B200_OK;
}

// =========================================================================================
// GELU
// =========================================================================================

// tanh form rewritten as x * sigmoid(2u): 0.5 x (1 + tanh(u)) == x / (1 + exp(-2u)).
// Signed zero, +inf (-> +inf) and -inf / NaN (-> NaN) come out as torch's formula gives them.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  return x / (1.0f + expf(-2.0f * u));
}

// The same formula on two MUFU operations (ex2.approx, rcp.approx: relative error ~2^-22) instead of
// a full-precision expf and an IEEE division (a dozen instructions each): used for bf16 tensors, whose
// 8-bit significand the approximation cannot move, and what makes that kernel HBM-bound instead of
// issue-bound. x == +inf gives +inf (inf * 1), -inf and NaN give NaN, like the exact form.
__device__ __forceinline__ float gelu_tanh_mufu(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-2.885390081777927f * u));  // exp(-2u)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// erf form for two bf16-bound values at once: 0.5 x (1 + erf(x / sqrt 2)) = x * (x < 0 ? h : 1 - h) with
//   h = 0.5 erfc(|x| / sqrt 2) = t Q(t) exp(-x^2 / 2),   t = 1 / (1 + |x| / (2 sqrt 2)),
// Q a degree-7 minimax fit (relative error of h 3.1e-6, a hundredth of a bf16 rounding step; over all
// 65536 bf16 inputs the rounded result equals the correctly rounded one wherever the exact result is
// a normal number). Two MUFU operations and packed two-wide FMAs per element in place of erff's two
// polynomial branches, which is what lets the bf16 kernel run at memory speed. Because h keeps its
// relative accuracy in the left tail, x < -5.6 gives the tiny true value where the fp32 formula's
// 1 + erf cancels to -0. +inf -> +inf (inf * 1), -inf -> NaN (-inf * 0), NaN -> NaN, +-0 -> +-0.
__device__ __forceinline__ float2 gelu_erf_pair(float2 x) {
  const float kHalfInvSqrt2 = 0.35355339059327373f;
  float2 t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.x) : "f"(fmaf(fabsf(x.x), kHalfInvSqrt2, 1.0f)));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.y) : "f"(fmaf(fabsf(x.y), kHalfInvSqrt2, 1.0f)));
  constexpr float q[8] = {1.410478354e-01f, 1.409928650e-01f, 1.244906485e-01f, 8.064989746e-02f,
                          6.382267177e-02f, -2.228422835e-02f, -5.376151577e-02f, 2.504315786e-02f};
  float2 acc = make_float2(q[7], q[7]);
#pragma unroll
  for (int i = 6; i >= 0; --i) acc = __ffma2_rn(acc, t, make_float2(q[i], q[i]));
  const float kNegHalfLog2e = -0.7213475204444817f;
  const float2 arg = __fmul2_rn(__fmul2_rn(x, x), make_float2(kNegHalfLog2e, kNegHalfLog2e));
  float2 e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(arg.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(arg.y));
  const float2 h = __fmul2_rn(__fmul2_rn(t, acc), e);
  float2 w = __ffma2_rn(h, make_float2(-1.0f, -1.0f), make_float2(1.0f, 1.0f));
  w.x = x.x < 0.0f ? h.x : w.x;
  w.y = x.y < 0.0f ? h.y : w.y;
  return __fmul2_rn(x, w);
}

template <typename T>
__device__ __forceinline__ float gelu_tanh_for(float x) {
  return sizeof(T) == 2 ? gelu_tanh_mufu(x) : gelu_tanh_fast(x);
}

constexpr int kGeluUnroll = 4;
constexpr int kGeluThreads = 256;

template <typename T, bool kTanh>
__global__ void __launch_bounds__(kGeluThreads)
gelu_vec_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t nvec) {
  constexpr int N = Elem<T>::kVec;
  // Each CTA owns kGeluUnroll consecutive slabs of blockDim vectors; all loads issue first.
  const int64_t base = (int64_t)blockIdx.x * (kGeluThreads * kGeluUnroll) + threadIdx.x;
  float v[kGeluUnroll][N];
#pragma unroll
  for (int u = 0; u < kGeluUnroll; ++u) {
    const int64_t i = base + (int64_t)u * kGeluThreads;
    if (i < nvec) load16_stream(x + i * N, v[u]);
  }
#pragma unroll
  for (int u = 0; u < kGeluUnroll; ++u) {
    const int64_t i = base + (int64_t)u * kGeluThreads;
    if (i < nvec) {
      if constexpr (!kTanh && sizeof(T) == 2) {
#pragma unroll
        for (int j = 0; j < N; j += 2) {
          const float2 r = gelu_erf_pair(make_float2(v[u][j], v[u][j + 1]));
          v[u][j] = r.x;
          v[u][j + 1] = r.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[u][j] = kTanh ? gelu_tanh_for<T>(v[u][j]) : gelu_erf_f32(v[u][j]);
      }
      store16_stream(y + i * N, v[u]);
    }
  }
}

template <typename T, bool kTanh>
__global__ void gelu_scalar_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t start,
                                   int64_t numel) {
  const int64_t i = start + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < numel) {
    const float v = Elem<T>::to_f32(x[i]);
    float r;
    if constexpr (!kTanh && sizeof(T) == 2) r = gelu_erf_pair(make_float2(v, v)).x;
    else r = kTanh ? gelu_tanh_for<T>(v) : gelu_erf_f32(v);
    y[i] = Elem<T>::from_f32(r);
  }
}

template <typename T, bool kTanh>
int32_t launch_gelu(const void* x, void* y, int64_t numel, cudaStream_t stream) {
  constexpr int N = Elem<T>::kVec;
  const T* xp = static_cast<const T*>(x);
  T* yp = static_cast<T*>(y);
  int64_t nvec = 0;
  if (aligned_to(x, 16) && aligned_to(y, 16)) nvec = numel / N;
  if (nvec > 0) {
    const int64_t per_cta = (int64_t)kGeluThreads * kGeluUnroll;
    const int64_t grid = (nvec + per_cta - 1) / per_cta;
    B200_REQUIRE(grid <= INT32_MAX, B200_ERR_UNSUPPORTED, "gelu: tensor too large");
    gelu_vec_kernel<T, kTanh><<<(unsigned)grid, kGeluThreads, 0, stream>>>(xp, yp, nvec);
    B200_CHECK_LAUNCH("gelu");
  }
  const int64_t tail_start = nvec * N;
  if (tail_start < numel) {
    const int64_t tail = numel - tail_start;
    const int64_t grid = (tail + 255) / 256;
    B200_REQUIRE(grid <= INT32_MAX, B200_ERR_UNSUPPORTED, "gelu: tensor too large");
    gelu_scalar_kernel<T, kTanh><<<(unsigned)grid, 256, 0, stream>>>(xp, yp, tail_start, numel);
    B200_CHECK_LAUNCH("gelu(tail)");
  }
  return B200_OK;
}

// =========================================================================================
// Trailing-dim reductions
// =========================================================================================

template <int OP>
__device__ __forceinline__ float red_init() { return OP == B200_REDUCE_AMAX ? -INFINITY : 0.0f; }
template <int OP>
__device__ __forceinline__ float red_step(float a, float b) {
  return OP == B200_REDUCE_AMAX ? nan_max(a, b) : a + b;
}

template <typename Tin, typename Tout, int OP>
__global__ void __launch_bounds__(kRowThreads)
reduce_warp_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, int64_t rows, int cols,
                   int64_t x_row_stride) {
  constexpr int N = Elem<Tin>::kVec;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nchunks = cols / N;
  const Tin* xr = x + row * x_row_stride;
  // Four independent accumulators and four predicated 16-byte loads per lane and step: a short row
  // (fewer than 128 chunks) still has all of its loads in flight at once.
  float acc[4] = {red_init<OP>(), red_init<OP>(), red_init<OP>(), red_init<OP>()};
  for (int c = lane; c < nchunks; c += 128) {
    float v[4][N];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (c + 32 * u < nchunks) {
        load16_stream(xr + (c + 32 * u) * N, v[u]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[u][j] = red_init<OP>();
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int j = 0; j < N; ++j) acc[u] = red_step<OP>(acc[u], v[u][j]);
  }
  float r = red_step<OP>(red_step<OP>(acc[0], acc[1]), red_step<OP>(acc[2], acc[3]));
  r = OP == B200_REDUCE_AMAX ? warp_max(r) : warp_sum(r);
  if (OP == B200_REDUCE_MEAN) r = r / (float)cols;
  if (lane == 0) y[row] = Elem<Tout>::from_f32(r);
}

template <typename Tin, typename Tout, int OP>
__global__ void reduce_block_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, int64_t cols,
                                    int64_t x_row_stride) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const Tin* xr = x + row * x_row_stride;
  float r = red_init<OP>();
  for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
    r = red_step<OP>(r, Elem<Tin>::to_f32(xr[j]));
  r = OP == B200_REDUCE_AMAX ? block_max(r, red) : block_sum(r, red);
  if (OP == B200_REDUCE_MEAN) r = r / (float)cols;
  if (threadIdx.x == 0) y[row] = Elem<Tout>::from_f32(r);
}

template <typename Tin, typename Tout, int OP>
int32_t launch_reduce(const void* x, void* y, int64_t rows, int64_t cols, int64_t x_row_stride,
                      cudaStream_t stream) {
  constexpr int N = Elem<Tin>::kVec;
  const Tin* xp = static_cast<const Tin*>(x);
  Tout* yp = static_cast<Tout*>(y);
  const bool vec_ok = cols % N == 0 && x_row_stride % N == 0 && aligned_to(x, 16) &&
                      cols <= (1 << 20) && rows >= 512 &&
                      rows <= (int64_t)INT32_MAX * kWarpsPerCta;
  if (vec_ok) {
    const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
    reduce_warp_kernel<Tin, Tout, OP><<<grid, kRowThreads, 0, stream>>>(xp, yp, rows, (int)cols,
                                                                       x_row_stride);
  } else {
    B200_REQUIRE(rows <= INT32_MAX, B200_ERR_UNSUPPORTED, "reduce: too many rows");
    const int threads = cols >= 4096 ? 1024 : (cols >= 512 ? 256 : 64);
    reduce_block_kernel<Tin, Tout, OP><<<(unsigned)rows, threads, 0, stream>>>(xp, yp, cols,
                                                                              x_row_stride);
  }
  B200_CHECK_LAUNCH("reduce_lastdim");
  return B200_OK;
}

template <typename Tin, typename Tout>
int32_t dispatch_reduce(int32_t op, const void* x, void* y, int64_t rows, int64_t cols,
                        int64_t x_row_stride, cudaStream_t stream) {
  switch (op) {
    case B200_REDUCE_SUM:
      return launch_reduce<Tin, Tout, B200_REDUCE_SUM>(x, y, rows, cols, x_row_stride, stream);
    case B200_REDUCE_MEAN:
      return launch_reduce<Tin, Tout, B200_REDUCE_MEAN>(x, y, rows, cols, x_row_stride, stream);
    default:
      return launch_reduce<Tin, Tout, B200_REDUCE_AMAX>(x, y, rows, cols, x_row_stride, stream);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;
using bf16 = __nv_bfloat16;

extern "C" B200_API int32_t b200_layer_norm(const void* x, const void* gamma, const void* beta, void* y,
                                   float* mean, float* rstd, int64_t rows, int64_t cols,
                                   int64_t x_row_stride, float eps, int32_t in_dtype,
                                   int32_t param_dtype, int32_t out_dtype,
                                   b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "layer_norm: negative size");
  B200_REQUIRE(valid_dtype(in_dtype) && valid_dtype(param_dtype) && valid_dtype(out_dtype),
               B200_ERR_INVALID_ARG, "layer_norm: bad dtype enum");
  if (rows == 0) return B200_OK;
  B200_REQUIRE(cols > 0, B200_ERR_INVALID_ARG, "layer_norm: cols must be positive");
  B200_REQUIRE(x != nullptr && y != nullptr, B200_ERR_INVALID_ARG, "layer_norm: null pointer");
  B200_REQUIRE(x_row_stride >= cols || rows == 1, B200_ERR_INVALID_ARG,
               "layer_norm: row stride smaller than cols");
  B200_REQUIRE(aligned_to(x, dtype_size(in_dtype)) && aligned_to(y, dtype_size(out_dtype)),
               B200_ERR_ALIGNMENT, "layer_norm: pointer not element aligned");
#define LN_CASE(TI, TP, TO) \
  return launch_layer_norm<TI, TP, TO>(x, gamma, beta, y, mean, rstd, rows, cols, x_row_stride, eps, stream)
  const int key = in_dtype * 4 + param_dtype * 2 + out_dtype;
  switch (key) {
    case 0: LN_CASE(float, float, float);
    case 1: LN_CASE(float, float, bf16);
    case 2: LN_CASE(float, bf16, float);
    case 3: LN_CASE(float, bf16, bf16);
    case 4: LN_CASE(bf16, float, float);
    case 5: LN_CASE(bf16, float, bf16);
    case 6: LN_CASE(bf16, bf16, float);
    default: LN_CASE(bf16, bf16, bf16);
  }
#undef LN_CASE
}

namespace {
int32_t softmax_entry(const void* x, void* y, int64_t rows, int64_t cols, int64_t x_row_stride, float scale,
                      int32_t causal, int64_t q_len, b200::RowMask mask, int32_t in_dtype, int32_t out_dtype,
                      cudaStream_t stream) {
  using namespace b200;
  B200_REQUIRE(rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "softmax: negative size");
  B200_REQUIRE(valid_dtype(in_dtype) && valid_dtype(out_dtype), B200_ERR_INVALID_ARG,
               "softmax: bad dtype enum");
  B200_REQUIRE(!(in_dtype == B200_F32 && out_dtype == B200_BF16), B200_ERR_UNSUPPORTED,
               "softmax: fp32 input with bf16 output is not a torch softmax signature");
  if (rows == 0 || cols == 0) return B200_OK;
  B200_REQUIRE(x != nullptr && y != nullptr, B200_ERR_INVALID_ARG, "softmax: null pointer");
  B200_REQUIRE(!causal || q_len > 0, B200_ERR_INVALID_ARG, "softmax: causal needs q_len > 0");
  B200_REQUIRE(x_row_stride >= cols || rows == 1, B200_ERR_INVALID_ARG,
               "softmax: row stride smaller than cols");
  if (in_dtype == B200_F32)
    return launch_softmax<float, float>(x, y, rows, cols, x_row_stride, scale, causal, q_len, mask, stream);
  if (out_dtype == B200_F32)
    return launch_softmax<bf16, float>(x, y, rows, cols, x_row_stride, scale, causal, q_len, mask, stream);
  return launch_softmax<bf16, bf16>(x, y, rows, cols, x_row_stride, scale, causal, q_len, mask, stream);
}
}  // namespace

extern "C" B200_API int32_t b200_softmax_lastdim(const void* x, void* y, int64_t rows, int64_t cols,
                                        int64_t x_row_stride, float scale, int32_t causal,
                                        int64_t q_len, int32_t in_dtype, int32_t out_dtype,
                                        b200_stream_t stream_) {
  const b200::RowMask none = {nullptr, 1, 0, 0, 0.0f};
  return softmax_entry(x, y, rows, cols, x_row_stride, scale, causal, q_len, none, in_dtype, out_dtype,
                       static_cast<cudaStream_t>(stream_));
}

extern "C" B200_API int32_t b200_softmax_masked(const void* x, const uint8_t* mask, void* y, int64_t rows,
                                       int64_t cols, int64_t x_row_stride, int64_t mask_rows,
                                       int64_t mask_row_stride, int32_t mask_invert, float fill,
                                       float scale, int32_t in_dtype, int32_t out_dtype,
                                       b200_stream_t stream_) {
  B200_REQUIRE(rows == 0 || cols == 0 || mask != nullptr, B200_ERR_INVALID_ARG, "softmax_masked: null mask");
  B200_REQUIRE(mask_rows > 0 && (mask_row_stride >= cols || mask_rows == 1), B200_ERR_INVALID_ARG,
               "softmax_masked: mask needs at least one row and a row stride of at least cols");
  B200_REQUIRE(rows % mask_rows == 0, B200_ERR_INVALID_ARG,
               "softmax_masked: rows (%lld) is not a multiple of mask_rows (%lld)", (long long)rows,
               (long long)mask_rows);
  const b200::RowMask m = {mask, mask_rows, mask_row_stride, mask_invert != 0 ? 1 : 0, fill};
  return softmax_entry(x, y, rows, cols, x_row_stride, scale, 0, 0, m, in_dtype, out_dtype,
                       static_cast<cudaStream_t>(stream_));
}

extern "C" B200_API int32_t b200_gelu(const void* x, void* y, int64_t numel, int32_t approximate_tanh,
                             int32_t dtype, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(numel >= 0, B200_ERR_INVALID_ARG, "gelu: negative size");
  B200_REQUIRE(valid_dtype(dtype), B200_ERR_INVALID_ARG, "gelu: bad dtype enum");
  if (numel == 0) return B200_OK;
  B200_REQUIRE(x != nullptr && y != nullptr, B200_ERR_INVALID_ARG, "gelu: null pointer");
  if (dtype == B200_F32)
    return approximate_tanh ? launch_gelu<float, true>(x, y, numel, stream)
                            : launch_gelu<float, false>(x, y, numel, stream);
  return approximate_tanh ? launch_gelu<bf16, true>(x, y, numel, stream)
                          : launch_gelu<bf16, false>(x, y, numel, stream);
}

extern "C" B200_API int32_t b200_reduce_lastdim(const void* x, void* y, int64_t rows, int64_t cols,
                                       int64_t x_row_stride, int32_t op, int32_t in_dtype,
                                       int32_t out_dtype, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "reduce: negative size");
  B200_REQUIRE(valid_dtype(in_dtype) && valid_dtype(out_dtype), B200_ERR_INVALID_ARG,
               "reduce: bad dtype enum");
  B200_REQUIRE(op >= B200_REDUCE_SUM && op <= B200_REDUCE_AMAX, B200_ERR_INVALID_ARG,
               "reduce: bad op enum");
  if (rows == 0) return B200_OK;
  B200_REQUIRE(x != nullptr || cols == 0, B200_ERR_INVALID_ARG, "reduce: null input");
  B200_REQUIRE(y != nullptr, B200_ERR_INVALID_ARG, "reduce: null output");
  B200_REQUIRE(cols > 0 || op == B200_REDUCE_SUM, B200_ERR_INVALID_ARG,
               "reduce: mean/amax over an empty dim");
  if (in_dtype == B200_F32 && out_dtype == B200_F32)
    return dispatch_reduce<float, float>(op, x, y, rows, cols, x_row_stride, stream);
  if (in_dtype == B200_BF16 && out_dtype == B200_BF16)
    return dispatch_reduce<bf16, bf16>(op, x, y, rows, cols, x_row_stride, stream);
  if (in_dtype == B200_BF16 && out_dtype == B200_F32)
    return dispatch_reduce<bf16, float>(op, x, y, rows, cols, x_row_stride, stream);
  return dispatch_reduce<float, bf16>(op, x, y, rows, cols, x_row_stride, stream);
}

// Backward kernels of the bandwidth-bound ops: GELU, row softmax, LayerNorm (dx, dgamma, dbeta) and
// the sum over rows that a bias gradient is. All of them read their operands once from HBM (a second
// use of a row comes from L1/L2 or from registers), accumulate in fp32 and reduce in a fixed order,
// so the results do not depend on the launch.
#include "common.cuh"

namespace b200 {
namespace {

// ---- element vectors: N consecutive elements of T <-> N fp32 values -------------------------------
template <typename T, int N>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[N]);

template <>
__device__ __forceinline__ void load_vec<float, 4>(const float* p, float (&v)[4]) {
  const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16, 4>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void store_vec4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store_vec4<float>(float* p, const float (&v)[4]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
}
template <>
__device__ __forceinline__ void store_vec4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 t;
  t.x = pack_bf16x2(v[0], v[1]);
  t.y = pack_bf16x2(v[2], v[3]);
  __stcs(reinterpret_cast<uint2*>(p), t);
}

// =========================================================================================
// GELU backward: dx = dy * gelu'(x)
// =========================================================================================

// tanh form. With sg = sigmoid(2u), u = k0 (x + k1 x^3): 0.5 (1 + tanh u) = sg and
// 1 - tanh^2 u = 4 sg (1 - sg), so gelu'(x) = sg + 2 x sg (1 - sg) k0 (1 + 3 k1 x^2).
template <bool kFast>
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float x2 = x * x;
  const float u = k0 * (x + k1 * x2 * x);
  float sg;
  if (kFast) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-2.885390081777927f * u));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(sg) : "f"(1.0f + e));
  } else {
    sg = 1.0f / (1.0f + expf(-2.0f * u));
  }
  return sg + 2.0f * x * sg * (1.0f - sg) * k0 * (1.0f + 3.0f * k1 * x2);
}

// erf form: gelu'(x) = Phi(x) + x phi(x), Phi = 0.5 (1 + erf(x / sqrt 2)), phi = exp(-x^2 / 2) / sqrt(2 pi).
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.7071067811865476f));
  const float pdf = expf(-0.5f * x * x) * 0.3989422804014327f;
  return cdf + x * pdf;
}

// The same derivative for bf16 tensors on two MUFU operations: Phi(x) = x < 0 ? h : 1 - h with
// h = 0.5 erfc(|x| / sqrt 2) = t Q(t) exp(-x^2 / 2), t = 1 / (1 + |x| / (2 sqrt 2)) and Q the degree-7 fit
// the forward kernel uses (relative error 3e-6, far inside a bf16 rounding step); the exponential is
// shared with phi(x).
__device__ __forceinline__ float gelu_erf_grad_mufu(float x) {
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(fabsf(x), 0.35355339059327373f, 1.0f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * x * -0.7213475204444817f));
  float q = 2.504315786e-02f;
  q = fmaf(q, t, -5.376151577e-02f);
  q = fmaf(q, t, -2.228422835e-02f);
  q = fmaf(q, t, 6.382267177e-02f);
  q = fmaf(q, t, 8.064989746e-02f);
  q = fmaf(q, t, 1.244906485e-01f);
  q = fmaf(q, t, 1.409928650e-01f);
  q = fmaf(q, t, 1.410478354e-01f);
  const float h = t * q * e;
  const float cdf = x < 0.0f ? h : 1.0f - h;
  return fmaf(x * e, 0.3989422804014327f, cdf);
}

template <typename T>
__device__ __forceinline__ float gelu_erf_grad_for(float x) {
  return sizeof(T) == 2 ? gelu_erf_grad_mufu(x) : gelu_erf_grad(x);
}

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 2;

template <typename T, bool kTanh>
__global__ void __launch_bounds__(kEwThreads)
gelu_backward_vec_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, int64_t nvec) {
  // vectors of four elements: 16-byte accesses for fp32, 8-byte for bf16
  const int64_t base = (int64_t)blockIdx.x * (kEwThreads * kEwUnroll) + threadIdx.x;
  float xv[kEwUnroll][4], gv[kEwUnroll][4];
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec) {
      load_vec<T, 4>(x + i * 4, xv[u]);
      load_vec<T, 4>(dy + i * 4, gv[u]);
    }
  }
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec) {
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = gv[u][j] * (kTanh ? gelu_tanh_grad<sizeof(T) == 2>(xv[u][j]) : gelu_erf_grad_for<T>(xv[u][j]));
      store_vec4<T>(dx + i * 4, o);
    }
  }
}

template <typename T, bool kTanh>
__global__ void gelu_backward_scalar_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                                            int64_t start, int64_t numel) {
  const int64_t i = start + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < numel) {
    const float xv = Elem<T>::to_f32(x[i]);
    const float g = Elem<T>::to_f32(dy[i]);
    dx[i] = Elem<T>::from_f32(g * (kTanh ? gelu_tanh_grad<sizeof(T) == 2>(xv) : gelu_erf_grad_for<T>(xv)));
  }
}

template <typename T, bool kTanh>
int32_t launch_gelu_backward(const void* dy, const void* x, void* dx, int64_t numel, cudaStream_t stream) {
  const T* gp = static_cast<const T*>(dy);
  const T* xp = static_cast<const T*>(x);
  T* op = static_cast<T*>(dx);
  const size_t align = 4 * sizeof(T);
  int64_t nvec = 0;
  if (aligned_to(dy, align) && aligned_to(x, align) && aligned_to(dx, align)) nvec = numel / 4;
  if (nvec > 0) {
    const int64_t per_cta = (int64_t)kEwThreads * kEwUnroll;
    const int64_t grid = (nvec + per_cta - 1) / per_cta;
    B200_REQUIRE(grid <= INT32_MAX, B200_ERR_UNSUPPORTED, "gelu_backward: tensor too large");
    gelu_backward_vec_kernel<T, kTanh><<<(unsigned)grid, kEwThreads, 0, stream>>>(gp, xp, op, nvec);
    B200_CHECK_LAUNCH("gelu_backward");
  }
  const int64_t tail_start = nvec * 4;
  if (tail_start < numel) {
    const int64_t grid = (numel - tail_start + 255) / 256;
    B200_REQUIRE(grid <= INT32_MAX, B200_ERR_UNSUPPORTED, "gelu_backward: tensor too large");
    gelu_backward_scalar_kernel<T, kTanh><<<(unsigned)grid, 256, 0, stream>>>(gp, xp, op, tail_start, numel);
    B200_CHECK_LAUNCH("gelu_backward(tail)");
  }
  return B200_OK;
}

// =========================================================================================
// Row softmax backward: dx = scale * y * (dy - sum_j dy_j y_j)
// =========================================================================================

constexpr int kSbWarps = 8;

// One warp per row, two passes over the row: the dot product, then the result. The second pass
// finds the row in L1 (a warp's row is a few KB), so HBM sees each operand once.
template <typename Tin, typename Tout, bool VEC>
__global__ void __launch_bounds__(kSbWarps * 32)
softmax_backward_kernel(const Tin* __restrict__ dy, const Tin* __restrict__ y, Tout* __restrict__ dx, int64_t rows,
                        int64_t cols, int64_t dy_rs, int64_t y_rs, float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kSbWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const Tin* gr = dy + row * dy_rs;
  const Tin* yr = y + row * y_rs;
  Tout* xr = dx + row * cols;
  float dot = 0.0f;
  if (VEC) {
    float acc[2] = {0.0f, 0.0f};
    for (int64_t c = lane * 4; c < cols; c += 256) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int64_t cc = c + 128 * u;
        if (cc < cols) {
          float a[4], b[4];
          // plain loads: the lines are wanted again by the second pass
          if (sizeof(Tin) == 4) {
            const float4 ta = *reinterpret_cast<const float4*>(gr + cc), tb = *reinterpret_cast<const float4*>(yr + cc);
            a[0] = ta.x; a[1] = ta.y; a[2] = ta.z; a[3] = ta.w;
            b[0] = tb.x; b[1] = tb.y; b[2] = tb.z; b[3] = tb.w;
          } else {
            const uint2 ta = *reinterpret_cast<const uint2*>(gr + cc), tb = *reinterpret_cast<const uint2*>(yr + cc);
            a[0] = __uint_as_float(ta.x << 16); a[1] = __uint_as_float(ta.x & 0xffff0000u);
            a[2] = __uint_as_float(ta.y << 16); a[3] = __uint_as_float(ta.y & 0xffff0000u);
            b[0] = __uint_as_float(tb.x << 16); b[1] = __uint_as_float(tb.x & 0xffff0000u);
            b[2] = __uint_as_float(tb.y << 16); b[3] = __uint_as_float(tb.y & 0xffff0000u);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[u] = fmaf(a[j], b[j], acc[u]);
        }
      }
    }
    dot = acc[0] + acc[1];
  } else {
    for (int64_t c = lane; c < cols; c += 32) dot = fmaf(Elem<Tin>::to_f32(gr[c]), Elem<Tin>::to_f32(yr[c]), dot);
  }
  dot = warp_sum(dot);
  if (VEC) {
    for (int64_t c = lane * 4; c < cols; c += 128) {
      float a[4], b[4], o[4];
      load_vec<Tin, 4>(gr + c, a);
      load_vec<Tin, 4>(yr + c, b);
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = scale * b[j] * (a[j] - dot);
      store_vec4<Tout>(xr + c, o);
    }
  } else {
    for (int64_t c = lane; c < cols; c += 32)
      xr[c] = Elem<Tout>::from_f32(scale * Elem<Tin>::to_f32(yr[c]) * (Elem<Tin>::to_f32(gr[c]) - dot));
  }
}

template <typename Tin, typename Tout>
int32_t launch_softmax_backward(const void* dy, const void* y, void* dx, int64_t rows, int64_t cols, int64_t dy_rs,
                                int64_t y_rs, float scale, cudaStream_t stream) {
  const int64_t grid = (rows + kSbWarps - 1) / kSbWarps;
  B200_REQUIRE(grid <= INT32_MAX, B200_ERR_UNSUPPORTED, "softmax_backward: too many rows");
  const size_t a_in = 4 * sizeof(Tin), a_out = 4 * sizeof(Tout);
  const bool vec = cols % 4 == 0 && dy_rs % 4 == 0 && y_rs % 4 == 0 && aligned_to(dy, a_in) && aligned_to(y, a_in) &&
                   aligned_to(dx, a_out);
  if (vec)
    softmax_backward_kernel<Tin, Tout, true><<<(unsigned)grid, kSbWarps * 32, 0, stream>>>(
        static_cast<const Tin*>(dy), static_cast<const Tin*>(y), static_cast<Tout*>(dx), rows, cols, dy_rs, y_rs, scale);
  else
    softmax_backward_kernel<Tin, Tout, false><<<(unsigned)grid, kSbWarps * 32, 0, stream>>>(
        static_cast<const Tin*>(dy), static_cast<const Tin*>(y), static_cast<Tout*>(dx), rows, cols, dy_rs, y_rs, scale);
  B200_CHECK_LAUNCH("softmax_backward");
  return B200_OK;
}

// =========================================================================================
// LayerNorm backward and the sum over rows (bias gradient)
// =========================================================================================

// out[c] = sum over the partial rows of part[nparts, cols], for up to two arrays at once
// (blockIdx.y). A CTA of 32 x 32 threads takes 32 columns: thread (cx, ry) adds rows ry, ry + 32, ...
// of column cx, then the 32 row sums of a column are added in ry order: a fixed order whatever the
// launch, and short dependent chains instead of one thread walking every partial row.
struct PartialSums {
  const float* part[2];
  void* out[2];
};

template <typename Tout>
__global__ void __launch_bounds__(1024)
sum_partials_kernel(PartialSums ps, int64_t nparts, int cols) {
  __shared__ float tile[32][33];
  const float* part = ps.part[blockIdx.y];
  Tout* out = static_cast<Tout*>(ps.out[blockIdx.y]);
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s0 = 0.0f, s1 = 0.0f;
  if (c < cols) {
    int64_t r = ry;
    for (; r + 32 < nparts; r += 64) {
      s0 += part[r * cols + c];
      s1 += part[(r + 32) * cols + c];
    }
    if (r < nparts) s0 += part[r * cols + c];
  }
  tile[ry][cx] = s0 + s1;
  __syncthreads();
  if (ry == 0 && c < cols) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) s += tile[i][cx];
    out[c] = Elem<Tout>::from_f32(s);
  }
}

template <typename Tout>
int32_t launch_sum_partials(const float* part_a, void* out_a, const float* part_b, void* out_b, int64_t nparts,
                            int64_t cols, cudaStream_t stream, const char* what) {
  PartialSums ps;
  int n = 0;
  if (out_a != nullptr) { ps.part[n] = part_a; ps.out[n] = out_a; ++n; }
  if (out_b != nullptr) { ps.part[n] = part_b; ps.out[n] = out_b; ++n; }
  if (n == 0) return B200_OK;
  if (n == 1) { ps.part[1] = ps.part[0]; ps.out[1] = ps.out[0]; }
  sum_partials_kernel<Tout><<<dim3((unsigned)((cols + 31) / 32), (unsigned)n), 1024, 0, stream>>>(ps, nparts, (int)cols);
  B200_CHECK_LAUNCH(what);
  return B200_OK;
}

constexpr int kLnbWarps = 4;      // warps per CTA
constexpr int kLnbCtasPerSm = 2;  // two rows of up to 2048 columns in registers per lane: 8 warps per SM

// Four consecutive elements as loaded (fp32: 16 bytes, bf16: 8 bytes), widened on use.
template <typename T>
struct Raw4;
template <>
struct Raw4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void load_stream(const float* p) { v = __ldcs(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ void load_shared(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void unpack(float (&o)[4]) const { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};
template <>
struct Raw4<__nv_bfloat16> {
  uint2 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void load_stream(const __nv_bfloat16* p) { v = __ldcs(reinterpret_cast<const uint2*>(p)); }
  __device__ __forceinline__ void load_shared(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void unpack(float (&o)[4]) const {
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
  }
};
// Asynchronous global -> shared copy of 8 or 16 bytes (both addresses aligned to the size), read
// back by the thread that issued it after cp_async_wait_all().
template <int BYTES>
__device__ __forceinline__ void cp_async_small(void* smem_dst, const void* gmem_src) {
  static_assert(BYTES == 8 || BYTES == 16, "cp.async.ca copies 4, 8 or 16 bytes");
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src), "n"(BYTES)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int kLnbMaxChunks = 16; // 128-column chunks a lane can keep column sums for (2048 columns)

// LayerNorm backward, one WARP per row and no CTA-wide synchronisation while rows stream. A warp
// walks rows (warp, warp + total, ...); lane l owns columns {128 i + 4 l .. + 3}. With
// xhat = (x - mean) rstd and g = dy gamma:
//   dx = rstd (g - mean_j(g) - xhat mean_j(g xhat)),  dgamma = sum_rows dy xhat,  dbeta = sum_rows dy.
// A row is worked on out of registers: pass 1 takes the two row sums and adds the row into the
// warp's own column sums (a private strip of shared memory, row order), pass 2 writes dx. The
// warp's NEXT row is loaded into a second register set meanwhile (all loads issued at once), so
// HBM sees every operand once and every warp always has a row of loads in flight. (Measured
// against it and no faster: twice the warps with one register set each; a second pass over L1
// instead of the second register set.) At the end the warps of a CTA add their column sums in warp order and
// the CTA leaves one partial row in part_g / part_b [grid, cols]; a second kernel adds the CTAs up.
template <typename Tx, typename Tg, typename Tp, typename Td, int MAXC>
__global__ void __launch_bounds__(kLnbWarps * 32, kLnbCtasPerSm)
layer_norm_backward_kernel(const Tg* __restrict__ dy, const Tx* __restrict__ x, const float* __restrict__ mean,
                           const float* __restrict__ rstd, const Tp* __restrict__ gamma, const Td* __restrict__ dx_add,
                           Td* __restrict__ dx, __nv_bfloat16* __restrict__ dx_cast, float* __restrict__ part_g,
                           float* __restrict__ part_b, float* __restrict__ part_s, int64_t rows, int cols, int64_t dy_rs,
                           int64_t x_rs) {
  // [kLnbWarps][2][cols] floats: every warp's column sums of dy xhat and dy; with a part_s,
  // [kLnbWarps][cols] floats: its column sums of dx; with a dx_add, [kLnbWarps][cols] Td: the dx_add
  // row of the warp's next row, copied asynchronously
  extern __shared__ float lnb_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t total_warps = (int64_t)gridDim.x * kLnbWarps;
  float* sm_g = lnb_smem + (size_t)warp * 2 * cols;
  float* sm_b = sm_g + cols;
  float* sm_sums = lnb_smem + (size_t)kLnbWarps * 2 * cols;  // all warps' strips of dx column sums
  float* sm_s = sm_sums + (size_t)warp * cols;
  Td* sm_add = reinterpret_cast<Td*>(sm_sums + (part_s != nullptr ? (size_t)kLnbWarps * cols : 0)) + (size_t)warp * cols;
  // Every lane copies the columns it will add itself, so no other lane waits for the copy. The row
  // is asked for one row ahead (after the previous row's values were read and used), which leaves
  // the whole first pass of the row to cover the latency without holding registers for it.
  auto stage_add = [&](int64_t row) {
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < cols) cp_async_small<4 * (int)sizeof(Td)>(sm_add + c, dx_add + row * (int64_t)cols + c);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = 128 * i + 4 * lane;
    if (c < cols) {
      *reinterpret_cast<float4*>(sm_g + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      *reinterpret_cast<float4*>(sm_b + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (part_s != nullptr) *reinterpret_cast<float4*>(sm_s + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  }
  const float inv_cols = 1.0f / (float)cols;

  // gamma of the lane's columns, four at a time
  auto gamma4 = [&](int c, float (&w)[4]) {
    if (gamma == nullptr) {
      w[0] = w[1] = w[2] = w[3] = 1.0f;
    } else {
      Raw4<Tp> t;
      t.load(gamma + c);
      t.unpack(w);
    }
  };
  // Two register sets hold two rows (as loaded: fp32 or bf16): while one row is worked on, the
  // loads of the warp's next row -- all issued at once -- are in flight into the other.
  Raw4<Tx> xa[MAXC], xb[MAXC];
  Raw4<Tg> ga[MAXC], gb[MAXC];
  float2 stat_a, stat_b;  // (mean, rstd) of the row, fetched with it
  auto fetch = [&](int64_t row, Raw4<Tx> (&xr)[MAXC], Raw4<Tg> (&gr)[MAXC], float2& stat) {
    stat = make_float2(mean[row], rstd[row]);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < cols) {
        xr[i].load_stream(x + row * x_rs + c);
        gr[i].load_stream(dy + row * dy_rs + c);
      }
    }
  };
  // The arithmetic is arranged for the packed two-wide FMA pipe and few operations per element:
  //   xhat = x rs - mu rs,  t = dy xhat,  s1 += dy w,  s2 += t w,  dgamma += t,  dbeta += dy   (pass 1)
  //   dx = dy (w rs) + x A + B  with  A = -rs^2 c2,  B = rs^2 c2 mu - rs c1                       (pass 2)
  auto process = [&](int64_t row, int64_t next_row, const Raw4<Tx> (&xr)[MAXC], const Raw4<Tg> (&gr)[MAXC],
                     float2 stat) {
    const float mu = stat.x, rs = stat.y;
    const float2 rs2 = make_float2(rs, rs), nmurs2 = make_float2(-mu * rs, -mu * rs);
    float2 s1 = make_float2(0.0f, 0.0f), s2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < cols) {
        float xv[4], gv[4], w[4];
        xr[i].unpack(xv);
        gr[i].unpack(gv);
        gamma4(c, w);
        float4 ag = *reinterpret_cast<const float4*>(sm_g + c), ab = *reinterpret_cast<const float4*>(sm_b + c);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 x2 = make_float2(xv[2 * h], xv[2 * h + 1]), g2 = make_float2(gv[2 * h], gv[2 * h + 1]);
          const float2 w2 = make_float2(w[2 * h], w[2 * h + 1]);
          const float2 xh = __ffma2_rn(x2, rs2, nmurs2);
          const float2 t = __fmul2_rn(g2, xh);
          s1 = __ffma2_rn(g2, w2, s1);
          s2 = __ffma2_rn(t, w2, s2);
          float2* agp = reinterpret_cast<float2*>(&ag) + h;
          float2* abp = reinterpret_cast<float2*>(&ab) + h;
          *agp = __fadd2_rn(*agp, t);
          *abp = __fadd2_rn(*abp, g2);
        }
        *reinterpret_cast<float4*>(sm_g + c) = ag;
        *reinterpret_cast<float4*>(sm_b + c) = ab;
      }
    }
    const float c1 = warp_sum(s1.x + s1.y) * inv_cols, c2 = warp_sum(s2.x + s2.y) * inv_cols;
    const float a = -rs * rs * c2, b = rs * rs * c2 * mu - rs * c1;
    const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
    Td* dr = dx + row * (int64_t)cols;
    if (dx_add != nullptr) cp_async_wait_all();
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < cols) {
        float xv[4], gv[4], w[4], o[4];
        xr[i].unpack(xv);
        gr[i].unpack(gv);
        gamma4(c, w);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 x2 = make_float2(xv[2 * h], xv[2 * h + 1]), g2 = make_float2(gv[2 * h], gv[2 * h + 1]);
          const float2 wr = __fmul2_rn(make_float2(w[2 * h], w[2 * h + 1]), rs2);
          const float2 r = __ffma2_rn(g2, wr, __ffma2_rn(x2, a2, b2));
          o[2 * h] = r.x;
          o[2 * h + 1] = r.y;
        }
        if (dx_add != nullptr) {  // the gradient that reaches x along the residual branch, added in the same pass
          float extra[4];
          Raw4<Td> staged;
          staged.load_shared(sm_add + c);
          staged.unpack(extra);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] += extra[j];
        }
        store_vec4<Td>(dr + c, o);
        // the same values once more as bf16 (the operand of the next gradient GEMMs), and their
        // column sums (the bias gradient of the layer that produced x): of the rounded values when
        // the bf16 copy is written, as a sum over that copy would give
        uint2 narrow;  // two packed conversions (the unpacked form runs at a quarter of their rate)
        if (dx_cast != nullptr || (part_s != nullptr && sizeof(Td) == 2)) {
          narrow.x = pack_bf16x2(o[0], o[1]);
          narrow.y = pack_bf16x2(o[2], o[3]);
        }
        if (dx_cast != nullptr) __stcs(reinterpret_cast<uint2*>(dx_cast + row * (int64_t)cols + c), narrow);
        if (part_s != nullptr) {
          if (dx_cast != nullptr || sizeof(Td) == 2) {
            o[0] = __uint_as_float(narrow.x << 16); o[1] = __uint_as_float(narrow.x & 0xffff0000u);
            o[2] = __uint_as_float(narrow.y << 16); o[3] = __uint_as_float(narrow.y & 0xffff0000u);
          }
          float4 acc = *reinterpret_cast<const float4*>(sm_s + c);
          acc.x += o[0]; acc.y += o[1]; acc.z += o[2]; acc.w += o[3];
          *reinterpret_cast<float4*>(sm_s + c) = acc;
        }
      }
    }
    if (dx_add != nullptr && next_row < rows) stage_add(next_row);
  };

  int64_t row = (int64_t)blockIdx.x * kLnbWarps + warp;
  if (row < rows) {
    fetch(row, xa, ga, stat_a);
    if (dx_add != nullptr) stage_add(row);
  }
  while (row < rows) {
    const int64_t row_b = row + total_warps;
    if (row_b < rows) fetch(row_b, xb, gb, stat_b);
    process(row, row_b, xa, ga, stat_a);
    if (row_b >= rows) break;
    row = row_b + total_warps;
    if (row < rows) fetch(row, xa, ga, stat_a);
    process(row_b, row, xb, gb, stat_b);
  }

  // column sums of the CTA: warp order, then one partial row per CTA
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += kLnbWarps * 32) {
    float g = 0.0f, b = 0.0f;
#pragma unroll
    for (int w = 0; w < kLnbWarps; ++w) {
      g += lnb_smem[(size_t)w * 2 * cols + c];
      b += lnb_smem[(size_t)w * 2 * cols + cols + c];
    }
    part_g[(int64_t)blockIdx.x * cols + c] = g;
    part_b[(int64_t)blockIdx.x * cols + c] = b;
    if (part_s != nullptr) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < kLnbWarps; ++w) t += sm_sums[(size_t)w * cols + c];
      part_s[(int64_t)blockIdx.x * cols + c] = t;
    }
  }
}

// Sum over the rows of x[rows, cols]. A CTA of eight warps covers a slab of 8 x 32 x V columns
// (V = elements of a 16-byte vector); every lane owns V columns and walks the rows of its stream
// (blockIdx.y, + gridDim.y, ...) four at a time, so four 16-byte loads per lane are in flight and
// nothing is ever exchanged between threads. One partial row per stream, added up by a second kernel.
constexpr int kSumThreads = 256;
constexpr int kSumUnroll = 4;

template <typename T>
__global__ void __launch_bounds__(kSumThreads)
sum_rows_kernel(const T* __restrict__ x, float* __restrict__ part, int64_t rows, int cols, int64_t x_rs) {
  constexpr int V = Elem<T>::kVec;
  const int c = ((int)blockIdx.x * kSumThreads + (int)threadIdx.x) * V;
  if (c >= cols) return;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.0f;
  const int64_t step = gridDim.y;
  for (int64_t row = blockIdx.y; row < rows; row += kSumUnroll * step) {
    float v[kSumUnroll][V];
#pragma unroll
    for (int u = 0; u < kSumUnroll; ++u) {
      const int64_t r = row + u * step;
      if (r < rows) {
        load16_stream(x + r * x_rs + c, v[u]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[u][j] = 0.0f;
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] += (v[0][j] + v[1][j]) + (v[2][j] + v[3][j]);
  }
#pragma unroll
  for (int j = 0; j < V; ++j) part[(int64_t)blockIdx.y * cols + c + j] = acc[j];
}

// Generic forms (columns not a multiple of the vector, unaligned pointers, rows too wide for the
// register path): one CTA per row for dx, one thread per column and row slab for the column sums.
constexpr int kGenThreads = 256;

__device__ __forceinline__ void block_sum2(float& a, float& b, float (*red)[2]) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[warp][0] = a; red[warp][1] = b; }
  __syncthreads();
  float sa = 0.0f, sb = 0.0f;
#pragma unroll
  for (int w = 0; w < kGenThreads / 32; ++w) { sa += red[w][0]; sb += red[w][1]; }
  a = sa;
  b = sb;
}

template <typename Tx, typename Tg, typename Tp, typename Td>
__global__ void __launch_bounds__(kGenThreads)
layer_norm_backward_dx_generic_kernel(const Tg* __restrict__ dy, const Tx* __restrict__ x,
                                      const float* __restrict__ mean, const float* __restrict__ rstd,
                                      const Tp* __restrict__ gamma, const Td* __restrict__ dx_add, Td* __restrict__ dx,
                                      __nv_bfloat16* __restrict__ dx_cast, int64_t cols, int64_t dy_rs, int64_t x_rs) {
  __shared__ float red[kGenThreads / 32][2];
  const int64_t row = blockIdx.x;
  const float mu = mean[row], rs = rstd[row];
  float s1 = 0.0f, s2 = 0.0f;
  for (int64_t c = threadIdx.x; c < cols; c += kGenThreads) {
    const float g = Elem<Tg>::to_f32(dy[row * dy_rs + c]) * (gamma != nullptr ? Elem<Tp>::to_f32(gamma[c]) : 1.0f);
    s1 += g;
    s2 = fmaf(g, (Elem<Tx>::to_f32(x[row * x_rs + c]) - mu) * rs, s2);
  }
  block_sum2(s1, s2, red);
  const float c1 = s1 / (float)cols, c2 = s2 / (float)cols;
  for (int64_t c = threadIdx.x; c < cols; c += kGenThreads) {
    const float g = Elem<Tg>::to_f32(dy[row * dy_rs + c]) * (gamma != nullptr ? Elem<Tp>::to_f32(gamma[c]) : 1.0f);
    const float xh = (Elem<Tx>::to_f32(x[row * x_rs + c]) - mu) * rs;
    const float extra = dx_add != nullptr ? Elem<Td>::to_f32(dx_add[row * cols + c]) : 0.0f;
    // a separate rounding for the add: the sum equals (dx as it would be stored in fp32) + dx_add
    const float out = __fadd_rn(__fmul_rn(rs, g - c1 - xh * c2), extra);
    dx[row * cols + c] = Elem<Td>::from_f32(out);
    if (dx_cast != nullptr) dx_cast[row * cols + c] = __float2bfloat16_rn(out);
  }
}

template <typename Tx, typename Tg>
__global__ void layer_norm_backward_params_generic_kernel(const Tg* __restrict__ dy, const Tx* __restrict__ x,
                                                          const float* __restrict__ mean,
                                                          const float* __restrict__ rstd, float* __restrict__ part_g,
                                                          float* __restrict__ part_b, int64_t rows, int64_t cols,
                                                          int64_t dy_rs, int64_t x_rs, int64_t rows_per_slab) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float sg = 0.0f, sb = 0.0f;
  for (int64_t r = r0; r < r1; ++r) {
    const float g = Elem<Tg>::to_f32(dy[r * dy_rs + c]);
    sg = fmaf(g, (Elem<Tx>::to_f32(x[r * x_rs + c]) - mean[r]) * rstd[r], sg);
    sb += g;
  }
  part_g[(int64_t)blockIdx.y * cols + c] = sg;
  part_b[(int64_t)blockIdx.y * cols + c] = sb;
}

template <typename T>
__global__ void sum_rows_generic_kernel(const T* __restrict__ x, float* __restrict__ part, int64_t rows, int64_t cols,
                                        int64_t x_rs, int64_t rows_per_slab) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float s = 0.0f;
  for (int64_t r = r0; r < r1; ++r) s += Elem<T>::to_f32(x[r * x_rs + c]);
  part[(int64_t)blockIdx.y * cols + c] = s;
}

constexpr int kGenericSlabs = 64;  // row slabs of the generic column-sum kernels

int64_t generic_parts(int64_t rows) { return rows < kGenericSlabs ? (rows > 0 ? rows : 1) : kGenericSlabs; }

// ---- LayerNorm backward: which form, how many partial rows ----
bool lnb_fast(int64_t cols) { return cols % 4 == 0 && cols <= 128 * kLnbMaxChunks; }
int64_t lnb_parts(int64_t rows, int64_t cols) {
  if (!lnb_fast(cols)) return generic_parts(rows);
  const int64_t want = (int64_t)sm_count() * kLnbCtasPerSm, need = (rows + kLnbWarps - 1) / kLnbWarps;
  return need < want ? (need > 0 ? need : 1) : want;
}

template <typename Tx, typename Tg, typename Tp, typename Td>
int32_t launch_layer_norm_backward(const void* dy, const void* x, const float* mean, const float* rstd,
                                   const void* gamma, const void* dx_add, void* dx, void* dgamma, void* dbeta,
                                   void* dx_cast, void* dx_sum, int32_t dx_sum_dtype, float* ws, int64_t rows,
                                   int64_t cols, int64_t dy_rs, int64_t x_rs, cudaStream_t stream) {
  const Tg* gp = static_cast<const Tg*>(dy);
  const Tx* xp = static_cast<const Tx*>(x);
  const Tp* wp = static_cast<const Tp*>(gamma);
  Td* op = static_cast<Td*>(dx);
  const Td* ap = static_cast<const Td*>(dx_add);
  const int64_t nparts = lnb_parts(rows, cols);
  float* part_g = ws;
  float* part_b = ws + nparts * cols;
  float* part_s = dx_sum != nullptr ? ws + 2 * nparts * cols : nullptr;
  __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(dx_cast);
  const bool fast = lnb_fast(cols) && (dx_cast == nullptr || aligned_to(dx_cast, 8)) && dy_rs % 4 == 0 && x_rs % 4 == 0 && aligned_to(dy, 4 * sizeof(Tg)) &&
                    aligned_to(x, 4 * sizeof(Tx)) && aligned_to(dx, 4 * sizeof(Td)) &&
                    (dx_add == nullptr || aligned_to(dx_add, 4 * sizeof(Td)));
  if (fast) {
    const int chunks = (int)((cols + 127) / 128);
    // at most 64 KiB of column sums, 32 KiB for those of dx and 32 KiB for the staged dx_add rows
    const size_t smem = (size_t)kLnbWarps * (size_t)cols *
                        (2 * sizeof(float) + (part_s != nullptr ? sizeof(float) : 0) + (dx_add != nullptr ? sizeof(Td) : 0));
#define LNB(MAXC)                                                                                              \
  do {                                                                                                         \
    auto kernel = layer_norm_backward_kernel<Tx, Tg, Tp, Td, MAXC>;                                            \
    /* opt in once per kernel and device to the most this kernel can ask for (2048 columns) */                 \
    static thread_local bool attr_set[64] = {false};                                                           \
    int dev = 0;                                                                                               \
    cudaGetDevice(&dev);                                                                                       \
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {                                                              \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                                           kLnbWarps * 128 * kLnbMaxChunks * (int)(3 * sizeof(float) + sizeof(Td))); \
      if (e != cudaSuccess)                                                                                    \
        B200_FAIL(B200_ERR_CUDA, "layer_norm_backward: cannot opt in to shared memory: %s",                    \
                  cudaGetErrorString(e));                                                                      \
      attr_set[dev] = true;                                                                                    \
    }                                                                                                          \
    kernel<<<(unsigned)nparts, kLnbWarps * 32, smem, stream>>>(gp, xp, mean, rstd, wp, ap, op, cp, part_g,      \
                                                               part_b, part_s, rows, (int)cols, dy_rs, x_rs);  \
  } while (0)
    if (chunks <= 2) LNB(2);
    else if (chunks <= 4) LNB(4);
    else if (chunks <= 6) LNB(6);
    else if (chunks <= 8) LNB(8);
    else if (chunks <= 13) LNB(13);
    else LNB(16);
#undef LNB
    B200_CHECK_LAUNCH("layer_norm_backward");
  } else {
    B200_REQUIRE(rows <= INT32_MAX, B200_ERR_UNSUPPORTED, "layer_norm_backward: too many rows");
    layer_norm_backward_dx_generic_kernel<Tx, Tg, Tp, Td><<<(unsigned)rows, kGenThreads, 0, stream>>>(
        gp, xp, mean, rstd, wp, ap, op, cp, cols, dy_rs, x_rs);
    B200_CHECK_LAUNCH("layer_norm_backward(dx)");
    const int64_t per_slab = (rows + nparts - 1) / nparts;
    const int64_t bx = (cols + 255) / 256;
    layer_norm_backward_params_generic_kernel<Tx, Tg><<<dim3((unsigned)bx, (unsigned)nparts), 256, 0, stream>>>(
        gp, xp, mean, rstd, part_g, part_b, rows, cols, dy_rs, x_rs, per_slab);
    B200_CHECK_LAUNCH("layer_norm_backward(params)");
    if (part_s != nullptr) {  // column sums of what was just written (the bf16 copy when there is one)
      if (cp != nullptr)
        sum_rows_generic_kernel<__nv_bfloat16><<<dim3((unsigned)bx, (unsigned)nparts), 256, 0, stream>>>(
            cp, part_s, rows, cols, cols, per_slab);
      else
        sum_rows_generic_kernel<Td><<<dim3((unsigned)bx, (unsigned)nparts), 256, 0, stream>>>(op, part_s, rows, cols, cols,
                                                                                              per_slab);
      B200_CHECK_LAUNCH("layer_norm_backward(dx sums)");
    }
  }
  if (part_s != nullptr) {
    const int32_t st = dx_sum_dtype == B200_F32
                           ? launch_sum_partials<float>(part_s, dx_sum, nullptr, nullptr, nparts, cols, stream,
                                                        "layer_norm_backward(dx sums)")
                           : launch_sum_partials<__nv_bfloat16>(part_s, dx_sum, nullptr, nullptr, nparts, cols, stream,
                                                                "layer_norm_backward(dx sums)");
    if (st != B200_OK) return st;
  }
  return launch_sum_partials<Tp>(part_g, dgamma, part_b, dbeta, nparts, cols, stream, "layer_norm_backward(sums)");
}

// ---- sum over rows: which form, how many partial rows ----
bool sum_rows_fast(int64_t cols, int elem_size) { return cols % (16 / elem_size) == 0; }
int64_t sum_rows_parts(int64_t rows, int64_t cols, int elem_size) {
  if (!sum_rows_fast(cols, elem_size)) return generic_parts(rows);
  const int64_t slabs = (cols + (int64_t)kSumThreads * (16 / elem_size) - 1) / ((int64_t)kSumThreads * (16 / elem_size));
  int64_t streams = ((int64_t)sm_count() * 6 + slabs - 1) / slabs;  // ~six CTAs per SM over all slabs
  const int64_t most = (rows + kSumUnroll - 1) / kSumUnroll;       // at least one unrolled step per stream
  if (streams > most) streams = most;
  if (streams > 65535) streams = 65535;
  return streams > 0 ? streams : 1;
}

template <typename T, typename Tout>
int32_t launch_sum_rows(const void* x, void* y, float* ws, int64_t rows, int64_t cols, int64_t x_rs,
                        cudaStream_t stream) {
  const T* xp = static_cast<const T*>(x);
  constexpr int V = Elem<T>::kVec;
  const int64_t nparts = sum_rows_parts(rows, cols, (int)sizeof(T));
  const bool fast = sum_rows_fast(cols, (int)sizeof(T)) && x_rs % V == 0 && aligned_to(x, 16);
  if (fast) {
    const int64_t slabs = (cols + (int64_t)kSumThreads * V - 1) / ((int64_t)kSumThreads * V);
    sum_rows_kernel<T><<<dim3((unsigned)slabs, (unsigned)nparts), kSumThreads, 0, stream>>>(xp, ws, rows, (int)cols, x_rs);
  } else {
    const int64_t gparts = nparts < kGenericSlabs ? nparts : kGenericSlabs;
    const int64_t per_slab = (rows + gparts - 1) / gparts;
    const int64_t bx = (cols + 255) / 256;
    B200_REQUIRE(bx <= INT32_MAX, B200_ERR_UNSUPPORTED, "sum_rows: too many columns");
    // (an unaligned tensor whose shape would have taken the vector form: fewer, longer slabs; the
    // partial rows beyond gparts are zeroed so that the final sum may read them all)
    if (gparts < nparts &&
        cudaMemsetAsync(ws + gparts * cols, 0, (size_t)(nparts - gparts) * (size_t)cols * sizeof(float), stream) != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "sum_rows: memset failed");
    sum_rows_generic_kernel<T><<<dim3((unsigned)bx, (unsigned)gparts), 256, 0, stream>>>(xp, ws, rows, cols, x_rs,
                                                                                       per_slab);
  }
  B200_CHECK_LAUNCH("sum_rows");
  return launch_sum_partials<Tout>(ws, y, nullptr, nullptr, nparts, cols, stream, "sum_rows(final)");
}

}  // namespace
}  // namespace b200

using namespace b200;
using bf16 = __nv_bfloat16;

extern "C" B200_API int32_t b200_gelu_backward(const void* dy, const void* x, void* dx, int64_t numel,
                                               int32_t approximate_tanh, int32_t dtype, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(numel >= 0, B200_ERR_INVALID_ARG, "gelu_backward: negative size");
  B200_REQUIRE(valid_dtype(dtype), B200_ERR_INVALID_ARG, "gelu_backward: bad dtype enum");
  if (numel == 0) return B200_OK;
  B200_REQUIRE(dy != nullptr && x != nullptr && dx != nullptr, B200_ERR_INVALID_ARG, "gelu_backward: null pointer");
  const size_t es = dtype_size(dtype);
  B200_REQUIRE(aligned_to(dy, es) && aligned_to(x, es) && aligned_to(dx, es), B200_ERR_ALIGNMENT,
               "gelu_backward: pointer not element aligned");
  if (dtype == B200_F32)
    return approximate_tanh ? launch_gelu_backward<float, true>(dy, x, dx, numel, stream)
                            : launch_gelu_backward<float, false>(dy, x, dx, numel, stream);
  return approximate_tanh ? launch_gelu_backward<bf16, true>(dy, x, dx, numel, stream)
                          : launch_gelu_backward<bf16, false>(dy, x, dx, numel, stream);
}

extern "C" B200_API int32_t b200_softmax_backward(const void* dy, const void* y, void* dx, int64_t rows, int64_t cols,
                                                  int64_t dy_row_stride, int64_t y_row_stride, float scale,
                                                  int32_t in_dtype, int32_t out_dtype, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "softmax_backward: negative size");
  B200_REQUIRE(valid_dtype(in_dtype) && valid_dtype(out_dtype), B200_ERR_INVALID_ARG, "softmax_backward: bad dtype enum");
  if (rows == 0 || cols == 0) return B200_OK;
  B200_REQUIRE(dy != nullptr && y != nullptr && dx != nullptr, B200_ERR_INVALID_ARG, "softmax_backward: null pointer");
  B200_REQUIRE((dy_row_stride >= cols && y_row_stride >= cols) || rows == 1, B200_ERR_INVALID_ARG,
               "softmax_backward: row stride smaller than cols");
  B200_REQUIRE(aligned_to(dy, dtype_size(in_dtype)) && aligned_to(y, dtype_size(in_dtype)) &&
                   aligned_to(dx, dtype_size(out_dtype)),
               B200_ERR_ALIGNMENT, "softmax_backward: pointer not element aligned");
  if (in_dtype == B200_F32 && out_dtype == B200_F32)
    return launch_softmax_backward<float, float>(dy, y, dx, rows, cols, dy_row_stride, y_row_stride, scale, stream);
  if (in_dtype == B200_BF16 && out_dtype == B200_BF16)
    return launch_softmax_backward<bf16, bf16>(dy, y, dx, rows, cols, dy_row_stride, y_row_stride, scale, stream);
  if (in_dtype == B200_F32 && out_dtype == B200_BF16)
    return launch_softmax_backward<float, bf16>(dy, y, dx, rows, cols, dy_row_stride, y_row_stride, scale, stream);
  return launch_softmax_backward<bf16, float>(dy, y, dx, rows, cols, dy_row_stride, y_row_stride, scale, stream);
}

extern "C" B200_API size_t b200_layer_norm_backward_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return (size_t)lnb_parts(rows, cols) * (size_t)cols * 3 * sizeof(float);  // dgamma, dbeta and dx_sum partial rows
}

extern "C" B200_API int32_t b200_layer_norm_backward(const void* dy, const void* x, const float* mean,
                                                     const float* rstd, const void* gamma, const void* dx_add,
                                                     void* dx, void* dgamma, void* dbeta, void* dx_cast, void* dx_sum,
                                                     void* workspace, size_t workspace_bytes,
                                                     int64_t rows, int64_t cols, int64_t dy_row_stride,
                                                     int64_t x_row_stride, int32_t x_dtype, int32_t dy_dtype,
                                                     int32_t param_dtype, int32_t dx_dtype, int32_t dx_sum_dtype,
                                                     b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(dx_cast == nullptr || dx_dtype == B200_F32, B200_ERR_UNSUPPORTED,
               "layer_norm_backward: the bf16 copy of dx is offered for an fp32 dx");
  B200_REQUIRE(dx_sum == nullptr || valid_dtype(dx_sum_dtype), B200_ERR_INVALID_ARG,
               "layer_norm_backward: bad dx_sum dtype enum");
  B200_REQUIRE(rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "layer_norm_backward: negative size");
  B200_REQUIRE(valid_dtype(x_dtype) && valid_dtype(dy_dtype) && valid_dtype(param_dtype) && valid_dtype(dx_dtype),
               B200_ERR_INVALID_ARG, "layer_norm_backward: bad dtype enum");
  B200_REQUIRE(cols > 0 || rows == 0, B200_ERR_INVALID_ARG, "layer_norm_backward: cols must be positive");
  B200_REQUIRE(cols <= INT32_MAX, B200_ERR_UNSUPPORTED, "layer_norm_backward: too many columns");
  B200_REQUIRE(dy_dtype == dx_dtype || (x_dtype == B200_F32 && dy_dtype == B200_BF16 && dx_dtype == B200_F32),
               B200_ERR_UNSUPPORTED,
               "layer_norm_backward: dx takes the dtype of dy (or fp32 for a bf16 dy and an fp32 x)");
  if (rows == 0) {
    // no rows: the parameter gradients are zero
    if (dgamma != nullptr && cudaMemsetAsync(dgamma, 0, (size_t)cols * dtype_size(param_dtype), stream) != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "layer_norm_backward: memset failed");
    if (dbeta != nullptr && cudaMemsetAsync(dbeta, 0, (size_t)cols * dtype_size(param_dtype), stream) != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "layer_norm_backward: memset failed");
    if (dx_sum != nullptr && cudaMemsetAsync(dx_sum, 0, (size_t)cols * dtype_size(dx_sum_dtype), stream) != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "layer_norm_backward: memset failed");
    return B200_OK;
  }
  B200_REQUIRE(dy != nullptr && x != nullptr && mean != nullptr && rstd != nullptr && dx != nullptr,
               B200_ERR_INVALID_ARG, "layer_norm_backward: null pointer");
  B200_REQUIRE((dy_row_stride >= cols && x_row_stride >= cols) || rows == 1, B200_ERR_INVALID_ARG,
               "layer_norm_backward: row stride smaller than cols");
  B200_REQUIRE(aligned_to(dy, dtype_size(dy_dtype)) && aligned_to(x, dtype_size(x_dtype)) &&
                   aligned_to(dx, dtype_size(dx_dtype)) && aligned_to(dx_add, dtype_size(dx_dtype)) &&
                   aligned_to(dx_cast, 2) && (dx_sum == nullptr || aligned_to(dx_sum, dtype_size(dx_sum_dtype))),
               B200_ERR_ALIGNMENT, "layer_norm_backward: pointer not element aligned");
  const size_t need = b200_layer_norm_backward_workspace_bytes(rows, cols);
  B200_REQUIRE(workspace != nullptr && workspace_bytes >= need, B200_ERR_WORKSPACE,
               "layer_norm_backward: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  B200_REQUIRE(aligned_to(workspace, 16), B200_ERR_ALIGNMENT, "layer_norm_backward: workspace not 16-byte aligned");
  float* ws = static_cast<float*>(workspace);
#define LNB_CASE_D(TX, TG, TP, TD)                                                                                  \
  return launch_layer_norm_backward<TX, TG, TP, TD>(dy, x, mean, rstd, gamma, dx_add, dx, dgamma, dbeta, dx_cast,   \
                                                    dx_sum, dx_sum_dtype, ws, rows, cols, dy_row_stride,             \
                                                    x_row_stride, stream)
#define LNB_CASE(TX, TG, TP) LNB_CASE_D(TX, TG, TP, TG)
  if (dx_dtype != dy_dtype) {  // fp32 x, bf16 dy, fp32 dx: the gradient of a bf16 consumer of an fp32 stream
    if (param_dtype == B200_F32) LNB_CASE_D(float, bf16, float, float);
    LNB_CASE_D(float, bf16, bf16, float);
  }
  const int key = x_dtype * 4 + dy_dtype * 2 + param_dtype;
  switch (key) {
    case 0: LNB_CASE(float, float, float);
    case 1: LNB_CASE(float, float, bf16);
    case 2: LNB_CASE(float, bf16, float);
    case 3: LNB_CASE(float, bf16, bf16);
    case 4: LNB_CASE(bf16, float, float);
    case 5: LNB_CASE(bf16, float, bf16);
    case 6: LNB_CASE(bf16, bf16, float);
    default: LNB_CASE(bf16, bf16, bf16);
  }
#undef LNB_CASE
#undef LNB_CASE_D
}

extern "C" B200_API size_t b200_sum_rows_workspace_bytes(int64_t rows, int64_t cols, int32_t in_dtype) {
  if (rows <= 0 || cols <= 0 || !valid_dtype(in_dtype)) return 0;
  return (size_t)sum_rows_parts(rows, cols, dtype_size(in_dtype)) * (size_t)cols * sizeof(float);
}

extern "C" B200_API int32_t b200_sum_rows(const void* x, void* y, void* workspace, size_t workspace_bytes, int64_t rows,
                                          int64_t cols, int64_t x_row_stride, int32_t in_dtype, int32_t out_dtype,
                                          b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "sum_rows: negative size");
  B200_REQUIRE(valid_dtype(in_dtype) && valid_dtype(out_dtype), B200_ERR_INVALID_ARG, "sum_rows: bad dtype enum");
  B200_REQUIRE(cols <= INT32_MAX, B200_ERR_UNSUPPORTED, "sum_rows: too many columns");
  if (cols == 0) return B200_OK;
  B200_REQUIRE(y != nullptr, B200_ERR_INVALID_ARG, "sum_rows: null pointer");
  if (rows == 0) {
    if (cudaMemsetAsync(y, 0, (size_t)cols * dtype_size(out_dtype), stream) != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "sum_rows: memset failed");
    return B200_OK;
  }
  B200_REQUIRE(x != nullptr, B200_ERR_INVALID_ARG, "sum_rows: null pointer");
  B200_REQUIRE(x_row_stride >= cols || rows == 1, B200_ERR_INVALID_ARG, "sum_rows: row stride smaller than cols");
  B200_REQUIRE(aligned_to(x, dtype_size(in_dtype)) && aligned_to(y, dtype_size(out_dtype)), B200_ERR_ALIGNMENT,
               "sum_rows: pointer not element aligned");
  const size_t need = b200_sum_rows_workspace_bytes(rows, cols, in_dtype);
  B200_REQUIRE(workspace != nullptr && workspace_bytes >= need, B200_ERR_WORKSPACE,
               "sum_rows: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  B200_REQUIRE(aligned_to(workspace, 16), B200_ERR_ALIGNMENT, "sum_rows: workspace not 16-byte aligned");
  float* ws = static_cast<float*>(workspace);
  if (in_dtype == B200_F32)
    return out_dtype == B200_F32 ? launch_sum_rows<float, float>(x, y, ws, rows, cols, x_row_stride, stream)
                                 : launch_sum_rows<float, bf16>(x, y, ws, rows, cols, x_row_stride, stream);
  return out_dtype == B200_F32 ? launch_sum_rows<bf16, float>(x, y, ws, rows, cols, x_row_stride, stream)
                               : launch_sum_rows<bf16, bf16>(x, y, ws, rows, cols, x_row_stride, stream);
}

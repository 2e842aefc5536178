// Attention forward for a handful of query rows (decode: one new token against a KV cache).
// The work is reading K and V once, so it is HBM bound and the only question is how many SMs
// pull on it: with one CTA per (batch, head) a small batch would leave most of the GPU idle.
// Each (batch, head, query row) is therefore given a cluster of eight CTAs; CTA r of the cluster
// takes the r-th eighth of the keys, computes a partial softmax (its own maximum m_r, sum l_r and
// unnormalised output o_r), and the cluster's first CTA merges the eight partials straight out of
// its peers' shared memory (distributed shared memory) - no scratch buffer in HBM, no second
// launch:   m = max m_r,  l = sum l_r e^(m_r - m),  O = sum o_r e^(m_r - m) / l.
//
// Inside a CTA (128 threads): scores one key per thread (the query row sits in shared memory,
// scaled), block-wide maximum and sum, then P V with two head dimensions per thread and the keys
// spread over 128 / (D/2) thread groups, so every V row is read with consecutive threads on
// consecutive addresses.
//
// fp32 or bf16 tensors, head_dim 32 / 64 / 128, arbitrary (batch, head, position) strides with
// the head dimension contiguous, causal masks aligned to the top-left corner like
// torch.nn.functional.scaled_dot_product_attention.
#include "ptx.cuh"
#include "sdpa_internal.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 128;
constexpr int kCluster = 8;
constexpr int kMaxChunk = 4096;  // keys per CTA (their scores live in shared memory)
constexpr int kMaxRows = 16;     // query rows above this take the other kernels
constexpr int kMaxD = 128;

__device__ __forceinline__ float ld_peer_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__device__ float block_reduce(float v, float* red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) t = is_max ? nan_max(t, red[i]) : t + red[i];
  return t;
}

// VEC: K and V rows are read as 16-byte vectors (pointers and strides 16-byte friendly).
// D is a template parameter so that the per-key loops unroll and all loads of a row are in flight
// together: with ~130 keys per CTA the kernel is one latency chain, not a streaming loop.
template <typename T, int D, bool VEC>
__global__ void __launch_bounds__(kThreads)
sdpa_decode_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                   T* __restrict__ O, float* __restrict__ LSE, int64_t heads, int64_t q_len,
                   int64_t kv_len, int64_t qs_b, int64_t qs_h, int64_t qs_t, int64_t ks_b,
                   int64_t ks_h, int64_t ks_t, int64_t vs_b, int64_t vs_h, int64_t vs_t,
                   int64_t os_b, int64_t os_h, int64_t os_t, float scale, int causal, int chunk) {
  constexpr int N = VEC ? Elem<T>::kVec : 2;  // head dims per thread in the P V phase
  constexpr int TPK = D / N;                  // threads per key
  constexpr int GROUPS = kThreads / TPK;      // keys in flight per pass over the chunk
  static_assert(D % N == 0 && kThreads % TPK == 0 && TPK <= kThreads, "head_dim does not tile the CTA");
  // shared: q[D] | partial: m, l, o[D] | red[8] | group partial sums [GROUPS][D] | scores[chunk]
  extern __shared__ __align__(16) float dsm[];
  float* q_s = dsm;
  float* part = q_s + kMaxD;        // part[0] = m, part[1] = l, part[2 .. 2+D) = o
  float* red = part + 2 + kMaxD;
  float* grp = red + 8;
  float* sc = grp + GROUPS * D;

  const uint32_t rank = ptx::cluster_ctarank();
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / heads, h = bh % heads;
  const int64_t row = blockIdx.z;
  const int tid = threadIdx.x;

  const T* qp = Q + b * qs_b + h * qs_h + row * qs_t;
  for (int d = tid; d < D; d += kThreads) q_s[d] = Elem<T>::to_f32(qp[d]) * scale;

  int64_t kv_end = kv_len;
  if (causal && row + 1 < kv_end) kv_end = row + 1;
  const int64_t k0 = (int64_t)rank * chunk;
  int n = 0;  // keys of this CTA
  if (k0 < kv_end) n = (int)(kv_end - k0 < chunk ? kv_end - k0 : chunk);
  __syncthreads();

  // ---- scores: one key per thread ----
  const T* kbase = K + b * ks_b + h * ks_h + k0 * ks_t;
  float local_max = -INFINITY;
  for (int j = tid; j < n; j += kThreads) {
    const T* kr = kbase + (int64_t)j * ks_t;
    float s0 = 0.0f, s1 = 0.0f;
    if (VEC) {
      constexpr int KV = Elem<T>::kVec;
      float kv[D / KV][KV];
#pragma unroll
      for (int c = 0; c < D / KV; ++c) load16_stream(kr + c * KV, kv[c]);
#pragma unroll
      for (int c = 0; c < D / KV; ++c) {
#pragma unroll
        for (int e = 0; e < KV; e += 2) {
          s0 = fmaf(q_s[c * KV + e], kv[c][e], s0);
          s1 = fmaf(q_s[c * KV + e + 1], kv[c][e + 1], s1);
        }
      }
    } else {
#pragma unroll 8
      for (int d = 0; d < D; d += 2) {
        s0 = fmaf(q_s[d], Elem<T>::to_f32(kr[d]), s0);
        s1 = fmaf(q_s[d + 1], Elem<T>::to_f32(kr[d + 1]), s1);
      }
    }
    const float s = s0 + s1;
    sc[j] = s;
    local_max = nan_max(local_max, s);
  }
  const float m = block_reduce(local_max, red, true);
  float local_sum = 0.0f;
  for (int j = tid; j < n; j += kThreads) {
    const float pj = expf(sc[j] - m);  // n > 0 implies a finite or NaN m
    sc[j] = pj;
    local_sum += pj;
  }
  const float l = block_reduce(local_sum, red, false);  // also publishes sc[] to every thread

  // ---- P V: N head dims per thread, keys spread over the thread groups ----
  const int g = tid / TPK, dd = (tid - g * TPK) * N;
  const T* vbase = V + b * vs_b + h * vs_h + k0 * vs_t + dd;
  float acc[N];
#pragma unroll
  for (int e = 0; e < N; ++e) acc[e] = 0.0f;
#pragma unroll 4
  for (int j = g; j < n; j += GROUPS) {
    const T* vr = vbase + (int64_t)j * vs_t;
    const float pj = sc[j];
    float vv[N];
    if (VEC) {
      load16_stream(vr, reinterpret_cast<float(&)[Elem<T>::kVec]>(vv));
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) vv[e] = Elem<T>::to_f32(vr[e]);
    }
#pragma unroll
    for (int e = 0; e < N; ++e) acc[e] = fmaf(pj, vv[e], acc[e]);
  }
#pragma unroll
  for (int e = 0; e < N; ++e) grp[g * D + dd + e] = acc[e];
  __syncthreads();
  for (int d = tid; d < D; d += kThreads) {
    float t = 0.0f;
#pragma unroll
    for (int gg = 0; gg < GROUPS; ++gg) t += grp[gg * D + d];
    part[2 + d] = t;
  }
  if (tid == 0) {
    part[0] = n > 0 ? m : -INFINITY;
    part[1] = n > 0 ? l : 0.0f;
  }

  // ---- merge the cluster's partials in its first CTA ----
  ptx::cluster_sync();  // every CTA's partial is written (release/acquire at cluster scope)
  if (rank == 0) {
    const uint32_t part_addr = ptx::smem_u32(part);
    float m_all = -INFINITY;
    float m_r[kCluster], l_r[kCluster];
#pragma unroll
    for (int r = 0; r < kCluster; ++r) {
      const uint32_t peer = ptx::mapa(part_addr, (uint32_t)r);
      m_r[r] = ld_peer_f32(peer);
      l_r[r] = ld_peer_f32(peer + 4);
      m_all = nan_max(m_all, m_r[r]);
    }
    float l_all = 0.0f;
    float w_r[kCluster];
#pragma unroll
    for (int r = 0; r < kCluster; ++r) {
      w_r[r] = (m_r[r] == -INFINITY) ? 0.0f : expf(m_r[r] - m_all);
      l_all += l_r[r] * w_r[r];
    }
    // no visible key at all (kv_len == 0): l_all == 0 and 0/0 gives NaN like torch
    const float inv = 1.0f / l_all;
    T* op = O + b * os_b + h * os_h + row * os_t;
    for (int d = tid; d < D; d += kThreads) {
      float t = 0.0f;
#pragma unroll
      for (int r = 0; r < kCluster; ++r)
        t += ld_peer_f32(ptx::mapa(part_addr, (uint32_t)r) + 8u + 4u * (uint32_t)d) * w_r[r];
      op[d] = Elem<T>::from_f32(t * inv);
    }
    if (LSE != nullptr && tid == 0) LSE[(b * heads + h) * q_len + row] = m_all + logf(l_all);
  }
  ptx::cluster_sync();  // peers keep their shared memory alive until the merge has read it
}

template <typename T, int D>
int32_t launch_d(const b200_sdpa_args& a, cudaStream_t stream) {
  int64_t chunk = (a.kv_len + kCluster - 1) / kCluster;
  if (chunk < 1) chunk = 1;
  const int64_t es = (int64_t)sizeof(T);
  bool vec = true;
  for (const void* ptr : {a.k, a.v}) vec = vec && aligned_to(ptr, 16);
  for (int i = 0; i < 3; ++i) vec = vec && (a.k_strides[i] * es) % 16 == 0 && (a.v_strides[i] * es) % 16 == 0;
  // the group partial sums take 128 * (head dims per thread) floats in either variant
  const size_t smem = (size_t)(kMaxD + 2 + kMaxD + 8 + kThreads * Elem<T>::kVec + chunk) * sizeof(float);
  auto kernel = vec ? sdpa_decode_kernel<T, D, true> : sdpa_decode_kernel<T, D, false>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kCluster, (unsigned)(a.batch * a.heads), (unsigned)a.q_len);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(
      &cfg, kernel, static_cast<const T*>(a.q), static_cast<const T*>(a.k), static_cast<const T*>(a.v),
      static_cast<T*>(a.o), a.lse, a.heads, a.q_len, a.kv_len, a.q_strides[0], a.q_strides[1],
      a.q_strides[2], a.k_strides[0], a.k_strides[1], a.k_strides[2], a.v_strides[0], a.v_strides[1],
      a.v_strides[2], a.o_strides[0], a.o_strides[1], a.o_strides[2], a.scale, (int)a.causal, (int)chunk);
  if (e != cudaSuccess) B200_FAIL(B200_ERR_CUDA, "sdpa(decode): launch failed: %s", cudaGetErrorString(e));
  return B200_OK;
}

template <typename T>
int32_t launch(const b200_sdpa_args& a, cudaStream_t stream) {
  if (a.head_dim == 32) return launch_d<T, 32>(a, stream);
  if (a.head_dim == 64) return launch_d<T, 64>(a, stream);
  return launch_d<T, 128>(a, stream);
}

}  // namespace

const char* sdpa_decode_ineligible(const b200_sdpa_args& a) {
  if (a.q_len > kMaxRows) return "more than 16 query rows";
  if (a.head_dim != 32 && a.head_dim != 64 && a.head_dim != 128) return "head_dim is not 32, 64 or 128";
  if (a.kv_len > (int64_t)kCluster * kMaxChunk) return "more than 32768 keys";
  if (a.batch * a.heads > 65535) return "batch*heads above 65535";
  return nullptr;
}

int32_t launch_sdpa_decode(const b200_sdpa_args& a, cudaStream_t stream) {
  return a.dtype == B200_F32 ? launch<float>(a, stream) : launch<__nv_bfloat16>(a, stream);
}

}  // namespace b200

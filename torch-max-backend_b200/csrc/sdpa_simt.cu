// Generic scaled-dot-product attention forward on CUDA cores: fp32 or bf16 tensors, any
// head_dim <= 128, causal or full, arbitrary (batch, head, position) strides, fp32 online
// softmax. It is the exact-fp32 route and the route for shapes the tensor-core kernel does not
// take. One warp per query row, four rows per CTA sharing K/V tiles of 32 keys in shared memory.
#include "common.cuh"
#include "sdpa_internal.cuh"

namespace b200 {
namespace {

constexpr int kRowsPerCta = 4;
constexpr int kKeysPerTile = 32;
constexpr int kMaxD = 128;

template <typename T>
__global__ void __launch_bounds__(kRowsPerCta * 32)
sdpa_simt_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                 T* __restrict__ O, float* __restrict__ LSE, int64_t heads, int64_t q_len,
                 int64_t kv_len, int D, int64_t qs_b, int64_t qs_h, int64_t qs_t, int64_t ks_b,
                 int64_t ks_h, int64_t ks_t, int64_t vs_b, int64_t vs_h, int64_t vs_t,
                 int64_t os_b, int64_t os_h, int64_t os_t, float scale, int causal) {
  extern __shared__ float smem[];
  const int DP = D + 1;  // padded row pitch: lanes walk different banks
  float* q_s = smem;                                   // [kRowsPerCta][D]
  float* k_s = q_s + kRowsPerCta * D;                  // [kKeysPerTile][DP]
  float* v_s = k_s + kKeysPerTile * DP;                // [kKeysPerTile][DP]

  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / heads, h = bh % heads;
  const int64_t row0 = (int64_t)blockIdx.x * kRowsPerCta;
  const int64_t row = row0 + w;
  const bool row_ok = row < q_len;

  const T* qp = Q + b * qs_b + h * qs_h + row * qs_t;
  for (int d = lane; d < D; d += 32) q_s[w * D + d] = row_ok ? Elem<T>::to_f32(qp[d]) * scale : 0.0f;

  float o[kMaxD / 32];
#pragma unroll
  for (int i = 0; i < kMaxD / 32; ++i) o[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;

  int64_t last_row = row0 + kRowsPerCta - 1;
  if (last_row >= q_len) last_row = q_len - 1;
  const int64_t kv_end = causal ? (last_row + 1 < kv_len ? last_row + 1 : kv_len) : kv_len;
  const T* kbase = K + b * ks_b + h * ks_h;
  const T* vbase = V + b * vs_b + h * vs_h;

  for (int64_t j0 = 0; j0 < kv_end; j0 += kKeysPerTile) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < kKeysPerTile * D; idx += blockDim.x) {
      const int j = idx / D, d = idx - j * D;
      const int64_t key = j0 + j;
      float kv = 0.0f, vv = 0.0f;
      if (key < kv_len) {
        kv = Elem<T>::to_f32(kbase[key * ks_t + d]);
        vv = Elem<T>::to_f32(vbase[key * vs_t + d]);
      }
      k_s[j * DP + d] = kv;
      v_s[j * DP + d] = vv;
    }
    __syncthreads();
    if (!row_ok) continue;
    const int64_t key = j0 + lane;
    const bool allowed = key < kv_len && (!causal || key <= row);
    float s = 0.0f;
    for (int d = 0; d < D; ++d) s = fmaf(q_s[w * D + d], k_s[lane * DP + d], s);
    s = allowed ? s : -INFINITY;
    const float tile_max = warp_max(s);
    const float m_new = nan_max(m, tile_max);
    if (m_new == -INFINITY) continue;  // every key of this tile is masked for this row
    const float corr = expf(m - m_new);
    const float pj = allowed ? expf(s - m_new) : 0.0f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) o[i] *= corr;
    for (int j = 0; j < kKeysPerTile; ++j) {
      const float p = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
      for (int i = 0; i < kMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) o[i] = fmaf(p, v_s[j * DP + d], o[i]);
      }
    }
  }
  if (!row_ok) return;
  // A row with no allowed key (kv_len == 0) has l == 0: 0/0 gives NaN like torch.
  const float inv = 1.0f / l;
  T* op = O + b * os_b + h * os_h + row * os_t;
#pragma unroll
  for (int i = 0; i < kMaxD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) op[d] = Elem<T>::from_f32(o[i] * inv);
  }
  if (LSE != nullptr && lane == 0) LSE[(b * heads + h) * q_len + row] = m + logf(l);
}

template <typename T>
int32_t launch(const b200_sdpa_args& a, cudaStream_t stream) {
  const int D = (int)a.head_dim;
  const size_t smem = (size_t)(kRowsPerCta * D + 2 * kKeysPerTile * (D + 1)) * sizeof(float);
  const int64_t gx = (a.q_len + kRowsPerCta - 1) / kRowsPerCta;
  const int64_t gy = a.batch * a.heads;
  B200_REQUIRE(gx <= INT32_MAX && gy <= 65535, B200_ERR_UNSUPPORTED,
               "sdpa(simt): grid too large (q_len=%lld batch*heads=%lld)", (long long)a.q_len,
               (long long)gy);
  dim3 grid((unsigned)gx, (unsigned)gy);
  sdpa_simt_kernel<T><<<grid, kRowsPerCta * 32, smem, stream>>>(
      static_cast<const T*>(a.q), static_cast<const T*>(a.k), static_cast<const T*>(a.v),
      static_cast<T*>(a.o), a.lse, a.heads, a.q_len, a.kv_len, D, a.q_strides[0], a.q_strides[1],
      a.q_strides[2], a.k_strides[0], a.k_strides[1], a.k_strides[2], a.v_strides[0],
      a.v_strides[1], a.v_strides[2], a.o_strides[0], a.o_strides[1], a.o_strides[2], a.scale,
      a.causal);
  B200_CHECK_LAUNCH("sdpa(simt)");
  return B200_OK;
}

}  // namespace

const char* sdpa_simt_ineligible(const b200_sdpa_args& a) {
  if (a.head_dim > kMaxD) return "head_dim above 128";
  return nullptr;
}

int32_t launch_sdpa_simt(const b200_sdpa_args& a, cudaStream_t stream) {
  return a.dtype == B200_F32 ? launch<float>(a, stream) : launch<__nv_bfloat16>(a, stream);
}

}  // namespace b200

// Shared helpers for the libb200ops kernels: status plumbing, vector loads, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "b200ops.h"

namespace b200 {

// ---- host-side status plumbing -----------------------------------------------------------
// Thread-local text behind b200_last_error(); defined in abi.cu.
void set_error(const char* fmt, ...);

#define B200_FAIL(code, ...)        \
  do {                              \
    ::b200::set_error(__VA_ARGS__); \
    return (code);                  \
  } while (0)

#define B200_REQUIRE(cond, code, ...)      \
  do {                                     \
    if (!(cond)) B200_FAIL(code, __VA_ARGS__); \
  } while (0)

// Launch-error check: cudaGetLastError reports a bad launch configuration, never waits.
#define B200_CHECK_LAUNCH(what)                                                        \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess)                                                            \
      B200_FAIL(B200_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e__)); \
  } while (0)

inline bool valid_dtype(int32_t d) { return d == B200_F32 || d == B200_BF16; }
inline int dtype_size(int32_t d) { return d == B200_F32 ? 4 : 2; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Device status word: bit set by a kernel whose bounded wait ran out. One per device
// (a __device__ variable is instantiated on every device that loads the module). Kernels get
// its address as an argument; device_status_ptr() resolves it for the current device.
unsigned int* device_status_ptr();
constexpr unsigned int STATUS_GEMM_TIMEOUT = 1u << 0;
constexpr unsigned int STATUS_SDPA_TIMEOUT = 1u << 1;
constexpr unsigned int STATUS_TEST_TIMEOUT = 1u << 2;  // b200_debug_wait_timeout
constexpr unsigned int STATUS_INDEX_OUT_OF_RANGE = 1u << 3;  // an embedding index outside its table

int sm_count();  // SM count of the current device (cached per device)

// ---- device helpers ----------------------------------------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<float> {
  static constexpr int kVec = 4;  // elements per 16-byte vector
  __device__ static float to_f32(float v) { return v; }
  __device__ static float from_f32(float v) { return v; }
};

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T held as fp32 lanes.
template <typename T>
struct Vec16 {
  static constexpr int N = Elem<T>::kVec;
  float v[N];
};

__device__ __forceinline__ void load16(const float* p, float (&out)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p);
  out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
}

__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&out)[8]) {
  uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bf16 -> fp32 is a 16-bit shift of the bit pattern.
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ void store16(float* p, const float (&in)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&in)[8]) {
  uint4 t;
  t.x = pack_bf16x2(in[0], in[1]);
  t.y = pack_bf16x2(in[2], in[3]);
  t.z = pack_bf16x2(in[4], in[5]);
  t.w = pack_bf16x2(in[6], in[7]);
  *reinterpret_cast<uint4*>(p) = t;
}

// Streaming variants: data touched once should not displace reusable lines in L1.
__device__ __forceinline__ void load16_stream(const float* p, float (&out)[4]) {
  float4 t = __ldcs(reinterpret_cast<const float4*>(p));
  out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
}

__device__ __forceinline__ void load16_stream(const __nv_bfloat16* p, float (&out)[8]) {
  uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ void store16_stream(float* p, const float (&in)[4]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(in[0], in[1], in[2], in[3]));
}

__device__ __forceinline__ void store16_stream(__nv_bfloat16* p, const float (&in)[8]) {
  uint4 t;
  t.x = pack_bf16x2(in[0], in[1]);
  t.y = pack_bf16x2(in[2], in[3]);
  t.z = pack_bf16x2(in[4], in[5]);
  t.w = pack_bf16x2(in[6], in[7]);
  __stcs(reinterpret_cast<uint4*>(p), t);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// max that propagates NaN like torch.amax / softmax do.
__device__ __forceinline__ float nan_max(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));  // one instruction; NaN if either is
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = nan_max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float gelu_tanh_f32(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  const float k0 = 0.7978845608028654f;
  const float k1 = 0.044715f;
  float inner = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

__device__ __forceinline__ float gelu_erf_f32(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
}

}  // namespace b200

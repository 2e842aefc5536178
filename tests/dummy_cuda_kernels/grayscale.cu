// Test kernels for user CUDA ops: a weighted channel sum of an [H, W, 3] uint8 picture, and a
// two-output variant that adds a per-pixel uint8 noise plane to every channel first.
#include <cuda_runtime.h>

#include "b200_user_op.h"

namespace {

__device__ __forceinline__ float luminance(float r, float g, float b) { return fminf(0.21f * r + 0.71f * g + 0.07f * b, 255.0f); }

__global__ void grayscale_kernel(b200_user_tensor out, b200_user_tensor pic) {
  const int64_t h = pic.shape[0], w = pic.shape[1];
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < h * w; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t y = i / w, x = i % w;
    const uint8_t* p = static_cast<const uint8_t*>(pic.data) + y * pic.strides[0] + x * pic.strides[1];
    float* o = static_cast<float*>(out.data) + y * out.strides[0] + x * out.strides[1];
    *o = luminance(p[0], p[pic.strides[2]], p[2 * pic.strides[2]]);
  }
}

__global__ void grayscale_multi_kernel(b200_user_tensor gray, b200_user_tensor red, b200_user_tensor pic,
                                       b200_user_tensor noise) {
  const int64_t h = pic.shape[0], w = pic.shape[1];
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < h * w; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t y = i / w, x = i % w;
    const uint8_t* p = static_cast<const uint8_t*>(pic.data) + y * pic.strides[0] + x * pic.strides[1];
    const float n = static_cast<const uint8_t*>(noise.data)[y * noise.strides[0] + x * noise.strides[1]];
    const float r = p[0] + n, g = p[pic.strides[2]] + n, b = p[2 * pic.strides[2]] + n;
    static_cast<float*>(gray.data)[y * gray.strides[0] + x * gray.strides[1]] = luminance(r, g, b);
    static_cast<float*>(red.data)[y * red.strides[0] + x * red.strides[1]] = r;
  }
}

bool picture_ok(const b200_user_tensor& pic) { return pic.rank == 3 && pic.shape[2] == 3 && pic.dtype == B200_USER_U8; }
bool plane_ok(const b200_user_tensor& t, const b200_user_tensor& pic, int dtype) {
  return t.rank == 2 && t.shape[0] == pic.shape[0] && t.shape[1] == pic.shape[1] && t.dtype == dtype;
}
unsigned blocks_for(int64_t n) { return (unsigned)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184); }

}  // namespace

extern "C" int32_t grayscale(const b200_user_tensor* outputs, int32_t num_outputs, const b200_user_tensor* inputs,
                             int32_t num_inputs, void* stream) {
  if (num_outputs != 1 || num_inputs != 1) return 1;
  if (!picture_ok(inputs[0]) || !plane_ok(outputs[0], inputs[0], B200_USER_F32)) return 2;
  const int64_t n = inputs[0].shape[0] * inputs[0].shape[1];
  if (n == 0) return 0;
  grayscale_kernel<<<blocks_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(outputs[0], inputs[0]);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

extern "C" int32_t grayscale_multi(const b200_user_tensor* outputs, int32_t num_outputs, const b200_user_tensor* inputs,
                                   int32_t num_inputs, void* stream) {
  if (num_outputs != 2 || num_inputs != 2) return 1;
  if (!picture_ok(inputs[0]) || !plane_ok(inputs[1], inputs[0], B200_USER_U8) ||
      !plane_ok(outputs[0], inputs[0], B200_USER_F32) || !plane_ok(outputs[1], inputs[0], B200_USER_F32))
    return 2;
  const int64_t n = inputs[0].shape[0] * inputs[0].shape[1];
  if (n == 0) return 0;
  grayscale_multi_kernel<<<blocks_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(outputs[0], outputs[1], inputs[0],
                                                                                     inputs[1]);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

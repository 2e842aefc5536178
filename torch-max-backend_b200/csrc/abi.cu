// Library-level entry points: ABI version, status text, per-device status word.
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

__device__ unsigned int g_device_status = 0;

namespace {
thread_local char tls_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
}

unsigned int* device_status_ptr() {
  static std::mutex mu;
  static unsigned int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned int*>(p);
  }
  return cached[dev];
}

int sm_count() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

// One warp waits on an mbarrier that nothing ever signals, with the caller's limit, and then
// leaves the way the GEMM and attention kernels leave when one of their waits runs out: abort
// flag, status bit, return.
__global__ void wait_timeout_kernel(unsigned long long limit_ns, unsigned int* status) {
  __shared__ __align__(8) unsigned long long barrier_storage;
  __shared__ uint32_t abort_flag_storage;
  volatile uint32_t* abort_flag = &abort_flag_storage;
  const uint32_t bar = ptx::smem_u32(&barrier_storage);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  const bool arrived = ptx::mbar_wait_limited(bar, 0, abort_flag, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0 && (!arrived || *abort_flag != 0)) atomicOr(status, STATUS_TEST_TIMEOUT);
}

}  // namespace
}  // namespace b200

extern "C" B200_API int32_t b200_debug_wait_timeout(uint64_t limit_ns, b200_stream_t stream_) {
  using namespace b200;
  B200_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ull, B200_ERR_INVALID_ARG,
               "debug_wait_timeout: limit must be in (0, 100 ms]");
  unsigned int* status = device_status_ptr();
  B200_REQUIRE(status != nullptr, B200_ERR_CUDA, "debug_wait_timeout: device status word unavailable");
  wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(limit_ns, status);
  B200_CHECK_LAUNCH("debug_wait_timeout");
  return B200_OK;
}

extern "C" B200_API int32_t b200_abi_version(void) { return B200_ABI_VERSION; }

extern "C" B200_API const char* b200_status_string(int32_t status) {
  switch (status) {
    case B200_OK: return "ok";
    case B200_ERR_INVALID_ARG: return "invalid argument";
    case B200_ERR_UNSUPPORTED: return "unsupported request";
    case B200_ERR_ALIGNMENT: return "misaligned pointer or stride";
    case B200_ERR_WORKSPACE: return "workspace missing or too small";
    case B200_ERR_CUDA: return "CUDA call failed";
    case B200_ERR_DEVICE_TIMEOUT: return "bounded device-side wait gave up";
    default: return "unknown status";
  }
}

extern "C" B200_API const char* b200_last_error(void) { return b200::tls_error; }

extern "C" B200_API int32_t b200_device_status(uint32_t* word) {
  B200_REQUIRE(word != nullptr, B200_ERR_INVALID_ARG, "device_status: null pointer");
  unsigned int host = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&host, b200::g_device_status, sizeof(host));
  if (e != cudaSuccess)
    B200_FAIL(B200_ERR_CUDA, "device_status: read failed: %s", cudaGetErrorString(e));
  if (host != 0) {
    const unsigned int zero = 0;
    e = cudaMemcpyToSymbol(b200::g_device_status, &zero, sizeof(zero));
    if (e != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "device_status: clear failed: %s", cudaGetErrorString(e));
  }
  *word = host;
  return host == 0 ? B200_OK : B200_ERR_DEVICE_TIMEOUT;
}

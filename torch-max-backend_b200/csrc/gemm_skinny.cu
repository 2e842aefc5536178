// Small-M (decode-shaped) GEMM: the weights are read once and the problem is HBM-bound, but with
// few rows there are too few output tiles to keep every SM streaming. The K range is therefore
// split across CTAs: stage 1 writes fp32 partial sums into a scratch buffer [splits, m, n] -- the
// tensor-core kernel in batched mode (one "batch" per K slice) for 9 to 128 bf16 rows, the
// CUDA-core kernels of gemm_gemv.cu for up to 8 rows of either dtype -- and a second kernel adds
// the slices in a fixed order (deterministic, no atomics) and applies the epilogue.
//
// The scratch buffer is the caller's workspace (b200_gemm_workspace_bytes says how large).
#include "gemm_internal.cuh"

#include <mutex>

namespace b200 {
namespace {

// Scratch for b200_gemm_small_m_static: lives in the library image, so every GPU that loads the
// library holds these bytes until the process exits. In host code this name is only a stand-in
// for the symbol (not a device address); static_scratch_ptr() asks the runtime for the real one.
static __device__ __align__(256) unsigned char g_static_scratch[B200_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
void* static_scratch_ptr() {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("gemm_small_m_static: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("gemm_small_m_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = ptr;
  }
  return cached[dev];
}

constexpr int kReduceThreads = 256;

struct ReduceParams {
  const float* partial;  // [splits, m, n]
  const void* bias;
  const void* residual;
  int64_t m, n, splits;
  int64_t c_rs, bias_rs, residual_rs;
  float alpha, beta;
  int32_t bias_dtype, residual_dtype, epilogue;
};

__device__ __forceinline__ float ld_any(const void* p, int64_t idx, int32_t dtype) {
  return dtype == B200_F32 ? __ldg(static_cast<const float*>(p) + idx)
                           : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

// One thread per output element; consecutive threads walk a row, so partial reads and the
// store are coalesced. Slices are added in index order.
template <typename Tout>
__global__ void __launch_bounds__(kReduceThreads)
splitk_reduce_kernel(Tout* __restrict__ C, ReduceParams p) {
  const int64_t idx = (int64_t)blockIdx.x * kReduceThreads + threadIdx.x;
  const int64_t total = p.m * p.n;
  if (idx >= total) return;
  const int64_t row = idx / p.n, col = idx - row * p.n;
  float acc = 0.0f;
  for (int64_t s = 0; s < p.splits; ++s) acc += __ldg(p.partial + s * total + idx);
  float v = p.alpha * acc;
  if (p.bias != nullptr) v += p.beta * ld_any(p.bias, row * p.bias_rs + col, p.bias_dtype);
  if (p.epilogue == B200_EPILOGUE_GELU_TANH) v = gelu_tanh_f32(v);
  else if (p.epilogue == B200_EPILOGUE_GELU_ERF) v = gelu_erf_f32(v);
  if (p.residual != nullptr) v += ld_any(p.residual, row * p.residual_rs + col, p.residual_dtype);
  C[row * p.c_rs + col] = Elem<Tout>::from_f32(v);
}

}  // namespace

// Number of K slices for these arguments; < 2 means the route does not apply.
int gemm_skinny_splits(const b200_gemm_args& g) {
  if (g.batch != 1 || g.m > 128 || g.m <= 0) return 0;
  if (gemm_tcgen05_ineligible(g) != nullptr) return 0;
  const int64_t tiles = (g.n + 127) / 128;
  const int64_t by_sm = sm_count() / (tiles > 0 ? tiles : 1);
  // scratch traffic (write + read of fp32 partials) must stay well below the weight bytes
  const int64_t by_traffic = g.k / (8 * g.m);
  int64_t limit = by_sm < by_traffic ? by_sm : by_traffic;
  if (limit > 16) limit = 16;
  for (int64_t s = limit; s >= 2; --s)
    if (g.k % (s * 64) == 0) return (int)s;  // every slice a whole number of 64-wide k-blocks
  return 0;
}

const char* gemm_skinny_ineligible(const b200_gemm_args& g) {
  if (gemm_gemv_ineligible(g) == nullptr) return nullptr;  // up to 8 rows: the CUDA-core stage 1
  if (g.batch != 1) return "batched";
  if (g.m > 128) return "more than 128 rows";
  if (gemm_tcgen05_ineligible(g) != nullptr) return "operands not eligible for the tensor-core kernel";
  if (gemm_skinny_splits(g) < 2) return "no useful K split (few SMs idle, shallow K, or K not divisible)";
  return nullptr;
}

size_t gemm_skinny_scratch_bytes(const b200_gemm_args& g) {
  if (gemm_gemv_ineligible(g) == nullptr) return gemm_gemv_scratch_bytes(g);
  const int s = gemm_skinny_splits(g);
  return s < 2 ? 0 : (size_t)s * (size_t)g.m * (size_t)g.n * sizeof(float);
}

int32_t launch_gemm_skinny(const b200_gemm_args& g, void* scratch, size_t scratch_bytes, cudaStream_t stream) {
  const bool gemv = gemm_gemv_ineligible(g) == nullptr;
  // up to eight rows against a K-contiguous weight: partial sums, their sum and the epilogue in one launch
  if (gemv && gemm_gemv_one_launch(g)) return launch_gemm_gemv_one_launch(g, stream);
  const int splits = gemv ? gemm_gemv_slices(g) : gemm_skinny_splits(g);
  B200_REQUIRE(gemv || splits >= 2, B200_ERR_UNSUPPORTED, "gemm(skinny): no K split for these arguments");
  const size_t need = (size_t)splits * (size_t)g.m * (size_t)g.n * sizeof(float);
  B200_REQUIRE(scratch != nullptr && scratch_bytes >= need, B200_ERR_WORKSPACE,
               "gemm(skinny): scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  B200_REQUIRE(aligned_to(scratch, 16), B200_ERR_ALIGNMENT, "gemm(skinny): scratch not 16-byte aligned");

  if (gemv) {
    // Stage 1 on the CUDA cores: fp32 partial sums of every (column block, K slice).
    const int32_t st = launch_gemm_gemv_partials(g, static_cast<float*>(scratch), splits, stream);
    if (st != B200_OK) return st;
  } else {
  // Stage 1: batched tensor-core GEMM, one batch per K slice, fp32 partials into the scratch.
  b200_gemm_args part = g;
  const int64_t ks = g.k / splits;
  part.k = ks;
  part.batch = splits;
  part.a_batch_stride = ks * g.a_col_stride;  // a_col_stride == 1 on this route
  part.b_batch_stride = ks * g.b_row_stride;
  part.c = scratch;
  part.c_row_stride = g.n;
  part.c_batch_stride = g.m * g.n;
  part.bias = nullptr;
  part.residual = nullptr;
  part.alpha = 1.0f;
  part.beta = 0.0f;
  part.epilogue = B200_EPILOGUE_NONE;
  part.out_dtype = B200_F32;
  part.route = B200_ROUTE_TCGEN05;
  const char* why = gemm_tcgen05_ineligible(part);
  B200_REQUIRE(why == nullptr, B200_ERR_UNSUPPORTED, "gemm(skinny): K slices not eligible: %s", why);
  int32_t st = launch_gemm_tcgen05(part, stream);
  if (st != B200_OK) return st;
  }

  // Stage 2: add the slices and apply the epilogue.
  ReduceParams rp;
  rp.partial = static_cast<const float*>(scratch);
  rp.bias = g.bias; rp.residual = g.residual;
  rp.m = g.m; rp.n = g.n; rp.splits = splits;
  rp.c_rs = g.c_row_stride; rp.bias_rs = g.bias_row_stride; rp.residual_rs = g.residual_row_stride;
  rp.alpha = g.alpha; rp.beta = g.beta;
  rp.bias_dtype = g.bias_dtype; rp.residual_dtype = g.residual_dtype; rp.epilogue = g.epilogue;
  const int64_t total = g.m * g.n;
  const unsigned grid = (unsigned)((total + kReduceThreads - 1) / kReduceThreads);
  if (g.out_dtype == B200_F32)
    splitk_reduce_kernel<float><<<grid, kReduceThreads, 0, stream>>>(static_cast<float*>(g.c), rp);
  else
    splitk_reduce_kernel<__nv_bfloat16><<<grid, kReduceThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(g.c), rp);
  B200_CHECK_LAUNCH("gemm(skinny reduce)");
  return B200_OK;
}

}  // namespace b200

// The split-K small-M GEMM with its scratch taken from the library's own static device array
// instead of a caller-provided workspace. See include/b200ops.h for the contract.
extern "C" B200_API int32_t b200_gemm_small_m_static(const b200_gemm_args* args, b200_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // the same checks as b200_gemm, before anything is launched
  const int32_t st = validate_gemm_args(args);
  if (st != B200_OK) return st;
  const b200_gemm_args& g = *args;
  B200_REQUIRE(g.m > 0 && g.n > 0 && g.k > 0 && g.batch == 1, B200_ERR_INVALID_ARG,
               "gemm_small_m_static: needs one non-empty problem (batch == 1)");
  const char* why = gemm_skinny_ineligible(g);
  B200_REQUIRE(why == nullptr, B200_ERR_UNSUPPORTED,
               "gemm_small_m_static: these arguments do not take the split-K route (%s); use b200_gemm", why);
  const size_t need = gemm_skinny_scratch_bytes(g);
  B200_REQUIRE(need <= (size_t)B200_STATIC_SCRATCH_BYTES, B200_ERR_WORKSPACE,
               "gemm_small_m_static: needs %zu bytes of scratch, the static array holds %d; use b200_gemm with a "
               "workspace", need, B200_STATIC_SCRATCH_BYTES);
  void* scratch = static_scratch_ptr();
  if (scratch == nullptr) return B200_ERR_CUDA;
  // Every partial element is written by the first stage before the second reads it, so nothing
  // left over from an earlier call is ever read and the array needs no clearing.
  return launch_gemm_skinny(g, scratch, (size_t)B200_STATIC_SCRATCH_BYTES, stream);
}

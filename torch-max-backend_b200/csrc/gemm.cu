// b200_gemm: argument validation and route selection. No kernel lives here.
#include "gemm_internal.cuh"

namespace b200 {

int32_t validate_gemm_args(const b200_gemm_args* a) {
  B200_REQUIRE(a != nullptr, B200_ERR_INVALID_ARG, "gemm: null args");
  const b200_gemm_args& g = *a;
  B200_REQUIRE(g.m >= 0 && g.n >= 0 && g.k >= 0 && g.batch >= 0, B200_ERR_INVALID_ARG,
               "gemm: negative extent");
  B200_REQUIRE(valid_dtype(g.in_dtype) && valid_dtype(g.out_dtype), B200_ERR_INVALID_ARG,
               "gemm: bad dtype enum");
  B200_REQUIRE(g.bias == nullptr || valid_dtype(g.bias_dtype), B200_ERR_INVALID_ARG,
               "gemm: bad bias dtype enum");
  B200_REQUIRE(g.residual == nullptr || valid_dtype(g.residual_dtype), B200_ERR_INVALID_ARG,
               "gemm: bad residual dtype enum");
  B200_REQUIRE(g.epilogue >= B200_EPILOGUE_NONE && g.epilogue <= B200_EPILOGUE_GELU_ERF,
               B200_ERR_INVALID_ARG, "gemm: bad epilogue enum");
  B200_REQUIRE(g.route >= B200_ROUTE_AUTO && g.route <= B200_ROUTE_SPLIT3, B200_ERR_INVALID_ARG,
               "gemm: bad route enum");
  if (g.m == 0 || g.n == 0 || g.batch == 0) return B200_OK;
  B200_REQUIRE(g.c != nullptr, B200_ERR_INVALID_ARG, "gemm: null output");
  B200_REQUIRE(g.k == 0 || (g.a != nullptr && g.b != nullptr), B200_ERR_INVALID_ARG,
               "gemm: null operand");
  B200_REQUIRE(g.c_row_stride >= g.n || g.m == 1, B200_ERR_INVALID_ARG,
               "gemm: output row stride smaller than n");
  B200_REQUIRE(aligned_to(g.a, dtype_size(g.in_dtype)) && aligned_to(g.b, dtype_size(g.in_dtype)) &&
                   aligned_to(g.c, dtype_size(g.out_dtype)),
               B200_ERR_ALIGNMENT, "gemm: pointer not element aligned");
  B200_REQUIRE(g.bias == nullptr || aligned_to(g.bias, dtype_size(g.bias_dtype)), B200_ERR_ALIGNMENT,
               "gemm: bias pointer not element aligned");
  B200_REQUIRE(g.residual == nullptr || aligned_to(g.residual, dtype_size(g.residual_dtype)), B200_ERR_ALIGNMENT,
               "gemm: residual pointer not element aligned");
  B200_REQUIRE(g.residual == nullptr || g.residual_row_stride >= g.n || g.m == 1, B200_ERR_INVALID_ARG,
               "gemm: residual row stride smaller than n");
  B200_REQUIRE(g.batch == 1 || ((g.bias == nullptr || g.bias_row_stride == 0) && g.residual == nullptr),
               B200_ERR_UNSUPPORTED, "gemm: matrix bias/residual with batch > 1");
  return B200_OK;
}

namespace {

// Below this many multiply-adds an fp32 product stays on the exact CUDA-core kernel: the two split
// launches in front of the tensor-core launch would cost more than they save.
constexpr double kSplitMinMacs = 16777216.0;  // 2^24

int32_t resolve_route(const b200_gemm_args& g) {
  if (g.route == B200_ROUTE_SIMT) return B200_ROUTE_SIMT;
  if (g.route == B200_ROUTE_SPLIT3) {
    const char* why = gemm_split_ineligible(g);
    if (why != nullptr) B200_FAIL(B200_ERR_UNSUPPORTED, "gemm: split-precision route refused: %s", why);
    return B200_ROUTE_SPLIT3;
  }
  // one to eight rows of either dtype: the CUDA-core small-M route (exact fp32 products)
  if (g.route == B200_ROUTE_AUTO && gemm_gemv_ineligible(g) == nullptr) return B200_ROUTE_SKINNY;
  if (g.route == B200_ROUTE_AUTO && g.in_dtype == B200_F32 && gemm_split_ineligible(g) == nullptr &&
      (double)g.m * (double)g.n * (double)g.k >= kSplitMinMacs)
    return B200_ROUTE_SPLIT3;
  const char* why_tc = gemm_tcgen05_ineligible(g);
  const char* why_skinny = gemm_skinny_ineligible(g);
  if (g.route == B200_ROUTE_TCGEN05) {
    if (why_tc != nullptr) B200_FAIL(B200_ERR_UNSUPPORTED, "gemm: tcgen05 route refused: %s", why_tc);
    return B200_ROUTE_TCGEN05;
  }
  if (g.route == B200_ROUTE_SKINNY) {
    if (why_skinny != nullptr) B200_FAIL(B200_ERR_UNSUPPORTED, "gemm: skinny route refused: %s", why_skinny);
    return B200_ROUTE_SKINNY;
  }
  if (why_skinny == nullptr) return B200_ROUTE_SKINNY;
  if (why_tc == nullptr) return B200_ROUTE_TCGEN05;
  return B200_ROUTE_SIMT;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" B200_API int32_t b200_gemm_route(const b200_gemm_args* args) {
  int32_t st = validate_gemm_args(args);
  if (st != B200_OK) return st;
  return resolve_route(*args);
}

extern "C" B200_API size_t b200_gemm_workspace_bytes(const b200_gemm_args* args) {
  if (validate_gemm_args(args) != B200_OK) return 0;
  const b200_gemm_args& g = *args;
  if (g.m == 0 || g.n == 0 || g.batch == 0) return 0;
  const int32_t route = resolve_route(g);
  if (route == B200_ROUTE_SKINNY) return gemm_skinny_scratch_bytes(g);
  if (route == B200_ROUTE_SPLIT3) return gemm_split_scratch_bytes(g);
  return 0;
}

extern "C" B200_API int32_t b200_gemm(const b200_gemm_args* args, void* workspace, size_t workspace_bytes,
                             b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int32_t st = validate_gemm_args(args);
  if (st != B200_OK) return st;
  const b200_gemm_args& g = *args;
  if (g.m == 0 || g.n == 0 || g.batch == 0) return B200_OK;
  const int32_t route = resolve_route(g);
  if (route < 0) return route;
  switch (route) {
    case B200_ROUTE_TCGEN05: return launch_gemm_tcgen05(g, stream);
    case B200_ROUTE_SKINNY: return launch_gemm_skinny(g, workspace, workspace_bytes, stream);
    case B200_ROUTE_SPLIT3: return launch_gemm_split(g, workspace, workspace_bytes, stream);
    default: return launch_gemm_simt(g, stream);
  }
}

// b200_sdpa_fwd: argument validation and route selection. No kernel lives here.
#include "sdpa_internal.cuh"

namespace b200 {
namespace {

int32_t validate(const b200_sdpa_args* p) {
  B200_REQUIRE(p != nullptr, B200_ERR_INVALID_ARG, "sdpa: null args");
  const b200_sdpa_args& a = *p;
  B200_REQUIRE(a.batch >= 0 && a.heads >= 0 && a.q_len >= 0 && a.kv_len >= 0 && a.head_dim > 0,
               B200_ERR_INVALID_ARG, "sdpa: bad extent");
  B200_REQUIRE(valid_dtype(a.dtype), B200_ERR_INVALID_ARG, "sdpa: bad dtype enum");
  B200_REQUIRE(a.route == B200_ROUTE_AUTO || a.route == B200_ROUTE_SIMT || a.route == B200_ROUTE_TCGEN05 ||
                   a.route == B200_ROUTE_SKINNY,
               B200_ERR_INVALID_ARG, "sdpa: bad route enum");
  if (a.batch == 0 || a.heads == 0 || a.q_len == 0) return B200_OK;
  B200_REQUIRE(a.q != nullptr && a.o != nullptr && (a.kv_len == 0 || (a.k != nullptr && a.v != nullptr)),
               B200_ERR_INVALID_ARG, "sdpa: null pointer");
  const size_t es = dtype_size(a.dtype);
  B200_REQUIRE(aligned_to(a.q, es) && aligned_to(a.k, es) && aligned_to(a.v, es) && aligned_to(a.o, es),
               B200_ERR_ALIGNMENT, "sdpa: pointer not element aligned");
  return B200_OK;
}

int32_t resolve_route(const b200_sdpa_args& a) {
  const char* why_tc = sdpa_tcgen05_ineligible(a);
  const char* why_simt = sdpa_simt_ineligible(a);
  const char* why_decode = sdpa_decode_ineligible(a);
  if (a.route == B200_ROUTE_SKINNY) {
    if (why_decode != nullptr) B200_FAIL(B200_ERR_UNSUPPORTED, "sdpa: decode route refused: %s", why_decode);
    return B200_ROUTE_SKINNY;
  }
  // a handful of query rows would leave a 128-row tensor-core tile almost empty
  if (a.route == B200_ROUTE_AUTO && why_decode == nullptr) return B200_ROUTE_SKINNY;
  if (a.route == B200_ROUTE_TCGEN05) {
    if (why_tc != nullptr) B200_FAIL(B200_ERR_UNSUPPORTED, "sdpa: tcgen05 route refused: %s", why_tc);
    return B200_ROUTE_TCGEN05;
  }
  if (a.route == B200_ROUTE_AUTO && why_tc == nullptr) return B200_ROUTE_TCGEN05;
  if (why_simt != nullptr) B200_FAIL(B200_ERR_UNSUPPORTED, "sdpa: no kernel takes this request: %s", why_simt);
  return B200_ROUTE_SIMT;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" B200_API int32_t b200_sdpa_route(const b200_sdpa_args* args) {
  int32_t st = validate(args);
  if (st != B200_OK) return st;
  return resolve_route(*args);
}

extern "C" B200_API int32_t b200_sdpa_fwd(const b200_sdpa_args* args, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int32_t st = validate(args);
  if (st != B200_OK) return st;
  const b200_sdpa_args& a = *args;
  if (a.batch == 0 || a.heads == 0 || a.q_len == 0) return B200_OK;
  const int32_t route = resolve_route(a);
  if (route < 0) return route;
  if (route == B200_ROUTE_SKINNY) return launch_sdpa_decode(a, stream);
  return route == B200_ROUTE_TCGEN05 ? launch_sdpa_tcgen05(a, stream) : launch_sdpa_simt(a, stream);
}

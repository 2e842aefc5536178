// Small-M (decode) GEMM route. Placeholder until the weight-streaming kernel lands: reports
// itself ineligible so that the router never selects it.
#include "gemm_internal.cuh"

namespace b200 {

const char* gemm_skinny_ineligible(const b200_gemm_args&) { return "no small-M kernel in this build"; }

int32_t launch_gemm_skinny(const b200_gemm_args&, cudaStream_t) {
  B200_FAIL(B200_ERR_UNSUPPORTED, "gemm(skinny): not built");
}

}  // namespace b200

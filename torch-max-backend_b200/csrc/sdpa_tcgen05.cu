// Causal attention forward on tcgen05/TMEM. Placeholder until the kernel lands: reports itself
// ineligible so that the router never selects it.
#include "sdpa_internal.cuh"

namespace b200 {

const char* sdpa_tcgen05_ineligible(const b200_sdpa_args&) { return "no tensor-core attention kernel in this build"; }

int32_t launch_sdpa_tcgen05(const b200_sdpa_args&, cudaStream_t) {
  B200_FAIL(B200_ERR_UNSUPPORTED, "sdpa(tcgen05): not built");
}

}  // namespace b200

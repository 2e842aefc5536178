// Internal interfaces between the attention router (sdpa.cu) and its kernels.
#pragma once

#include "common.cuh"

namespace b200 {

const char* sdpa_simt_ineligible(const b200_sdpa_args& a);
int32_t launch_sdpa_simt(const b200_sdpa_args& a, cudaStream_t stream);

// Why the TMA/tcgen05 kernel cannot take these arguments, or nullptr when it can.
const char* sdpa_tcgen05_ineligible(const b200_sdpa_args& a);
int32_t launch_sdpa_tcgen05(const b200_sdpa_args& a, cudaStream_t stream);

// Few query rows against many keys (decode): split-KV over a thread-block cluster.
const char* sdpa_decode_ineligible(const b200_sdpa_args& a);
int32_t launch_sdpa_decode(const b200_sdpa_args& a, cudaStream_t stream);

}  // namespace b200

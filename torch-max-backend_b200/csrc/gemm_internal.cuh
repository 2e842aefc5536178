// Internal interfaces between the GEMM router (gemm.cu) and its kernels.
#pragma once

#include "common.cuh"

namespace b200 {

int32_t launch_gemm_simt(const b200_gemm_args& g, cudaStream_t stream);

// Why the TMA/tcgen05 kernel cannot take these arguments, or nullptr when it can.
const char* gemm_tcgen05_ineligible(const b200_gemm_args& g);
int32_t launch_gemm_tcgen05(const b200_gemm_args& g, cudaStream_t stream);

// Small-M (decode shapes) split-K route: tensor-core partials into a scratch buffer + reduce.
const char* gemm_skinny_ineligible(const b200_gemm_args& g);
int gemm_skinny_splits(const b200_gemm_args& g);
size_t gemm_skinny_scratch_bytes(const b200_gemm_args& g);
int32_t launch_gemm_skinny(const b200_gemm_args& g, void* scratch, size_t scratch_bytes, cudaStream_t stream);

}  // namespace b200

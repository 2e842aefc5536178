// Internal interfaces between the GEMM router (gemm.cu) and its kernels.
#pragma once

#include "common.cuh"

namespace b200 {

// Argument checks every GEMM entry point runs before anything is launched (null pointers, enums,
// extents, element alignment of every pointer, row pitches). B200_OK or a status with the error text set.
int32_t validate_gemm_args(const b200_gemm_args* args);

int32_t launch_gemm_simt(const b200_gemm_args& g, cudaStream_t stream);

// Why the TMA/tcgen05 kernel cannot take these arguments, or nullptr when it can.
const char* gemm_tcgen05_ineligible(const b200_gemm_args& g);

// A multi-pass K loop for the tensor-core kernel: `parts` passes over g.k, pass i reading A at k
// offset a_off[i] and B at k offset b_off[i] inside operands whose stored K extent is k_storage.
struct GemmKParts {
  int32_t parts;
  int64_t k_storage;
  int32_t a_off[3], b_off[3];
};
int32_t launch_gemm_tcgen05(const b200_gemm_args& g, cudaStream_t stream, const GemmKParts* k_parts = nullptr);

// At most 8 rows (fp32 or bf16): CUDA-core partial sums over (column block, K slice) CTAs.
const char* gemm_gemv_ineligible(const b200_gemm_args& g);
int gemm_gemv_slices(const b200_gemm_args& g);
size_t gemm_gemv_scratch_bytes(const b200_gemm_args& g);
int32_t launch_gemm_gemv_partials(const b200_gemm_args& g, float* partial, int slices, cudaStream_t stream);
bool gemm_gemv_one_launch(const b200_gemm_args& g);
int32_t launch_gemm_gemv_one_launch(const b200_gemm_args& g, cudaStream_t stream);

// fp32 operands on the tensor cores: each operand is split into bf16 halves (x = hi + lo), written
// K-major into scratch, and one tensor-core launch accumulates a_hi b_lo + a_lo b_hi + a_hi b_hi.
const char* gemm_split_ineligible(const b200_gemm_args& g);
size_t gemm_split_scratch_bytes(const b200_gemm_args& g);
int32_t launch_gemm_split(const b200_gemm_args& g, void* scratch, size_t scratch_bytes, cudaStream_t stream);

// Small-M (decode shapes) split-K route: tensor-core partials into a scratch buffer + reduce.
const char* gemm_skinny_ineligible(const b200_gemm_args& g);
int gemm_skinny_splits(const b200_gemm_args& g);
size_t gemm_skinny_scratch_bytes(const b200_gemm_args& g);
int32_t launch_gemm_skinny(const b200_gemm_args& g, void* scratch, size_t scratch_bytes, cudaStream_t stream);

}  // namespace b200

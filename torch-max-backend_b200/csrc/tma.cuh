// Host-side construction of TMA tensor maps. The driver's encoder is resolved at run time
// through the CUDA runtime, so the library does not link against libcuda.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200 {

// Tiled tensor map over `rank` dims (innermost first). strides_bytes has rank-1 entries (the
// innermost stride is the element size). swizzle_128b selects CU_TENSOR_MAP_SWIZZLE_128B.
// Out-of-range box elements read as zero. Returns B200_OK or a status with b200_last_error set.
int32_t encode_tensor_map(CUtensorMap* out, int32_t dtype, int rank, const void* base,
                          const uint64_t* dims, const uint64_t* strides_bytes,
                          const uint32_t* box, bool swizzle_128b);

}  // namespace b200

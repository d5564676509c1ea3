// Tiled TMA helpers shared by the kernels that stage 2-D/3-D tiles through shared memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace qb {

// Encodes a tiled tensor map (driver entry point resolved once at run time; no link dependency on libcuda).
// dims / box are innermost first; strides_bytes has rank-1 entries.  Element strides are 1.
bool tma_make_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, void const* base, cuuint64_t const* dims,
                  cuuint64_t const* strides_bytes, cuuint32_t const* box, CUtensorMapSwizzle sw);

// swizzle that spreads a tile whose rows are `row_bytes` long over all banks
inline CUtensorMapSwizzle tma_row_swizzle(int row_bytes) {
  return row_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                            : row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
}

}  // namespace qb

// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled, reached
// through the runtime's driver entry point so that the library does not link
// against libcuda).
#pragma once

#include <cuda.h>

#include <cstdint>

namespace tvb {

// A 2-D tiled map over a row-major matrix: `inner` contiguous elements per row,
// `outer` rows of `row_stride_bytes` (a multiple of 16), boxes of
// box_inner x box_outer elements, out-of-range elements read as zero.
// elem: CU_TENSOR_MAP_DATA_TYPE_*; swizzle: CU_TENSOR_MAP_SWIZZLE_*.
// Returns 0, or -1 with the thread's last error set.
int make_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType elem, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle);

}  // namespace tvb

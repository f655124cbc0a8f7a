// Host-side construction of TMA tensor maps without linking libcuda: the driver's encoder is looked up
// through the runtime (cudaGetDriverEntryPoint).  Encoding is pure host arithmetic (no device work, no
// allocation), so it is safe inside stream capture.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace b2 {

// 2-D row-major tensor [rows, cols] of `elem_bytes`-byte elements with box [box_rows, box_cols].
// The base address and the row pitch (cols * elem_bytes) must be multiples of 16 bytes.
bool make_tensor_map_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* ptr, uint64_t rows,
                        uint64_t cols, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz);

}  // namespace b2

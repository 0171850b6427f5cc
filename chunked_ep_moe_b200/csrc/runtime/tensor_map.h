// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver
// entry point, so the extension does not link against libcuda).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace cem {

// Row-major bf16 matrix [rows, cols]; box = [box_rows, 64 columns] with the 128-byte swizzle, so a
// box row is exactly one swizzle span. Out-of-range rows/columns read as zero.
// Throws std::runtime_error on failure (bad alignment, driver too old).
CUtensorMap make_bf16_map_2d(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// The same matrix described for MN-major operand loads: dimensions (64 columns, rows, cols / 64) with strides (row
// pitch, 128 bytes), box = (64, box_rows, chunks). One copy then brings `chunks` adjacent 64-column chunks of
// `box_rows` rows, each chunk as its own swizzled [box_rows][128 B] block. `cols` must be a multiple of 64.
CUtensorMap make_bf16_map_chunked(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t chunks);

}  // namespace cem

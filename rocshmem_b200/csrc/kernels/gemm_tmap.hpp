// Host helper shared by the GEMM translation units: encodes a 2-D tiled tensor map (TMA descriptor)
// for a row-major [rows, cols] matrix with 128-byte swizzle and a box of 128 bytes x box_rows.
#pragma once

#include <cuda.h>

#include <cstdint>

namespace rocshmem {
namespace kernels {

// elem_bytes: 2 (bf16) or 1 (fp8 / raw bytes). The row pitch (cols * elem_bytes) must be a multiple
// of 16 bytes and `base` 16-byte aligned. Returns false when the driver entry point is missing or
// refuses the arguments.
bool encode_tmap_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols_elems, int elem_bytes,
                    uint32_t box_rows);

}  // namespace kernels
}  // namespace rocshmem

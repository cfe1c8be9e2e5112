// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is fetched through the
// runtime (cudaGetDriverEntryPoint), so the library links against cudart only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace msk {

// Returns 0 on success, a negative MskStatus otherwise.
// dims/strides are innermost first; strides_bytes[i] is the byte stride of dim i+1 (rank-1 entries).
int make_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

// Row-major 2-D matrix [rows, cols] of 2-byte elements, box [box_rows x 64 elements] (128 B), 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                      uint32_t box_rows);

// The same matrix as a 3-D tensor (64 columns, rows, column groups of 64) with a box of `box_groups` column
// groups: one copy brings a [box_rows x 64 * box_groups] K-major tile as swizzled [box_rows x 64] parts, 64 *
// box_rows * 2 bytes apart (what a UMMA descriptor with the 128-byte swizzle wants).  Coordinates: (0, row, column / 64).
int make_tmap_bf16_kgroups(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                           uint32_t box_rows, uint32_t box_groups);

}  // namespace msk

// Host helpers shared by the kernel launchers: TMA descriptor encoding through the driver entry
// point (no link-time dependency on libcuda) and cached device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kb {

int device_sm_count();

// Generic bf16/fp32 tiled tensor map.  dims/strides are innermost first; strides_bytes has
// rank-1 entries (the innermost stride is the element size).  swizzle: 0 none, 1 32B, 2 64B, 3 128B.
int make_tmap(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// 2-D bf16 matrix with `inner` contiguous elements per row, `outer` rows, row stride `ld`
// elements; 128-byte swizzle (box_inner must be 64).
int make_tmap_2d_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

}  // namespace kb

// Host-side creation of TMA tensor maps (driver entry point fetched at run time, so the
// library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace fracssm {

// 3D bf16 tensor [d2][d1][d0] (d0 innermost, dense), box {b0, b1, 1}, 128-byte swizzle
// (b0 * 2 bytes must be 128), zero fill outside the tensor.  Returns 0 on success.
int make_tmap_bf16_3d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint32_t b0, uint32_t b1);

}  // namespace fracssm

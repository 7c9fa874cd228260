// Cached 2-D tensor maps (cuTensorMapEncodeTiled resolved at run time, see vx_gemm.cu).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace vx {

// Row-major [rows, cols] tensor of `dt` with a row pitch of `pitch_bytes`; box of box_cols x box_rows
// elements, 128-byte swizzle.  Encoded once per (pointer, extents, pitch, box, type) and cached.
int make_tmap_2d(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int64_t rows, int64_t cols, int64_t pitch_bytes,
                 int box_cols, int box_rows);

}  // namespace vx

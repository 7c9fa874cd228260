// Shared host-side helpers: error reporting, argument checks, format geometry.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/velox_b200.h"

namespace vx {

// Records a message for vx_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// Device status word shared by all kernels (bounded waits report here).
int* device_status_ptr();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Block size along K of one scale; 0 = whole row.
__host__ __device__ inline int fmt_block(int fmt) {
  switch (fmt) {
    case VX_FMT_BLK16_A:
    case VX_FMT_BLK16_B:
    case VX_FMT_NV16: return 16;
    case VX_FMT_MX32: return 32;
    case VX_FMT_FP8_1X128: return 128;
    default: return 0;
  }
}
inline bool fmt_has_sf(int fmt) {
  return fmt == VX_FMT_BLK16_A || fmt == VX_FMT_BLK16_B || fmt == VX_FMT_MX32 || fmt == VX_FMT_NV16;
}
inline bool fmt_valid(int fmt) { return fmt >= VX_FMT_ROWSCALE && fmt <= VX_FMT_FP8_1X128; }

// The GEMM consumes K in stages of 256 FP4 elements; SF atoms per row tile are padded to
// whole stages: 2 atoms per stage for 32-blocks, 4 for 16-blocks.
constexpr int kStageK4 = 256;
inline int64_t sf_kgroups(int fmt, int64_t K) {
  const int per_stage = (fmt == VX_FMT_MX32) ? 2 : 4;
  return ((K + kStageK4 - 1) / kStageK4) * per_stage;
}

// Whether launches of the kernels that call pdl_wait() carry the programmatic-serialization
// attribute (environment VELOX_B200_PDL, default on; "0" gives plain stream order).
bool pdl_enabled();

// Launch of a kernel that executes pdl_wait() before its first dependent access: its blocks may be
// scheduled while the previous kernel of the stream drains, so launch latency and the kernel's own
// set-up (barriers, tensor memory, constant operands) overlap the predecessor's tail.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define VX_CUDA_OK(expr)                                                        \
  do {                                                                          \
    cudaError_t _e = (expr);                                                    \
    if (_e != cudaSuccess)                                                      \
      return ::vx::fail(static_cast<int>(_e), "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

}  // namespace vx

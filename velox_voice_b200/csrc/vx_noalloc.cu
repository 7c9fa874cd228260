// vx_blkscale_gemm_noalloc: the per-16-column block-scaled FP4 GEMM for callers that must not
// allocate device memory.
//
// Who that is: a worker that handed the whole device to its own memory pool at start-up (a
// serving process, a streaming recogniser with a fixed arena), or a latency-critical audio
// thread.  For them cudaMalloc either fails -- nothing is left outside the pool -- or stalls
// every stream of the process while the driver synchronises the device, and a torch
// allocation is not available at all from plain C / C++ hosts.  The regular route
// (vx_sf_from_natural + vx_bsgemm) needs two caller-provided scratch buffers for the scale
// factors in tensor-core layout; this entry point keeps that scratch inside the library
// instead, in a fixed-size array that every GPU loading the library holds until exit.
//
// Limits and sharing rules are documented at the declaration in include/velox_b200.h.

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "vx_common.cuh"

namespace {

// Scale-factor scratch: [0] = A operand, [1] = B operand.  The name below is a HOST-side
// handle of the symbol; the device address comes from cudaGetSymbolAddress (set-up).
static __device__ __align__(256) uint8_t g_noalloc_sf_scratch[2][VX_NOALLOC_SF_MAX_BYTES];

constexpr int kMaxDevices = 64;
uint8_t* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Once per device, with that device current: resolve the device address of the scratch.
int scratch_for_current_device(uint8_t** out) {
  int dev = -1;
  VX_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return vx::fail(-2, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    uint8_t* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_sf_scratch);
    if (e != cudaSuccess || !p)
      return vx::fail(static_cast<int>(e ? e : cudaErrorUnknown), "cudaGetSymbolAddress(scratch): %s",
                      cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int vx_blkscale_gemm_noalloc(const void* pack_a, const void* pack_b, const void* scale_a,
                                        const void* scale_b, float* out, int64_t M, int64_t N,
                                        int64_t K, void* stream) {
  using namespace vx;
  if (M < 0 || N < 0 || K <= 0) return fail(-1, "bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (M == 0 || N == 0) return 0;
  if (!pack_a || !pack_b || !scale_a || !scale_b || !out) return fail(-1, "NULL argument");
  if (K % 32 != 0) return fail(-1, "K=%lld must be a multiple of 32", (long long)K);
  if (M % 2 != 0) return fail(-1, "M=%lld must be even (A-side scales are shared by row pairs)", (long long)M);
  const int64_t need_a = vx_sf_bytes(VX_FMT_BLK16_A, M, K);
  const int64_t need_b = vx_sf_bytes(VX_FMT_BLK16_B, N, K);
  if (need_a > VX_NOALLOC_SF_MAX_BYTES || need_b > VX_NOALLOC_SF_MAX_BYTES)
    return fail(-1,
                "problem too large for the built-in scratch: scale factors need %lld (A) / %lld (B) bytes, "
                "limit %d bytes per operand (roughly rows * K <= 32 Mi); use vx_sf_from_natural + vx_bsgemm "
                "with caller-owned buffers",
                (long long)need_a, (long long)need_b, VX_NOALLOC_SF_MAX_BYTES);
  uint8_t* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  uint8_t* sfa = scratch;
  uint8_t* sfb = scratch + VX_NOALLOC_SF_MAX_BYTES;
  // the relayout clears the bytes it owns (padding rows / K groups must read as zero), so the
  // previous call's contents never leak into this one
  rc = vx_sf_from_natural(VX_FMT_BLK16_A, scale_a, M, K, sfa, stream);
  if (rc) return rc;
  rc = vx_sf_from_natural(VX_FMT_BLK16_B, scale_b, N, K, sfb, stream);
  if (rc) return rc;
  vx_gemm_desc d = {};
  d.struct_size = static_cast<int32_t>(sizeof(vx_gemm_desc));
  d.fmt = VX_FMT_BLK16_A;
  d.M = M; d.N = N; d.K = K;
  d.a_codes = pack_a; d.lda = K / 2;
  d.b_codes = pack_b; d.ldb = K / 2;
  d.a_scales = sfa; d.b_scales = sfb;
  d.epilogue = VX_EPI_NONE;
  d.out_dtype = VX_F32;
  d.out = out; d.ldo = N;
  return vx_bsgemm(&d, stream);
}

// Attention fold pack: q | k | v of the fused QKV projection (+ the projected positional
// embedding, the two positional biases and the 1/sqrt(dk) scale) re-laid out per head for the
// attention kernel, in one pass.
//
//   q2[h, t, 0:dk]    = bf16(bf16(q + pos_u) * scale)     q2[h, t, dk:2dk] = bf16(bf16(q + pos_v) * scale)
//   k2[h, t, 0:dk]    = k                                  k2[h, t, dk:2dk] = p0[t, h*dk : (h+1)*dk]
//   v2[h, t, 0:dk]    = v                                  v2[h, t, dk:2dk] = 0
//
// Stand-alone form (the QKV GEMM can also write this layout from its epilogue, see vx_gemm.cu).
// One thread moves 8 consecutive output elements (16 bytes) of each of the three tensors.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vx_common.cuh"

namespace vx {
namespace {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// q word (two bf16) + bias word -> two bf16 of bf16(bf16(q + b) * scale)
__device__ __forceinline__ uint32_t q_word(uint32_t q, uint32_t b, float scale) {
  const float lo = __fmul_rn(rnd(__fadd_rn(bf16_lo(q), bf16_lo(b))), scale);
  const float hi = __fmul_rn(rnd(__fadd_rn(bf16_hi(q), bf16_hi(b))), scale);
  return pack2(lo, hi);
}

__global__ void __launch_bounds__(256) qkv_pack_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld_qkv,
                                                       const __nv_bfloat16* __restrict__ p0, int64_t ld_p0,
                                                       const __nv_bfloat16* __restrict__ pos_u,
                                                       const __nv_bfloat16* __restrict__ pos_v, float scale,
                                                       int64_t T, int heads, int dk, __nv_bfloat16* __restrict__ q2,
                                                       __nv_bfloat16* __restrict__ k2, __nv_bfloat16* __restrict__ v2) {
  const int per_row = dk >> 3;  // 16-byte pieces of one head's dk values
  const int64_t d = static_cast<int64_t>(heads) * dk;
  const int64_t total = static_cast<int64_t>(heads) * T * per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    // t fastest within a head is NOT wanted: consecutive threads read consecutive columns of a token
    const int piece = static_cast<int>(i % per_row);
    const int hh = static_cast<int>((i / per_row) % heads);
    const int64_t t = i / (static_cast<int64_t>(per_row) * heads);
    const int j = piece * 8;
    const int64_t col = static_cast<int64_t>(hh) * dk + j;
    const __nv_bfloat16* row = qkv + t * ld_qkv;
    const uint4 q = *reinterpret_cast<const uint4*>(row + col);
    const uint4 k = *reinterpret_cast<const uint4*>(row + d + col);
    const uint4 v = *reinterpret_cast<const uint4*>(row + 2 * d + col);
    const uint4 p = *reinterpret_cast<const uint4*>(p0 + t * ld_p0 + col);
    const uint4 bu = *reinterpret_cast<const uint4*>(pos_u + col);
    const uint4 bv = *reinterpret_cast<const uint4*>(pos_v + col);
    const int64_t o = (static_cast<int64_t>(hh) * T + t) * (2 * dk) + j;
    *reinterpret_cast<uint4*>(q2 + o) = make_uint4(q_word(q.x, bu.x, scale), q_word(q.y, bu.y, scale),
                                                   q_word(q.z, bu.z, scale), q_word(q.w, bu.w, scale));
    *reinterpret_cast<uint4*>(q2 + o + dk) = make_uint4(q_word(q.x, bv.x, scale), q_word(q.y, bv.y, scale),
                                                        q_word(q.z, bv.z, scale), q_word(q.w, bv.w, scale));
    *reinterpret_cast<uint4*>(k2 + o) = k;
    *reinterpret_cast<uint4*>(k2 + o + dk) = p;
    *reinterpret_cast<uint4*>(v2 + o) = v;
    *reinterpret_cast<uint4*>(v2 + o + dk) = make_uint4(0, 0, 0, 0);
  }
}

}  // namespace
}  // namespace vx

extern "C" int vx_qkv_pack(const void* qkv, int64_t ld_qkv, const void* p0, int64_t ld_p0, const void* pos_u,
                           const void* pos_v, float scale, int64_t T, int heads, int head_dim, void* q2, void* k2,
                           void* v2, void* stream) {
  using namespace vx;
  if (T < 0 || heads <= 0 || head_dim <= 0) return fail(-1, "bad shape");
  if (T == 0) return 0;
  if (head_dim % 8 != 0) return fail(-1, "head_dim must be a multiple of 8");
  const int64_t d = static_cast<int64_t>(heads) * head_dim;
  if (!qkv || !p0 || !pos_u || !pos_v || !q2 || !k2 || !v2) return fail(-1, "NULL pointer");
  if (ld_qkv < 3 * d || ld_p0 < d || ld_qkv % 8 != 0 || ld_p0 % 8 != 0) return fail(-1, "row strides must cover the row and be multiples of 8 elements");
  const void* ptrs[] = {qkv, p0, pos_u, pos_v, q2, k2, v2};
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return fail(-1, "pointers must be 16-byte aligned");
  const int64_t total = static_cast<int64_t>(heads) * T * (head_dim >> 3);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  qkv_pack_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld_qkv, static_cast<const __nv_bfloat16*>(p0), ld_p0,
      static_cast<const __nv_bfloat16*>(pos_u), static_cast<const __nv_bfloat16*>(pos_v), scale, T, heads, head_dim,
      static_cast<__nv_bfloat16*>(q2), static_cast<__nv_bfloat16*>(k2), static_cast<__nv_bfloat16*>(v2));
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

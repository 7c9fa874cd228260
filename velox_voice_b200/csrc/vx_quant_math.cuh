// Device-side arithmetic of the quantizers (shared by the stand-alone quantize kernels and
// the GEMM epilogue that re-quantizes its output).  See vx_quant.cu for the rounding rules.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vx {

__device__ __forceinline__ float amax8(const float (&v)[8]) {
  float a = fabsf(v[0]);
#pragma unroll
  for (int i = 1; i < 8; ++i) a = fmaxf(a, fabsf(v[i]));
  return a;
}

// UE8M0 of a block maximum: biased exponent byte of 2^ceil(log2(max(amax/6, 1e-6))) and the
// exact reciprocal 2^-e used to normalise.
__device__ __forceinline__ void ue8m0_from_amax(float amax, uint32_t& byte, float& rcp) {
  const float s = fmaxf(__fdiv_rn(amax, 6.0f), 1e-6f);
  const uint32_t b = __float_as_uint(s);
  const uint32_t ef = (b >> 23) + ((b & 0x7fffffu) ? 1u : 0u);
  byte = ef > 255u ? 255u : ef;
  rcp = ef <= 253u ? __uint_as_float((254u - ef) << 23) : 0.0f;
}

// Magnitude code of |q| (count of thresholds strictly exceeded), without compares.
// 2^23 + x rounded toward +inf leaves ceil(x) in the low mantissa bits, so
//   #{k : 0.25 + 0.5 k < a, k = 0..3} = clamp(ceil(2 a - 0.5), 0, 4)
//   #{2.5 < a, 3.5 < a}               = clamp(ceil(a - 2.5), 0, 2)
// Each sum is formed with a single rounding; below 2^23 (negative x) the clamp yields 0.
__device__ __forceinline__ uint32_t e2m1_mag(float a) {
  constexpr uint32_t kMagic = 0x4B000000u;  // bit pattern of 2^23
  uint32_t lo = __float_as_uint(__fmaf_ru(a, 2.0f, 8388607.5f));
  lo = min(max(lo, kMagic), kMagic + 4u);
  uint32_t hi = __float_as_uint(__fadd_ru(a, 8388605.5f));
  hi = min(max(hi, kMagic), kMagic + 2u);
  return (lo - kMagic) + (hi - kMagic);
}
__device__ __forceinline__ uint32_t e2m1_code(float q) {
  return e2m1_mag(fabsf(q)) | (q < 0.0f ? 8u : 0u);
}
__device__ __forceinline__ uint32_t e2m1_pack8(const float (&v)[8], float rcp) {
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) w |= e2m1_code(__fmul_rn(v[j], rcp)) << (4 * j);
  return w;
}

__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(__half(h));
}

// NV16 block: byte = E4M3_RN_sat(amax16 / (6 g)); q = x * rcp_rn(g * dec(byte)).
__device__ __forceinline__ void nv16_block(float a16, float g, uint32_t& byte, float& rcp) {
  const float t = __fdiv_rn(a16, __fmul_rn(6.0f, g));
  byte = __nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3);
  const float d = __fmul_rn(g, e4m3_to_float(byte));
  rcp = d > 0.0f ? __frcp_rn(d) : 0.0f;
}
__device__ __forceinline__ float nv16_global(float amax_t) {
  return amax_t == 0.0f ? 1.0f : __fdiv_rn(amax_t, 2688.0f);
}

// FP8 1x128 block: scale = amax128 / 448 (1 for a zero block); q = x * rcp_rn(scale).
__device__ __forceinline__ void fp8_block(float a128, float& scale, float& rcp) {
  scale = a128 == 0.0f ? 1.0f : __fdiv_rn(a128, 448.0f);
  rcp = __frcp_rn(scale);
}
__device__ __forceinline__ uint2 fp8_pack8(const float (&v)[8], float rcp) {
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = make_float2(__fmul_rn(v[2 * j], rcp), __fmul_rn(v[2 * j + 1], rcp));
    const uint32_t p = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
    w[j >> 1] |= p << (16 * (j & 1));
  }
  return make_uint2(w[0], w[1]);
}


// 2^(byte - 127) as fp32, including byte 0 (2^-127 is subnormal).
__device__ __forceinline__ float ue8m0_to_float(uint32_t byte) {
  return __uint_as_float(byte ? (byte << 23) : 0x00400000u);
}

}  // namespace vx

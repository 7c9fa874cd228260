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
// exact reciprocal 2^-e used to normalise.  Division-free: the correctly rounded quotient
// amax/6 is <= 2^e exactly when amax <= 6 * 2^e = 1.5 * 2^(e+2), so with amax = (1+m) 2^(E-127)
// the byte is E - 2 (+1 when 1+m > 1.5), floored at 108 (= ceil(log2 1e-6) + 127).
__device__ __forceinline__ void ue8m0_from_amax(float amax, uint32_t& byte, float& rcp) {
  const uint32_t b = __float_as_uint(amax);
  const int ef = max(static_cast<int>((b + 0x3FFFFFu) >> 23) - 2, 108);
  byte = ef > 255 ? 255u : static_cast<uint32_t>(ef);
  rcp = ef <= 253 ? __uint_as_float(static_cast<uint32_t>(254 - ef) << 23) : 0.0f;
}

// E2M1 encode of 8 normalised values (q = v * rcp) into one 32-bit word, low nibble first.
//
// The reference rule -- magnitude code = number of thresholds {0.25, 0.75, 1.25, 1.75, 2.5,
// 3.5} strictly exceeded, sign = (q < 0) -- is "round to nearest E2M1 value, ties toward zero,
// capped at 4.0".  The hardware converter (cvt.rn.satfinite.e2m1x2.f32) rounds ties to even
// and reaches 6.0, so it is fed a representative instead of q itself:
//   n   = ceil(4 |q|) clamped to 16      (2^23 + x rounded toward +inf leaves ceil(x) in the
//                                          low mantissa bits; all thresholds are multiples of 1/4)
//   rep = n * 31/128                      strictly inside the interval that rounds, to nearest,
//                                          to the reference's code for every n in 0..16
// and rep carries q's sign bit.  q is formed as (v * rcp) + (+0) with two separate roundings:
// a product that is -0 or underflows to -0 becomes +0, so the sign bit equals (q < 0) exactly
// (a fused multiply-add would keep the sign of the unrounded product).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// packed fp32 pair arithmetic of sm_100 (round to nearest, subnormals kept)
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// Two values at a time: the two fused multiply-adds run as packed fp32 instructions (one issue
// slot per pair).  The product, the "+0" and the clamp stay scalar: they must keep subnormal
// results (a tiny negative value still encodes as -0, i.e. nibble 8, like the reference).
__device__ __forceinline__ void e2m1_rep2(float v0, float v1, float rcp, float& r0, float& r1) {
  const float q0 = __fadd_rn(__fmul_rn(v0, rcp), 0.0f);  // -0 -> +0
  const float q1 = __fadd_rn(__fmul_rn(v1, rcp), 0.0f);
  const uint64_t a2 = pack_f32x2(fminf(fabsf(q0), 4.0f), fminf(fabsf(q1), 4.0f));
  uint64_t n2;  // 2^23 + ceil(4 a)
  asm("fma.rp.f32x2 %0, %1, %2, %3;" : "=l"(n2) : "l"(a2), "l"(pack_f32x2(4.0f, 4.0f)),
      "l"(pack_f32x2(8388608.0f, 8388608.0f)));
  uint64_t p2;  // n * 31/128, exact
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p2) : "l"(n2), "l"(pack_f32x2(0.2421875f, 0.2421875f)),
      "l"(pack_f32x2(-2031616.0f, -2031616.0f)));
  float p0, p1;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(p0), "=f"(p1) : "l"(p2));
  r0 = __uint_as_float(__float_as_uint(p0) | (__float_as_uint(q0) & 0x80000000u));
  r1 = __uint_as_float(__float_as_uint(p1) | (__float_as_uint(q1) & 0x80000000u));
}
__device__ __forceinline__ uint32_t e2m1_pack8(const float (&v)[8], float rcp) {
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; j += 2) e2m1_rep2(v[j], v[j + 1], rcp, r[j], r[j + 1]);
  uint32_t w;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(w)
      : "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]));
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

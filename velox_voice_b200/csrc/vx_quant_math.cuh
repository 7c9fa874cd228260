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
// and reaches 6.0.  It is made to follow the reference by two cheap corrections:
//   * the converter never sees a tie: q is replaced by q' = q when its last mantissa bit is
//     set, else by the next fp32 value toward zero, which has it set (all six thresholds have
//     that bit clear).  q <= t gives q' < t and q > t gives q' > t for every threshold t, so
//     round-to-nearest of q' is the reference's code.  q' = (q * (1 - 2^-24)) | 1: the product
//     rounds to the fp32 neighbour toward zero for every normal q (subnormal q stay put; they
//     encode as zero either way).  For a power-of-two rcp the factor is folded into rcp
//     (rcp * (1 - 2^-24) is exact), saving the second multiplication;
//   * code 7 (6.0, reached for |q| > 5) is turned into code 6 on the packed word.
// q is formed as (v * rcp) + (+0) with two separate roundings: a product that is -0 or
// underflows to -0 becomes +0, so the sign bit equals (q < 0) exactly (a fused multiply-add
// would keep the sign of the unrounded product); tiny negative q keep their sign and encode
// as -0 (nibble 8), like the reference.
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
constexpr float kTowardZero = 0.99999994f;  // 1 - 2^-24

// max(a, b, c) in one instruction (three-input form of sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// max |.| over eight values held as four packed pairs
__device__ __forceinline__ float amax8p(const uint64_t (&p)[4]) {
  float f[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) unpack_f32x2(p[j], f[2 * j], f[2 * j + 1]);
  float a = max3(fabsf(f[0]), fabsf(f[1]), fabsf(f[2]));
  a = max3(a, fabsf(f[3]), fabsf(f[4]));
  a = max3(a, fabsf(f[5]), fabsf(f[6]));
  return fmaxf(a, fabsf(f[7]));
}

// Eight already normalised-and-nudged values -> one word of E2M1 codes (low nibble first), with
// the converter's code 7 (6.0) turned into the reference's cap, code 6 (4.0).
__device__ __forceinline__ uint32_t e2m1_cvt8(const float (&r)[8]) {
  uint32_t w;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(w)
      : "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]));
  // nibbles with magnitude 7 -> 6: clear bit 0 where bits 0..2 are all set
  return w ^ (w & (w >> 1) & (w >> 2) & 0x11111111u);
}

// CANON_ZERO = false skips the "+ (+0)": a product that is (or underflows to) -0 then encodes as
// nibble 8 (-0) where the reference writes 0 -- the same value.  The GEMM epilogue uses it (its
// inputs are -0 only for an exactly -0 pre-activation); the quantizers keep the reference's bytes.
template <bool POW2, bool CANON_ZERO = true>
__device__ __forceinline__ uint32_t e2m1_pack8(const float (&v)[8], float rcp) {
  const float m = POW2 ? __fmul_rn(rcp, kTowardZero) : rcp;
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float q = __fmul_rn(v[j], m);
    if (CANON_ZERO) q = __fadd_rn(q, 0.0f);  // -0 -> +0
    if (!POW2) q = __fmul_rn(q, kTowardZero);
    r[j] = __uint_as_float(__float_as_uint(q) | 1u);
  }
  return e2m1_cvt8(r);
}

// The same encode on four packed pairs with packed fp32 arithmetic (two values per multiply /
// add; every element sees exactly the operations of e2m1_pack8, so the bytes are the same).
// NUDGE = false drops the "| 1": allowed when the values are bf16 numbers and rcp is a power of
// two.  q = v * rcp then has at most 8 significant bits, so its fp32 neighbour toward zero --
// which the folded factor (1 - 2^-24) produces -- lies on the same side of every threshold as q,
// below it when q is a threshold, and is never a threshold itself.
template <bool POW2, bool CANON_ZERO, bool NUDGE>
__device__ __forceinline__ uint32_t e2m1_pack8p(const uint64_t (&v)[4], float rcp) {
  const float m = POW2 ? __fmul_rn(rcp, kTowardZero) : rcp;
  const uint64_t m2 = pack_f32x2(m, m);
  const uint64_t t2 = pack_f32x2(kTowardZero, kTowardZero);
  float r[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint64_t q = mul_f32x2(v[j], m2);
    if (CANON_ZERO) {
      // -0 -> +0 with scalar additions: the packed add of a constant (+0, +0) was seen to leave a
      // product that underflowed to -0 negative (tiny negative value next to a huge one in a block)
      float a, b;
      unpack_f32x2(q, a, b);
      q = pack_f32x2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f));
    }
    if (!POW2) q = mul_f32x2(q, t2);
    float lo, hi;
    unpack_f32x2(q, lo, hi);
    if (NUDGE) {
      lo = __uint_as_float(__float_as_uint(lo) | 1u);
      hi = __uint_as_float(__float_as_uint(hi) | 1u);
    }
    r[2 * j] = lo;
    r[2 * j + 1] = hi;
  }
  return e2m1_cvt8(r);
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
__device__ __forceinline__ uint2 fp8_pack8p(const uint64_t (&v)[4], float rcp) {
  float f[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) unpack_f32x2(v[j], f[2 * j], f[2 * j + 1]);
  return fp8_pack8(f, rcp);
}

// 2^(byte - 127) as fp32, including byte 0 (2^-127 is subnormal).
__device__ __forceinline__ float ue8m0_to_float(uint32_t byte) {
  return __uint_as_float(byte ? (byte << 23) : 0x00400000u);
}

}  // namespace vx

// Block-scaled GEMMs on the 5th-generation tensor cores (tcgen05) with fused epilogues.
//
//   D[M,N] = epilogue( A[M,K] . B[N,K]^T )
//   FP4 operands (E2M1, two per byte):  tcgen05.mma kind::mxf4nvf4.block_scale, scale factors
//       (UE8M0 per 32 / per 16, or E4M3 per 16) read by the MMA from tensor memory;
//   FP8 operands (E4M3, fp32 scale per 1x128): tcgen05.mma kind::f8f6f4, one accumulation
//       group per 128-wide K block, each into its own 128-column accumulator (four in flight),
//       promoted into fp32 registers with sa[m,kb] * sb[n,kb].
//
// One persistent CTA per SM, 18 warps:
//   warp 0      TMA producer: A / B tiles (128 rows x 128 bytes, 128-byte swizzle) and the
//               scale-factor atoms of the stage into a shared-memory ring (B, or only B's
//               scale factors, stay resident when they fit);
//   warp 1      owns tensor memory; runs warp-uniformly, one elected lane copies scale
//               factors shared -> tensor memory (tcgen05.cp) and issues the MMAs;
//               tcgen05.commit releases ring slots and publishes finished accumulators;
//   warps 2..17 epilogue: each warp reads 32-lane x 32-column blocks of the fp32 accumulator
//               (tcgen05.ld, one row per thread), applies scales / bias / Swish / GLU /
//               residual / per-row argmax, then either a swizzled shared-memory staging
//               buffer + TMA store (clipped at the tensor edge by hardware) or direct vector
//               stores; optional re-quantization of the result to FP4.  Sixteen warps (four
//               per scheduler) hide the TMEM-load, shared-memory and MUFU latencies of each other.
// FP4: a 128 x 256 tile with one accumulator, drained into registers right after the commit,
// or a 128 x 128 tile with two accumulators (epilogue of tile i under the MMAs of tile i + 1).
// FP8: rounds of four K blocks into four accumulators, published per round and handed back in
// pairs, so the MMAs of the next round run while the epilogue promotes.
//
// Every mbarrier wait is bounded (vx_ptx.cuh); an expired wait sets the device status word
// and the CTA drains and exits instead of hanging.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "vx_common.cuh"
#include "vx_ptx.cuh"
#include "vx_quant_math.cuh"
#include "vx_tmap.cuh"

namespace vx {
namespace {

constexpr int BM = 128;            // rows of A per tile = TMEM lanes
constexpr int STAGE_ROW_BYTES = 128;  // K bytes per stage: 256 FP4 or 128 FP8 elements
constexpr int TILE_BYTES = BM * STAGE_ROW_BYTES;  // 16 KB
constexpr int MAX_STAGES = 8;          // ring slots (the arena size decides how many are used)
constexpr int ARENA_BYTES = 156 * 1024;
constexpr int RESIDENT_MAX_KSTAGES = 4;                  // B kept in shared memory up to 4 K stages
constexpr int NUM_THREADS = 576;       // 2 + 16 warps (2 + 28 for the FFN up-projection, see epi_warps)
// Registers are granted to a CTA in units of four warps: 18 warps count as 20, so the budget
// is 65536 / 640 = 102 -> 96 registers per thread (112 does not launch).


constexpr int EPI_WARP0 = 2;
constexpr int STAGING_BYTES = 32 * 128;  // 32 rows x up to 128 bytes per epilogue warp
constexpr int FP8_MAX_KB = 16;           // K <= 2048 for the FP8 path
constexpr int FP8_ACCS = 4;              // FP8 accumulators in tensor memory (128 columns each)
constexpr int FP8_SB_BYTES_PER_KB = 16 * 32 * 4;  // epilogue tables of B scales: 16 warps x 32 columns per K block

// tensor-memory columns
constexpr int TM_ACC0 = 0, TM_SFA = 256, TM_SFB = 320, TM_COLS = 512;  // SFA: 2 x 32, SFB: up to 128 columns

// FP4 kinds come in two tile shapes: 128 x 256 with one accumulator (fewest MMA instructions
// and least operand traffic per output) and 128 x 128 with two accumulators (the epilogue of
// tile i overlaps the MMAs of tile i + 1; best when K is short and B stays in shared memory).
enum Kind { KIND_FP4_VEC2 = 0, KIND_FP4_VEC4 = 1, KIND_FP8 = 2, KIND_FP4_VEC2_N128 = 3, KIND_FP4_VEC4_N128 = 4 };
// rows of B per tile = accumulator columns
__host__ __device__ constexpr int kind_bn(int kind) {
  return (kind == KIND_FP4_VEC2 || kind == KIND_FP4_VEC4) ? 256 : 128;
}
__host__ __device__ constexpr bool kind_vec4(int kind) { return kind == KIND_FP4_VEC4 || kind == KIND_FP4_VEC4_N128; }
// MX32 and the per-row-scaled format: every scale a power of two (see swish4p)
__host__ __device__ constexpr bool kind_pow2_scales(int kind) { return kind == KIND_FP4_VEC2 || kind == KIND_FP4_VEC2_N128; }

// Epilogue warps of a kernel instance.  A CTA holds at most 32 warps and the epilogue needs whole
// groups of four (one warp per 32-lane quadrant of tensor memory; the quadrant is also the warp's
// scheduler), so 28 is the ceiling.
//   16  every epilogue but one: warp (quadrant, column group) owns 32 rows x 64 columns of a wide
//       tile (32 x 32 of a narrow one), the same part of every tile;
//   28  Swish + FP4 output on the narrow tile (the FFN up-projection when the caller asks for
//       narrow tiles; the wide tile is the default).  That epilogue is bound by
//       the latency of its own arithmetic -- dependent multiply / ex2 / rcp chains, four warps
//       per scheduler, all in the same phase because one barrier starts them -- so it runs on
//       seven warps per scheduler which take the 32 x 32 chunks of the tile stream ROUND ROBIN
//       (chunk n = 4 * tile + column group goes to warp n mod 7 of the quadrant): the warps of a
//       scheduler then sit in different tiles and different phases, and the two accumulators of
//       the narrow tile keep the MMAs two tiles ahead.
// (The same round-robin hand-out on the WIDE tile was measured too: 178 vs 115 us -- its one
// accumulator is released only when the last of its eight chunks has found a free warp.)
#ifndef VX_RR_WIDE
#define VX_RR_WIDE 0
#endif
__host__ __device__ constexpr bool epi_round_robin(int kind, int epi, int out) {
  return epi == VX_EPI_BIAS_SWISH && out == 2 && (VX_RR_WIDE || kind_bn(kind) == 128);
}
__host__ __device__ constexpr int epi_warps(int kind, int epi, int out) { return epi_round_robin(kind, epi, out) ? 28 : 16; }
__host__ __device__ constexpr int num_threads(int kind, int epi, int out) { return (2 + epi_warps(kind, epi, out)) * 32; }

struct GemmParams {
  int64_t M, N, K;
  int m_tiles, n_tiles, k_stages;
  // scale factors
  const uint8_t* sfa;     // SF atoms of A (block formats)
  const uint8_t* sfb;
  int64_t sf_kg;          // atoms per 128-row tile
  int sf_unit;            // rowscale: unit scale factors in the MMA, row/col scales afterwards
  int sf_e8m0;            // 1 = UE8M0, 0 = E4M3
  const uint8_t* row_scale_u8;  // ROWSCALE: u8 [M]
  const uint8_t* col_scale_u8;  // ROWSCALE: u8 [N]
  const float* a_amax;    // NV16
  const float* b_amax;
  const float* fa;        // FP8: f32 [M, K/128]
  const float* fb;        // FP8: f32 [N, K/128]
  // epilogue
  // shared-memory plan
  int b_resident;         // 1: the CTA keeps its B tile (all K stages) in shared memory
  int sfb_resident;       // 1: B streams, but its scale factors are copied to tensor memory once
                          //    (the CTA owns one n-block, as with b_resident)
  int num_slots;          // ring slots in use (a multiple of `group`)
  int group;              // K stages per full / empty barrier (2 when a whole K = 512 tile is one wait)
  int a_slot_bytes;       // bytes of one A tile + its scale-factor atoms in the arena
  int b_slot_bytes;       // same for one B tile (BN rows)
  int tma_residual;       // 1: residual tiles are prefetched by TMA into the staging buffers
  unsigned long long* trace;  // phase trace buffer (CTA 0, first 32 tiles) or nullptr
  int out_dtype;          // vx_dtype
  int tma_store;
  void* out;
  int64_t ldo;
  const float* bias;
  const void* residual;
  int residual_dtype;
  int64_t ldr;
  float alpha;
  int out_fmt;
  uint8_t* out_sf;
  uint8_t* out_scales;
  int64_t out_sf_kg;
  const float* out_amax;
  // head-major bf16 output (attention fold pack)
  int heads, head_dim, head_col_off;
  const __nv_bfloat16* pos_u;
  const __nv_bfloat16* pos_v;
  float qk_scale;
  float2* lse_part;       // ARGMAX: per (64-column group, row) running (max, sum of exp) or nullptr
  const float* topk_thr;  // ARGMAX + lse_part: per-row threshold of the candidate pass, or nullptr
  unsigned long long* topk_cand;
  int* topk_cnt;
  int topk_cap;
  int* status;
};

// Operand arena, two plans:
//   streaming  slot s = [A tile 16K | SFA 2K | B tile 16K | SFB 2K], ARENA / 36K slots;
//   B resident [B stage 0 .. k-1: tile 16K | SFB 2K] then slots [A tile 16K | SFA 2K].
struct __align__(1024) SmemLayout {
  uint8_t arena[ARENA_BYTES];
  uint8_t staging[16][STAGING_BYTES];
  float bias_s[1024];    // per epilogue warp: bias of its columns (16 warps x 64: second chunk / GLU gate at [32..63]; 32 warps x 32)
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[FP8_ACCS];
  uint64_t tmem_empty[FP8_ACCS];
  uint64_t b_full;
  uint64_t sfb_done;   // sfb_resident: the scale-factor copies out of the borrowed ring slot are complete
  uint64_t res_full[2][16];  // residual block landed, per buffer and epilogue warp
  uint32_t tmem_base;
};

// sigmoid(g) = 1 / (1 + 2^(-g log2 e)) via ex2.approx + rcp.approx (relative error ~1e-6).  Alternatives measured and
// rejected: tanh.approx (one MUFU operation, but its 2^-11 error flips FP4 codes / bf16
// roundings of the re-quantized activations often enough to move CTC argmaxes), and a Newton
// reciprocal on the FMA pipe (one MUFU operation less, six instructions more: 20 % slower).
// ex2 / rcp with the .ftz qualifier are single MUFU instructions (the default forms wrap them
// in range fix-ups for denormal inputs / results).  Results are the same here: a flushed
// 2^x only ever feeds 1 + 2^x, and the reciprocal of a denominator above 2^126 belongs to
// |z| > 87, whose product rounds to zero in bf16 / FP4 either way.
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_ftz(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_f(float z) { return rcp_ftz(1.0f + ex2_ftz(-1.4426950408889634f * z)); }
// Four Swish values z * sigmoid(z), held as two packed pairs za = (z0, z1), zb = (z2, z3), with
// ONE reciprocal (the special-function unit is the busiest pipe of the Swish epilogues) and packed
// fp32x2 arithmetic (their cost is instruction issue):
//   d = 1 + 2^min(-z log2 e, 30)                          mul.f32x2, min, ex2 (MUFU), add.f32x2
//   A = (d0, d1), B = (d2, d3), P = A * B = (d0 d2, d1 d3), r = 1 / (P.lo P.hi)
//   (r P.hi, r P.lo) * B = (1/d0, 1/d1),   (r P.hi, r P.lo) * A = (1/d2, 1/d3)
// -- 1.25 special-function operations per value, seven packed / scalar multiplies per four.
// The exponent is capped at 2^30 so the product of four cannot overflow; a sigmoid below 2^-30
// only occurs for z < -20.8, where z * sigmoid(z) is below 1e-7 in magnitude either way.
// Every Swish of the library goes through this function, so the fp32 / bf16 outputs and the FP4
// re-quantized output of the same GEMM see the same bits.
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
//
// TANH = true: z sigmoid(z) = h + h tanh(h), h = z / 2, with tanh.approx -- one special-function
// operation, one packed multiply and one packed fused multiply-add per pair: 2 instructions per value
// instead of 5 (these epilogues are bound by instruction issue).  Used by the GEMMs whose operands carry
// power-of-two block scales (MX32, per-row): there the activation is re-quantized with power-of-two
// scales too, which absorbs the difference -- the 12-block MX32 stack still reproduces the CPU
// oracle's logits bit for bit (T = 1000) and agrees in every arg-max at M = 24000.  The formats with
// fp32 / E4M3 scales (NV16, FP8) keep the exponential form: their scales move with the last bits of a
// block maximum, and the same swap costs them arg-max agreement over 12 blocks (NV16 1.000 -> 0.991,
// FP8 0.992 -> 0.966 against the oracle in kernel order).
template <bool TANH>
__device__ __forceinline__ void swish4p(uint64_t& za, uint64_t& zb) {
  if constexpr (TANH) {
    const uint64_t half2 = pack_f32x2(0.5f, 0.5f);
    const uint64_t ha = mul_f32x2(za, half2), hb = mul_f32x2(zb, half2);
    float h0, h1, h2, h3;
    unpack_f32x2(ha, h0, h1);
    unpack_f32x2(hb, h2, h3);
    za = fma_f32x2(ha, pack_f32x2(tanh_approx(h0), tanh_approx(h1)), ha);
    zb = fma_f32x2(hb, pack_f32x2(tanh_approx(h2), tanh_approx(h3)), hb);
    return;
  }
  const uint64_t nl2e = pack_f32x2(-1.4426950408889634f, -1.4426950408889634f);
  const uint64_t one2 = pack_f32x2(1.0f, 1.0f);
  float t0, t1, t2, t3;
  unpack_f32x2(mul_f32x2(za, nl2e), t0, t1);
  unpack_f32x2(mul_f32x2(zb, nl2e), t2, t3);
  const uint64_t da = add_f32x2(pack_f32x2(ex2_ftz(fminf(t0, 30.0f)), ex2_ftz(fminf(t1, 30.0f))), one2);
  const uint64_t db = add_f32x2(pack_f32x2(ex2_ftz(fminf(t2, 30.0f)), ex2_ftz(fminf(t3, 30.0f))), one2);
  float p0, p1;
  unpack_f32x2(mul_f32x2(da, db), p0, p1);
  const float rr = rcp_ftz(__fmul_rn(p0, p1));
  const uint64_t rp = mul_f32x2(pack_f32x2(p1, p0), pack_f32x2(rr, rr));
  za = mul_f32x2(za, mul_f32x2(rp, db));
  zb = mul_f32x2(zb, mul_f32x2(rp, da));
}
template <bool TANH>
__device__ __forceinline__ void silu4_f(float& z0, float& z1, float& z2, float& z3) {
  uint64_t za = pack_f32x2(z0, z1), zb = pack_f32x2(z2, z3);
  swish4p<TANH>(za, zb);
  unpack_f32x2(za, z0, z1);
  unpack_f32x2(zb, z2, z3);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Swish + re-quantization of one 32-column chunk of one output row, straight from the accumulator
// registers to E2M1 codes: the epilogue of the FFN up-projection, whose cost is instruction issue
// (one thread per row, 32 values each), so everything that can is done two values per
// instruction with the packed fp32x2 forms:
//   z = acc (* tensor scales) + bias                      add.f32x2 (mul.f32x2)
//   s = z * sigmoid(z)                                    swish4p, four values at a time
//   block maximum with three-input max; the E2M1 encode of e2m1_pack8p.
// NV16 = false: one UE8M0 scale for the 32 values; true: two E4M3 scales (16 values each).
// Returns the scale byte(s), little end first.
// Eight accumulator values r[8 g .. 8 g + 7] -> (* tensor scales) + bias -> Swish, as four packed pairs.
template <bool NV16, bool BIAS>
__device__ __forceinline__ void swish_group8(const uint32_t (&r)[32], int g, const float* bias_s, bool scale_acc,
                                             uint64_t g2, uint64_t (&out)[4]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int q4 = 2 * g + i;
    uint64_t za = pack_f32x2(__uint_as_float(r[4 * q4]), __uint_as_float(r[4 * q4 + 1]));
    uint64_t zb = pack_f32x2(__uint_as_float(r[4 * q4 + 2]), __uint_as_float(r[4 * q4 + 3]));
    if (NV16 && scale_acc) {
      za = mul_f32x2(za, g2);
      zb = mul_f32x2(zb, g2);
    }
    if constexpr (BIAS) {
      const float4 b = *reinterpret_cast<const float4*>(bias_s + 4 * q4);
      za = add_f32x2(za, pack_f32x2(b.x, b.y));
      zb = add_f32x2(zb, pack_f32x2(b.z, b.w));
    }
    swish4p<!NV16>(za, zb);
    out[2 * i] = za;
    out[2 * i + 1] = zb;
  }
}
// Block scale(s) of 32 finished values (16 packed pairs): the scale byte(s), little end first, and
// the reciprocal(s) to normalise with (NV16: rcp0 for values 0..15, rcp1 for 16..31).
template <bool NV16>
__device__ __forceinline__ uint32_t chunk_scales_p(const uint64_t (&sv)[16], float g_out, float& rcp0, float& rcp1) {
  if constexpr (!NV16) {
    float a = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float lo, hi;
      unpack_f32x2(sv[j], lo, hi);
      a = max3(a, fabsf(lo), fabsf(hi));
    }
    uint32_t byte;
    ue8m0_from_amax(a, byte, rcp0);
    rcp1 = rcp0;
    return byte;
  } else {
    uint32_t sb = 0;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float a = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float lo, hi;
        unpack_f32x2(sv[8 * hh + j], lo, hi);
        a = max3(a, fabsf(lo), fabsf(hi));
      }
      uint32_t byte;
      float rcp;
      nv16_block(a, g_out, byte, rcp);
      if (hh == 0) rcp0 = rcp; else rcp1 = rcp;
      sb |= byte << (8 * hh);
    }
    return sb;
  }
}
// Codes of values 8 g .. 8 g + 7 of a finished chunk.
template <bool NV16>
__device__ __forceinline__ uint32_t encode_group8(const uint64_t (&sv)[16], int g, float rcp0, float rcp1) {
  const uint64_t v[4] = {sv[4 * g], sv[4 * g + 1], sv[4 * g + 2], sv[4 * g + 3]};
  if constexpr (NV16) return e2m1_pack8p<false, false, true>(v, g < 2 ? rcp0 : rcp1);
  else return e2m1_pack8p<true, false, true>(v, rcp0);
}

template <bool NV16>
__device__ __forceinline__ uint32_t swish_quant_chunk(const uint32_t (&r)[32], const float* bias_s, bool scale_acc,
                                                      float g_ab, float g_out, uint32_t (&w)[4]) {
  uint64_t sv[16];
  const uint64_t g2 = pack_f32x2(g_ab, g_ab);
  // (the bias test once per chunk, not once per four values: the epilogue is bound by instruction issue)
  if (bias_s) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint64_t o[4];
      swish_group8<NV16, true>(r, g, bias_s, scale_acc, g2, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) sv[4 * g + j] = o[j];
    }
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint64_t o[4];
      swish_group8<NV16, false>(r, g, bias_s, scale_acc, g2, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) sv[4 * g + j] = o[j];
    }
  }
  float rcp0, rcp1;
  const uint32_t sbytes = chunk_scales_p<NV16>(sv, g_out, rcp0, rcp1);
#pragma unroll
  for (int g = 0; g < 4; ++g) w[g] = encode_group8<NV16>(sv, g, rcp0, rcp1);
  return sbytes;
}

// ---------------------------------------------------------------------------------------
// Epilogue of one 32-column chunk held in registers by one thread (one output row).
//   z[i]  accumulator value of logical column `ncol0 + i` (after scales)
//   For GLU the caller passes value and gate chunks and `ncol0` in OUTPUT columns.
template <int EPI, bool RES_TMA, bool TANH = false>
struct ChunkOut {
  // Applies bias / activation / residual in place.  `bias_s` / `gate_s`: 32 bias values of the
  // chunk (and of its GLU gate chunk) in shared memory, or nullptr; `out_col0`: output column.
  static __device__ __forceinline__ void apply(const GemmParams& p, float (&z)[32], float (&gate)[32],
                                               int64_t row, const float* bias_s, const float* gate_s,
                                               int64_t out_col0, bool row_ok, const uint8_t* res_smem,
                                               int lane) {
    if constexpr (EPI != VX_EPI_NONE) {
      if (bias_s) {
        // bias values cached in shared memory by this warp (all lanes read the same words)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 b = *reinterpret_cast<const float4*>(bias_s + i);
          // (explicit roundings: every schedule of a kernel must produce the same bits)
          z[i] = __fadd_rn(z[i], b.x); z[i + 1] = __fadd_rn(z[i + 1], b.y);
          z[i + 2] = __fadd_rn(z[i + 2], b.z); z[i + 3] = __fadd_rn(z[i + 3], b.w);
        }
        if constexpr (EPI == VX_EPI_BIAS_GLU) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 b = *reinterpret_cast<const float4*>(gate_s + i);
            gate[i] = __fadd_rn(gate[i], b.x); gate[i + 1] = __fadd_rn(gate[i + 1], b.y);
            gate[i + 2] = __fadd_rn(gate[i + 2], b.z); gate[i + 3] = __fadd_rn(gate[i + 3], b.w);
          }
        }
      }
    }
    if constexpr (EPI == VX_EPI_BIAS_SWISH) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) silu4_f<TANH>(z[i], z[i + 1], z[i + 2], z[i + 3]);
    } else if constexpr (EPI == VX_EPI_BIAS_GLU) {
#pragma unroll
      // (one reciprocal per value here: the shared-reciprocal form's extra roundings flip enough
      // bf16 roundings of the GLU output to move the 12-block stack away from the CPU oracle)
      for (int i = 0; i < 32; ++i) z[i] *= sigmoid_f(gate[i]);
    } else if constexpr (EPI == VX_EPI_BIAS_RESIDUAL) {
      if (RES_TMA || res_smem) {
        // bf16 block staged by TMA: 64-byte rows, 16-byte slots swizzled by (row >> 1) & 3
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 u = *reinterpret_cast<const uint4*>(res_smem + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            z[8 * v + 2 * j] = fmaf(p.alpha, z[8 * v + 2 * j], __uint_as_float(w[j] << 16));
            z[8 * v + 2 * j + 1] = fmaf(p.alpha, z[8 * v + 2 * j + 1], __uint_as_float(w[j] & 0xffff0000u));
          }
        }
      } else if (row_ok) {
        if (p.residual_dtype == VX_BF16) {
          const __nv_bfloat16* r = static_cast<const __nv_bfloat16*>(p.residual) + row * p.ldr + out_col0;
          if (out_col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(r) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              const uint4 u = *reinterpret_cast<const uint4*>(r + i);  // plain load: may alias `out`
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                z[i + 2 * j] = fmaf(p.alpha, z[i + 2 * j], __uint_as_float(w[j] << 16));
                z[i + 2 * j + 1] = fmaf(p.alpha, z[i + 2 * j + 1], __uint_as_float(w[j] & 0xffff0000u));
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (out_col0 + i < p.N) z[i] = fmaf(p.alpha, z[i], __bfloat162float(r[i]));
          }
        } else {
          const float* r = static_cast<const float*>(p.residual) + row * p.ldr + out_col0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (out_col0 + i < p.N) z[i] = fmaf(p.alpha, z[i], r[i]);
        }
      }
    }
  }
};

// Direct global stores of one chunk: fp32 / bf16 with 16-byte vectors when aligned.
__device__ __forceinline__ void store_chunk_direct(const GemmParams& p, const float (&z)[32],
                                                   int64_t row, int64_t col0, int64_t n_out) {
  if (p.out_dtype == VX_BF16) {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + row * p.ldo + col0;
    if (col0 + 32 <= n_out && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 u;
        u.x = pack_bf16x2(z[i], z[i + 1]);
        u.y = pack_bf16x2(z[i + 2], z[i + 3]);
        u.z = pack_bf16x2(z[i + 4], z[i + 5]);
        u.w = pack_bf16x2(z[i + 6], z[i + 7]);
        *reinterpret_cast<uint4*>(o + i) = u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_out) o[i] = __float2bfloat16_rn(z[i]);
    }
  } else {
    float* o = static_cast<float*>(p.out) + row * p.ldo + col0;
    if (col0 + 32 <= n_out && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(o + i) = make_float4(z[i], z[i + 1], z[i + 2], z[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_out) o[i] = z[i];
    }
  }
}

// Re-quantize one 32-column chunk of an output row to E2M1 (MX32: one UE8M0 scale; NV16: two
// E4M3 scales) -- the same arithmetic as the stand-alone quantizer.  Returns the scale bytes
// (1 or 2, little end first) for the caller to assemble into SF words.
__device__ __forceinline__ uint32_t store_chunk_fp4(const GemmParams& p, const int out_fmt, const float (&z)[32],
                                                    int64_t row, int64_t col0, float g_out,
                                                    bool row_ok) {
  uint32_t w[4];
  uint32_t sbytes;
  if (out_fmt == VX_FMT_MX32) {
    float a = fabsf(z[0]);
#pragma unroll
    for (int i = 1; i < 32; ++i) a = fmaxf(a, fabsf(z[i]));
    uint32_t byte;
    float rcp;
    ue8m0_from_amax(a, byte, rcp);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float v[8] = {z[8 * q], z[8 * q + 1], z[8 * q + 2], z[8 * q + 3],
                          z[8 * q + 4], z[8 * q + 5], z[8 * q + 6], z[8 * q + 7]};
      w[q] = e2m1_pack8<true, false>(v, rcp);
    }
    sbytes = byte;
  } else {
    sbytes = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float a = fabsf(z[16 * h]);
#pragma unroll
      for (int i = 1; i < 16; ++i) a = fmaxf(a, fabsf(z[16 * h + i]));
      uint32_t byte;
      float rcp;
      nv16_block(a, g_out, byte, rcp);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int b = 16 * h + 8 * q;
        const float v[8] = {z[b], z[b + 1], z[b + 2], z[b + 3], z[b + 4], z[b + 5], z[b + 6], z[b + 7]};
        w[2 * h + q] = e2m1_pack8<false, false>(v, rcp);
      }
      sbytes |= byte << (8 * h);
    }
  }
  if (row_ok) {
    uint8_t* o = static_cast<uint8_t*>(p.out) + row * p.ldo + (col0 >> 1);
    *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return sbytes;
}

// Phase trace: SM cycle counter stamps of CTA 0's first 32 tiles, [role][tile][event].
// roles: 0 producer, 1 MMA issuer, 2 epilogue warp 0.  Enabled by vx_set_trace_buffer().
// Compiled in only with -DVX_PHASE_TRACE=1 (the stamps cost the epilogues a predicate and a branch per
// phase; the shipped build leaves them out and vx_set_trace_buffer reports that).
#ifndef VX_PHASE_TRACE
#define VX_PHASE_TRACE 0
#endif
constexpr bool kPhaseTrace = VX_PHASE_TRACE != 0;
constexpr int TRACE_TILES = 32, TRACE_EVENTS = 8;
__device__ __forceinline__ void trace_rec(const GemmParams& p, int role, int tile, int ev) {
  if (p.trace && blockIdx.x == 0 && tile < TRACE_TILES)
    p.trace[(role * TRACE_TILES + tile) * TRACE_EVENTS + ev] = clock64();
}

unsigned long long* g_trace_buffer = nullptr;

// ---------------------------------------------------------------------------------------
// OUT fixes the output route at compile time, which prunes the other routes from the kernel:
//   0  chosen at run time (fp32 / bf16 / FP4, TMA or direct stores, per-row-scaled format);
//   1  bf16 through staged TMA stores, residual (if any) prefetched by TMA;
//   2  FP4 re-quantized in the operands' own block format (MX32 for the 32-block kinds, NV16
//      for the 16-block kinds).
template <int KIND, int EPI, int OUT>
__global__ void __launch_bounds__(num_threads(KIND, EPI, OUT), 1)
bsgemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_res,
              const GemmParams p) {
  pdl_launch_dependents();  // the next kernel of the stream may be scheduled as SMs free up (it waits for this one)
  extern __shared__ uint8_t smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr bool FP8 = (KIND == KIND_FP8);
  constexpr int VEC = kind_vec4(KIND) ? 4 : 2;
  constexpr int APS = kind_vec4(KIND) ? 4 : 2;  // SF atoms per 128 rows per stage
  constexpr bool GLU = (EPI == VX_EPI_BIAS_GLU);
  // FP4 wide: one 128 x 256 accumulator (a single N = 256 MMA does twice the work per issued
  // instruction).  FP4 narrow: two 128 x 128 accumulators.  FP8: 128 x 128, four accumulators,
  // one per 128-wide K block of a round.
  constexpr bool WIDE = kind_bn(KIND) == 256;
  constexpr int BNT = kind_bn(KIND);         // accumulator columns = B rows per tile
  constexpr int NRT = BNT / 128;             // 128-row scale-factor tiles of B per tile
  constexpr int SFB_COLS = 4 * NRT;          // TMEM columns of one K atom of B scale factors
  constexpr int NCH = (WIDE && !GLU) ? 2 : 1;  // 32-column chunks per epilogue warp
  constexpr int GATE_OFF = BNT / 2;          // GLU: gate columns follow the value columns
  // Chunk-sequential reads of the wide tile: the second 32-column chunk is read only after the
  // first is finished.  That halves the live accumulator registers (the kernel is capped at 96
  // per thread; with both chunks live the plain-bias epilogue spills, 75 vs 67 us for the fused
  // QKV projection at T = 90000) and releases tensor memory a little later.  Swish epilogues
  // are bound by their own arithmetic, so the later release costs them nothing; the residual
  // epilogue is the one that loses by it (77 vs 79 us for the FFN down-projection) and keeps both
  // chunks in flight.
  constexpr bool SEQ = (EPI == VX_EPI_BIAS_SWISH || EPI == VX_EPI_BIAS || EPI == VX_EPI_NONE) && NCH == 2;
  // Swish + FP4 output (the FFN up-projection): its own register-lean path, see swish_quant_chunk.
  constexpr bool SWQ = EPI == VX_EPI_BIAS_SWISH && OUT == 2;
  constexpr int EPW = epi_warps(KIND, EPI, OUT);   // epilogue warps
  constexpr int BIAS_PER_WARP = 1024 / EPW;        // floats of sm.bias_s per epilogue warp
  constexpr bool SWQ_RR = epi_round_robin(KIND, EPI, OUT);     // chunks of the tile stream dealt round robin
  constexpr int NCH_SWQ = kind_bn(KIND) / 128;                 // 32-column chunks per warp on the Swish + FP4 path (16 warps)

  const int out_dtype = OUT == 1 ? static_cast<int>(VX_BF16) : (OUT == 2 ? static_cast<int>(VX_FP4) : p.out_dtype);
  const bool tma_store = OUT == 1 ? true : (OUT == 2 ? false : p.tma_store != 0);
  const bool tma_residual = OUT == 1 ? EPI == VX_EPI_BIAS_RESIDUAL : (OUT == 2 ? false : p.tma_residual != 0);
  const bool sf_unit = (OUT == 1 || OUT == 2) ? false : p.sf_unit != 0;
  constexpr bool TOPK = EPI == VX_EPI_BIAS_ARGMAX && OUT == 3;  // OUT 3: the run-time route + the top-k candidate pass
  const int out_fmt = OUT == 2 ? static_cast<int>(kind_vec4(KIND) ? VX_FMT_NV16 : VX_FMT_MX32) : p.out_fmt;
  const bool tr_on = kPhaseTrace && p.trace != nullptr && blockIdx.x == 0;  // phase trace requested (CTA 0 only)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // (The waits below take no abort flag: a flag that the roles poll was built and measured -- the
  // extra exits from every wait loop cost the 96-register epilogues spills, the fused-QKV kernel went
  // from 65 to 83 us -- and it buys little: when the pipeline stalls, every role has been waiting
  // since about the same moment, so their limits run out together, not one after the other.)
  const int nslots = p.num_slots;
  const bool resident = p.b_resident != 0;
  const bool with_sf = !(FP8 || sf_unit);
  const bool sfb_res = p.sfb_resident != 0;   // implies !resident && with_sf
  const bool owns_nb = resident || sfb_res;   // fixed n-block, B scale factors stay in TMEM

  // This CTA's tiles.  B resident: fixed n-block, m-blocks mb0, mb0 + mstep, ...; streaming:
  // tiles t0, t0 + grid, ... with n fastest.  No division inside the loops.
  const int total_tiles = p.m_tiles * p.n_tiles;
  int my_tiles, mb0, nb0;
  if (owns_nb) {
    nb0 = blockIdx.x % p.n_tiles;
    mb0 = blockIdx.x / p.n_tiles;
    const int mstep = gridDim.x / p.n_tiles;
    my_tiles = mb0 < p.m_tiles ? (p.m_tiles - mb0 + mstep - 1) / mstep : 0;
  } else {
    mb0 = blockIdx.x / p.n_tiles;
    nb0 = blockIdx.x - mb0 * p.n_tiles;
    my_tiles = static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  }
  const int step_m = static_cast<int>(gridDim.x) / p.n_tiles;
  const int step_n = owns_nb ? 0 : static_cast<int>(gridDim.x) % p.n_tiles;
  auto next_tile = [&](int& mb, int& nb) {
    mb += step_m;
    nb += step_n;
    if (nb >= p.n_tiles) { nb -= p.n_tiles; ++mb; }
  };

  // arena addressing: [resident B stages] then ring slots ([A | SFA] or [A | SFA | B | SFB])
  const uint32_t a_slot = p.a_slot_bytes, b_slot = p.b_slot_bytes;
  const uint32_t slot_bytes = resident ? a_slot : a_slot + b_slot;
  const uint32_t ring_off = resident ? p.k_stages * b_slot : 0;
  const uint32_t arena_u32 = smem_u32(sm.arena);
  constexpr uint32_t B_TILE_BYTES = BNT * STAGE_ROW_BYTES;

  // ---- set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int a = 0; a < FP8_ACCS; ++a) {
      mbar_init(&sm.tmem_full[a], 1);
      // one arrival per 32 x 32 part (16 per accumulator; a wide accumulator read chunk by chunk has 32),
      // or one per warp where a warp reads its two chunks of the wide tile itself
      mbar_init(&sm.tmem_empty[a], (SWQ_RR && WIDE) ? 32 : 16);
    }
    mbar_init(&sm.b_full, 1);
    mbar_init(&sm.sfb_done, 1);
    for (int w = 0; w < 16; ++w) { mbar_init(&sm.res_full[0][w], 1); mbar_init(&sm.res_full[1][w], 1); }
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    if (tma_store) prefetch_tmap(&tmap_out);
    if (tma_residual) prefetch_tmap(&tmap_res);
  }
  if (FP8 || p.N % BNT != 0) {
    // Scale-factor tiles of B that lie beyond N are never loaded; they must read as zero
    // (their B rows are zero-filled by TMA, and 0 x NaN-scale would poison the accumulator).
    // With N a whole number of column blocks every tile exists and is loaded: nothing to clear
    // (200 KB of shared-memory stores per CTA, about a microsecond of every launch).
    uint4* a4 = reinterpret_cast<uint4*>(sm.arena);
    for (int i = threadIdx.x; i < ARENA_BYTES / 16; i += blockDim.x) a4[i] = make_uint4(0, 0, 0, 0);
  }
  uint8_t* unit_sf = sm.staging[0];  // rowscale only: one atom of 0x7F, copied to TMEM before any tile
  if (!FP8 && sf_unit) {
    uint32_t* u = reinterpret_cast<uint32_t*>(unit_sf);
    for (int i = threadIdx.x; i < 512 / 4; i += blockDim.x) u[i] = 0x7F7F7F7Fu;
  }
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  const int n_sf_tiles = static_cast<int>((p.N + 127) >> 7);  // 128-row SF tiles of B that exist
  // Set-up is done.  Everything below may touch what the previous kernel of the stream produced (A,
  // residual, output buffers), so every thread waits for it here -- except the producer thread, which
  // first starts the loads of its resident weights (constants of the model) and then waits.
  const bool producer_thread = warp == 0 && lane == 0 && my_tiles > 0;
  if (!producer_thread) pdl_wait();

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0 && my_tiles > 0) {
      uint32_t s = 0, ph = 0;
      const uint32_t sf_atom_bytes = with_sf ? static_cast<uint32_t>(APS * 512) : 0u;
      const int64_t sf_stage = APS * 512;
      bool ok = true;
      // B tile (+ its scale factors) of n-block nb, K stage ks -> dst; returns bytes in flight
      auto load_b = [&](uint8_t* dst, int nb, int ks, uint64_t* bar) {
        tma_load_2d(dst, &tmap_b, ks * STAGE_ROW_BYTES, nb * BNT, bar);
        if (with_sf && !sfb_res) {
#pragma unroll
          for (int rt = 0; rt < NRT; ++rt)
            if (nb * NRT + rt < n_sf_tiles)
              bulk_load(dst + B_TILE_BYTES + rt * APS * 512,
                        p.sfb + (static_cast<int64_t>(nb * NRT + rt) * p.sf_kg) * 512 + ks * sf_stage, APS * 512, bar);
        }
      };
      auto b_tx = [&](int nb) -> uint32_t {
        uint32_t t = B_TILE_BYTES;
        if (with_sf && !sfb_res) {
#pragma unroll
          for (int rt = 0; rt < NRT; ++rt)
            if (nb * NRT + rt < n_sf_tiles) t += sf_atom_bytes;
        }
        return t;
      };
      uint8_t* const sfb_stage = sm.arena + (nslots - 1) * slot_bytes + a_slot;
      bool sfb_pending = sfb_res;
      if (resident) {
        mbar_expect_tx(&sm.b_full, p.k_stages * b_tx(nb0));
        for (int ks = 0; ks < p.k_stages; ++ks) load_b(sm.arena + ks * b_slot, nb0, ks, &sm.b_full);
      } else if (sfb_res) {
        // all scale factors of the n-block -> the B region of the last ring slot (zero-filled
        // at set-up), [ks][rt][atom]; the ring takes that slot over once they are in TMEM
        uint32_t tx = 0;
        for (int rt = 0; rt < NRT; ++rt)
          if (nb0 * NRT + rt < n_sf_tiles) tx += p.k_stages * sf_atom_bytes;
        mbar_expect_tx(&sm.b_full, tx);
        for (int ks = 0; ks < p.k_stages; ++ks)
          for (int rt = 0; rt < NRT; ++rt)
            if (nb0 * NRT + rt < n_sf_tiles)
              bulk_load(sfb_stage + (ks * NRT + rt) * APS * 512,
                        p.sfb + (static_cast<int64_t>(nb0 * NRT + rt) * p.sf_kg) * 512 + ks * sf_stage, APS * 512,
                        &sm.b_full);
      }
      pdl_wait();
      int mb = mb0, nb = nb0;
      const int G = p.group, k_groups = p.k_stages / G, ngs = nslots / G;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const uint8_t* sfa_row = p.sfa + (static_cast<int64_t>(mb) * p.sf_kg) * 512;
        const uint32_t slot_tx = TILE_BYTES + sf_atom_bytes + (resident ? 0u : b_tx(nb));
        for (int kg = 0; kg < k_groups; ++kg) {
          if (!mbar_wait(&sm.empty[s], ph ^ 1, p.status, 1)) { ok = false; break; }
          if (sfb_pending && s == static_cast<uint32_t>(nslots - 1)) {
            if (!mbar_wait(&sm.sfb_done, 0, p.status, 7)) { ok = false; break; }
            sfb_pending = false;
          }
          if (tr_on) trace_rec(p, 0, i, kg < 4 ? kg : 3);
          mbar_expect_tx(&sm.full[s], G * slot_tx);
          for (int u = 0; u < G; ++u) {
            const int ks = kg * G + u;
            uint8_t* dst = sm.arena + ring_off + (s * G + u) * slot_bytes;
            tma_load_2d(dst, &tmap_a, ks * STAGE_ROW_BYTES, mb * BM, &sm.full[s]);
            if (with_sf) bulk_load(dst + TILE_BYTES, sfa_row + ks * sf_stage, APS * 512, &sm.full[s]);
            if (!resident) load_b(dst + a_slot, nb, ks, &sm.full[s]);
          }
          if (++s == static_cast<uint32_t>(ngs)) { s = 0; ph ^= 1; }
        }
        next_tile(mb, nb);
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    // Every instruction here is on the critical path of a tile (K = 512 is only eight MMAs).
    // The whole warp runs the loop with warp-uniform control flow and one elected lane issues
    // the tcgen05 instructions: addresses and descriptors are then warp-uniform values (they
    // can live in uniform registers, which is where the tensor-core instructions read them).
    // Descriptors are formed with one add: low word = (shared address >> 4) + 2 j for the
    // j-th 64-element K step.
    if (my_tiles > 0) {
      const bool leader = elect_one();
      auto CP = [&](uint32_t taddr, uint64_t d) { if (leader) tc_cp_32x128b_warpx4(taddr, d); };
      auto COMMIT = [&](uint64_t* bar) { if (leader) tc_commit(bar); };
      auto TRACE = [&](int tile, int ev) { if (tr_on && leader) trace_rec(p, 1, tile, ev); };
      uint32_t s = 0, ph = 0;
      uint32_t group = 0;  // accumulation groups issued (FP4: one per tile; FP8: one per stage)
      bool ok = true;
      const uint32_t idesc_base =
          FP8 ? make_idesc_f8(BM, BNT) : make_idesc_mxf4(BM, BNT, p.sf_e8m0 != 0);
      // high words of the two descriptor kinds (see make_desc_k128 / make_desc_sf)
      const uint32_t k128_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t sf_hi = (128u >> 4) | (1u << 14);
      auto desc = [](uint32_t lo, uint32_t hi) -> uint64_t {
        return (static_cast<uint64_t>(hi) << 32) | (lo & 0x3fffu);
      };
      const uint32_t arena_lo = arena_u32 >> 4;
      const uint32_t ring_lo = (arena_u32 + ring_off) >> 4, slot_lo = slot_bytes >> 4;
      const uint32_t aslot_lo = a_slot >> 4, bslot_lo = b_slot >> 4;
      const uint32_t a_sf_lo = TILE_BYTES >> 4, b_sf_lo = B_TILE_BYTES >> 4;
      // idesc and scale-factor columns of the four K steps of a stage
      uint32_t idesc_j[4], sfa_col_j[4], sfb_col_j[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t atom, sf_id;
        if (FP8 || sf_unit) { atom = 0; sf_id = 0; }
        else if (VEC == 2) { atom = j >> 1; sf_id = (j & 1) * 2; }
        else { atom = j; sf_id = 0; }
        idesc_j[j] = idesc_with_sf_id(idesc_base, sf_id, sf_id);
        sfa_col_j[j] = atom * 4;
        sfb_col_j[j] = atom * SFB_COLS;
      }
      const uint32_t tm_sfa = tmem_base + TM_SFA, tm_sfb = tmem_base + TM_SFB;
      if (!FP8 && sf_unit) {
        const uint64_t d = make_desc_sf(smem_u32(unit_sf));
        CP(tm_sfa, d);
#pragma unroll
        for (int rt = 0; rt < NRT; ++rt) CP(tm_sfb + rt * 4, d);
      }
      // B scale factors of one stage: shared (lo = B slot >> 4) -> TMEM columns at `col0`
      auto cp_sfb = [&](uint32_t b_lo, uint32_t col0) {
#pragma unroll
        for (int a = 0; a < APS; ++a)
#pragma unroll
          for (int rt = 0; rt < NRT; ++rt)
            CP(col0 + a * SFB_COLS + rt * 4, desc(b_lo + b_sf_lo + (rt * APS + a) * 32, sf_hi));
      };
      if (resident) {
        if (!mbar_wait(&sm.b_full, 0, p.status, 5)) ok = false;
        tc_fence_after();
        if (ok && with_sf)  // B's scale factors stay in tensor memory for the whole kernel
          for (int ks = 0; ks < p.k_stages; ++ks) cp_sfb(arena_lo + ks * bslot_lo, tm_sfb + ks * APS * SFB_COLS);
      } else if (sfb_res) {
        if (!mbar_wait(&sm.b_full, 0, p.status, 5)) ok = false;
        tc_fence_after();
        if (ok) {
          const uint32_t st_lo = (arena_u32 + (nslots - 1) * slot_bytes + a_slot) >> 4;
          for (int ks = 0; ks < p.k_stages; ++ks)
#pragma unroll
            for (int a = 0; a < APS; ++a)
#pragma unroll
              for (int rt = 0; rt < NRT; ++rt)
                CP(tm_sfb + (ks * APS + a) * SFB_COLS + rt * 4,
                                     desc(st_lo + ((ks * NRT + rt) * APS + a) * 32, sf_hi));
          COMMIT(&sm.sfb_done);
        }
      }
      if constexpr (FP8) {
        // Rounds of up to four 128-wide K blocks, block u of a round into accumulator u.  The
        // accumulators are handed back in pairs (0,1) and (2,3) and published once per round,
        // so this thread -- which shares its scheduler with four busy epilogue warps -- waits
        // and commits a few times per tile instead of twice per K block.
        const int G = p.group, ngs = nslots / G;
        uint32_t use0 = 0, use1 = 0;  // rounds that used accumulator pair 0 / 1
        int in_group = 0;
        for (int i = 0; i < my_tiles && ok; ++i) {
          for (int kb0 = 0; kb0 < p.k_stages && ok; kb0 += FP8_ACCS) {
            const int nkb = p.k_stages - kb0 < FP8_ACCS ? p.k_stages - kb0 : FP8_ACCS;
            for (int u = 0; u < nkb; ++u) {
              if ((u & 1) == 0) {
                const int pr = u >> 1;
                const uint32_t use = pr ? use1 : use0;
                if (!mbar_wait_spin(&sm.tmem_empty[pr], (use & 1) ^ 1, p.status, 2)) { ok = false; break; }
                if (pr) ++use1; else ++use0;
                tc_fence_after();  // orders the epilogue's tcgen05.ld of these buffers before the MMAs
              }
              if (in_group == 0) {
                if (!mbar_wait_spin(&sm.full[s], ph, p.status, 3)) { ok = false; break; }
                tc_fence_after();
              }
              if (kb0 == 0) TRACE(i, 2 * u);
              const uint32_t a_lo = ring_lo + (s * G + in_group) * slot_lo;
              const uint32_t b_lo = resident ? arena_lo + (kb0 + u) * bslot_lo : a_lo + aslot_lo;
              const uint32_t d_tmem = tmem_base + TM_ACC0 + u * 128;
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (leader) mma_f8(d_tmem, desc(a_lo + 2 * j, k128_hi), desc(b_lo + 2 * j, k128_hi), idesc_base, j != 0);
              if (++in_group == G) {
                COMMIT(&sm.empty[s]);  // ring slots reusable once these MMAs have read them
                in_group = 0;
                if (++s == static_cast<uint32_t>(ngs)) { s = 0; ph ^= 1; }
              }
              if (kb0 == 0) TRACE(i, 2 * u + 1);
            }
            if (ok) COMMIT(&sm.tmem_full[0]);
          }
        }
      } else {
        const int G = p.group, k_groups = p.k_stages / G, ngs = nslots / G;
        uint32_t sfsel = 0;  // which half of the scale-factor columns this group uses
        for (int i = 0; i < my_tiles && ok; ++i) {
          for (int kg = 0; kg < k_groups; ++kg) {
            const uint32_t acc = WIDE ? 0u : (group & 1);
            if (kg == 0) {
              const uint32_t use = WIDE ? group : (group >> 1);
              if (!mbar_wait_spin(&sm.tmem_empty[acc], (use & 1) ^ 1, p.status, 2)) { ok = false; break; }
              tc_fence_after();  // orders the epilogue's tcgen05.ld of this buffer before the MMAs
              TRACE(i, 0);
            }
            if (!mbar_wait_spin(&sm.full[s], ph, p.status, 3)) { ok = false; break; }
            TRACE(i, kg < 2 ? 1 + kg : 2);
            const uint32_t d_tmem = tmem_base + TM_ACC0 + acc * 128;
            const uint32_t a_lo0 = ring_lo + s * G * slot_lo;
            // (Issuing the next tile's scale-factor copies ahead of this wait was tried: the
            // tcgen05.commit that publishes the accumulator then fires ~1400 cycles later.)
            const uint32_t sfa_buf = tm_sfa + sfsel * 32;
            const uint32_t sfb_buf = tm_sfb + (owns_nb ? 0u : sfsel * 64);
            {
              if (with_sf) {
                for (int u = 0; u < G; ++u) {
                  const uint32_t a_lo = a_lo0 + u * slot_lo;
  #pragma unroll
                  for (int a = 0; a < APS; ++a)
                    CP(sfa_buf + (u * APS + a) * 4, desc(a_lo + a_sf_lo + a * 32, sf_hi));
                  if (!owns_nb) cp_sfb(a_lo + aslot_lo, sfb_buf + u * APS * SFB_COLS);
                }
              }
              if (kg == 0) TRACE(i, 3);
            }
            for (int u = 0; u < G; ++u) {
              const int ks = kg * G + u;
              const uint32_t a_lo = a_lo0 + u * slot_lo;
              const uint32_t b_lo = resident ? arena_lo + ks * bslot_lo : a_lo + aslot_lo;
              {
                const uint32_t sfa_t = with_sf ? sfa_buf + u * APS * 4 : tm_sfa;
                const uint32_t sfb_t = with_sf ? sfb_buf + (owns_nb ? ks : u) * APS * SFB_COLS : tm_sfb;
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (leader) mma_mxf4<VEC>(d_tmem, desc(a_lo + 2 * j, k128_hi), desc(b_lo + 2 * j, k128_hi), idesc_j[j],
                                sfa_t + sfa_col_j[j], sfb_t + sfb_col_j[j], (ks | j) != 0);
                }
              }
            }
            if (kg == 0) TRACE(i, 4);
            COMMIT(&sm.empty[s]);  // ring slots reusable once these MMAs have read them
            if (kg == 0) TRACE(i, 5);
            if (kg == k_groups - 1) {
              COMMIT(&sm.tmem_full[acc]);
              ++group;
              TRACE(i, 6);
            }
            sfsel ^= 1;
            if (++s == static_cast<uint32_t>(ngs)) { s = 0; ph ^= 1; }
          }
        }
      }
    }
  } else {
    // =========================== epilogue ===========================
    // 16 warps; warp (q, cc) owns TMEM lanes [32 q, 32 q + 32) (the hardware ties a warp to
    // the lane quadrant warp_id % 4).  Columns: FP8 (128 wide) chunk cc; FP4 (256 wide) the two
    // chunks [64 cc, 64 cc + 64); GLU pairs value chunk cc with its gate chunk.
    const int q = warp & 3;
    const int ew = warp - EPI_WARP0;
    const int cc = ew >> 2;
    const int64_t n_out = GLU ? p.N / 2 : p.N;    // logical output columns
    constexpr int OUT_TILE_COLS = GLU ? BNT / 2 : BNT;
    const bool has_work = !(GLU && !WIDE) || cc < 2;  // 128-wide GLU: chunks 2, 3 are the gates of 0, 1
    const bool tr = tr_on && ew == 0 && lane == 0;
    uint32_t group = 0;
    bool ok = true;
    float g_ab = 1.0f, g_out = 1.0f;
    if (p.a_amax && p.b_amax) g_ab = nv16_global(__ldg(p.a_amax)) * nv16_global(__ldg(p.b_amax));
    if (p.out_amax) g_out = nv16_global(__ldg(p.out_amax));
    const int kb_count = FP8 ? p.k_stages : 0;
    uint8_t* const stage0 = sm.staging[ew & 15];
    // TMA residual: the two halves of the staging buffer alternate per 32-column chunk.  The
    // residual block of chunk c lands in half c & 1, the result is formed in place and stored
    // from there, while the block of chunk c + 1 is already in flight into the other half.
    uint32_t res_chunk = 0;  // chunks consumed so far
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const bool dbuf = out_dtype == VX_BF16 && !tma_residual;  // bf16 boxes alternate the two halves
    uint32_t store_count = 0;
    int bias_nb = -1;
    uint32_t best_key = 0;  // ARGMAX: best (value, column) of this thread's row in the current tile
    float lse_m = -INFINITY, lse_s = 0.0f;  // ARGMAX + log-sum-exp: running max / sum of 2^((z - max) log2 e) of the tile
    float* const bias_w = sm.bias_s + ew * BIAS_PER_WARP;
    const float* const bias_base = p.bias ? bias_w : nullptr;
    // FP8: per-warp tables of B scales at the end of the arena, [chunk][quadrant][kb][32];
    // a GLU warp also owns the table of its gate chunk (chunk cc + 2, whose warps are idle)
    int sb_nb = -1;
    float* const sb_all = reinterpret_cast<float*>(sm.arena + ARENA_BYTES - kb_count * FP8_SB_BYTES_PER_KB);
    float* const sb_tab = sb_all + ((cc * 4 + q) * kb_count) * 32;
    float* const sb_gate = sb_all + ((((cc + 2) & 3) * 4 + q) * kb_count) * 32;

    // residual block of (mb, tile column c0) -> staging half `c & 1` (TMA, 32 rows x 32 bf16)
    auto res_issue = [&](uint32_t c, int mb_, int64_t out_col) {
      if (lane == 0) {
        mbar_expect_tx(&sm.res_full[c & 1][ew], 32 * 64);
        tma_load_2d(stage0 + (c & 1) * (STAGING_BYTES / 2), &tmap_res, static_cast<int>(out_col), mb_ * BM + q * 32,
                    &sm.res_full[c & 1][ew]);
      }
    };

    int mb = mb0, nb = nb0;
    const int col_base = (WIDE && EPW == 16) ? (GLU ? cc * 32 : cc * 64) : cc * 32;  // first accumulator column of this warp
    bool res_inflight = false;
    if constexpr (EPI == VX_EPI_BIAS_RESIDUAL) {
      if (tma_residual && my_tiles > 0 && has_work) {
        res_issue(0, mb, static_cast<int64_t>(nb) * OUT_TILE_COLS + col_base);
        res_inflight = true;
      }
    }
    if constexpr (SWQ_RR) {
      // FFN up-projection, round robin: this quadrant's chunks n = CPT * tile + column group, this
      // warp takes n = j, j + 7, j + 14, ...  Narrow tile: accumulator t & 1, published for the
      // (t >> 1)-th time; wide tile: the one accumulator, published for the t-th time.  Every chunk
      // is read by exactly one warp, which arrives once.
      constexpr int CPT = BNT / 32;  // 32-column chunks per tile
      const int j = ew >> 2;
      const bool scale_acc = kind_vec4(KIND) && p.a_amax != nullptr;
      int t_cur = 0;
      for (int n = j; n < CPT * my_tiles && ok; n += EPW / 4) {
        const int t = n / CPT, ccn = n % CPT;
        while (t_cur < t) { next_tile(mb, nb); ++t_cur; }
        const uint32_t acc = WIDE ? 0u : (t & 1);
        if (tr) trace_rec(p, 2, t, 0);
        if (lane == 0) ok = mbar_wait_spin(&sm.tmem_full[acc], (WIDE ? t : (t >> 1)) & 1, p.status, 4);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        tc_fence_after();
        if (tr) trace_rec(p, 2, t, 1);
        uint32_t r[32];
        tc_ld_32x32b_x32(lane_addr + TM_ACC0 + acc * 128 + ccn * 32, r);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.tmem_empty[acc]);
        if (tr) trace_rec(p, 2, t, 2);
        const int64_t row = static_cast<int64_t>(mb) * BM + q * 32 + lane;
        const bool row_ok = row < p.M;
        const int64_t out_col0 = static_cast<int64_t>(nb) * BNT + ccn * 32;
        if (out_col0 >= p.N) continue;  // N % 128 == 0: a chunk is whole or (wide tile, last column block) absent
        uint32_t w[4];
        const uint32_t sb = swish_quant_chunk<kind_vec4(KIND)>(r, p.bias ? p.bias + out_col0 : nullptr, scale_acc, g_ab, g_out, w);
        if (row_ok)
          *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + row * p.ldo + (out_col0 >> 1)) = make_uint4(w[0], w[1], w[2], w[3]);
        // rows of the last tile beyond M get zero scale factors (the SF atoms cover whole 128-row tiles)
        const uint32_t sbw = row_ok ? sb : 0u;
        const int64_t sf_row = (row >> 7) * p.out_sf_kg * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
        if constexpr (!kind_vec4(KIND)) {
          p.out_sf[sf_row + (out_col0 >> 7) * 512 + ((out_col0 >> 5) & 3)] = static_cast<uint8_t>(sbw);
          if (p.out_scales && row_ok) p.out_scales[row * (p.N >> 5) + (out_col0 >> 5)] = static_cast<uint8_t>(sbw);
        } else {
          *reinterpret_cast<uint16_t*>(p.out_sf + sf_row + (out_col0 >> 6) * 512 + ((out_col0 >> 5) & 1) * 2) = static_cast<uint16_t>(sbw);
          if (p.out_scales && row_ok)
            *reinterpret_cast<uint16_t*>(p.out_scales + row * (p.N >> 4) + (out_col0 >> 4)) = static_cast<uint16_t>(sbw);
        }
        if (tr) trace_rec(p, 2, t, 4);
      }
    }
    for (int it = 0; it < (SWQ_RR ? 0 : my_tiles) && ok; ++it) {
      const int64_t row = static_cast<int64_t>(mb) * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const bool rows_ok = static_cast<int64_t>(mb) * BM + q * 32 < p.M;
      int mb_next = mb, nb_next = nb;
      next_tile(mb_next, nb_next);

      if (p.bias && nb != bias_nb && EPI != VX_EPI_NONE) {
        // (re)load this warp's bias values: lane i fetches the i-th column of each chunk
        __syncwarp();
        const int64_t c0 = static_cast<int64_t>(nb) * BNT + col_base + lane;
        const int64_t c1 = GLU ? c0 + GATE_OFF : c0 + 32;
        bias_w[lane] = c0 < p.N ? __ldg(p.bias + c0) : 0.0f;
        if (BIAS_PER_WARP >= 64) bias_w[32 + lane] = c1 < p.N ? __ldg(p.bias + c1) : 0.0f;
        __syncwarp();
        bias_nb = nb;
      }
      if constexpr (SWQ) {
        // FFN up-projection: accumulator -> bias + Swish -> E2M1 codes + scale factors, one
        // 32-column chunk at a time (the second chunk of a wide tile is read from tensor memory
        // only after the first is finished, so that one chunk's registers are live at a time;
        // the MMAs of the next tile then run under the arithmetic of the second chunk)
        const uint32_t acc = WIDE ? 0u : (group & 1);
        const uint32_t acc_addr = lane_addr + TM_ACC0 + acc * 128 + col_base;
        if (tr) trace_rec(p, 2, it, 0);
        if (lane == 0) ok = mbar_wait_spin(&sm.tmem_full[acc], (WIDE ? group : (group >> 1)) & 1, p.status, 4);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        tc_fence_after();
        if (tr) trace_rec(p, 2, it, 1);
        ++group;
        const bool scale_acc = kind_vec4(KIND) && p.a_amax != nullptr;
#pragma unroll
        for (int h = 0; h < NCH_SWQ; ++h) {
          uint32_t r[32];
          tc_ld_32x32b_x32(acc_addr + h * 32, r);
          tc_wait_ld();
          if (h == NCH_SWQ - 1) {  // the whole accumulator is out of tensor memory
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.tmem_empty[acc]);
          }
          if (tr && h == 0) trace_rec(p, 2, it, 2);
          const int64_t out_col0 = static_cast<int64_t>(nb) * BNT + col_base + h * 32;
          uint32_t w[4];
          const uint32_t sb = swish_quant_chunk<kind_vec4(KIND)>(r, bias_base ? bias_base + h * 32 : nullptr, scale_acc, g_ab,
                                                                 g_out, w);
          if (out_col0 < p.N) {
            if (row_ok)
              *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + row * p.ldo + (out_col0 >> 1)) =
                  make_uint4(w[0], w[1], w[2], w[3]);
            // rows of the last tile beyond M get zero scale factors (the SF atoms cover whole 128-row tiles)
            const uint32_t sbw = row_ok ? sb : 0u;
            const int64_t sf_row = (row >> 7) * p.out_sf_kg * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
            if constexpr (!kind_vec4(KIND)) {
              p.out_sf[sf_row + (out_col0 >> 7) * 512 + ((out_col0 >> 5) & 3)] = static_cast<uint8_t>(sbw);
              if (p.out_scales && row_ok) p.out_scales[row * (p.N >> 5) + (out_col0 >> 5)] = static_cast<uint8_t>(sbw);
            } else {
              *reinterpret_cast<uint16_t*>(p.out_sf + sf_row + (out_col0 >> 6) * 512 + ((out_col0 >> 5) & 1) * 2) =
                  static_cast<uint16_t>(sbw);
              if (p.out_scales && row_ok)
                *reinterpret_cast<uint16_t*>(p.out_scales + row * (p.N >> 4) + (out_col0 >> 4)) = static_cast<uint16_t>(sbw);
            }
          }
          if (tr && h == 0) trace_rec(p, 2, it, 4);
        }
        mb = mb_next;
        nb = nb_next;
        continue;
      }
      float z[NCH][32], gate[32];
      if constexpr (FP8) {
        // B scales of this warp's columns, transposed into its private table [kb][32]
        // (lane <-> column while loading; every lane reads whole rows of it afterwards)
        if (nb != sb_nb) {
          __syncwarp();
          const int64_t ncol = static_cast<int64_t>(nb) * BNT + col_base + lane;
          const float* src = p.fb + ncol * kb_count;
          for (int kb = 0; kb < kb_count; ++kb) sb_tab[kb * 32 + lane] = ncol < p.N ? __ldg(src + kb) : 0.0f;
          if constexpr (GLU) {
            if (has_work) {
              const int64_t gcol = ncol + GATE_OFF;
              const float* gsrc = p.fb + gcol * kb_count;
              for (int kb = 0; kb < kb_count; ++kb) sb_gate[kb * 32 + lane] = gcol < p.N ? __ldg(gsrc + kb) : 0.0f;
            }
          }
          __syncwarp();
          sb_nb = nb;
        }
        // promote each 128-wide K block: z += tmem * (sa[row, kb] * sb[col, kb])
#pragma unroll
        for (int i = 0; i < 32; ++i) { z[0][i] = 0.0f; gate[i] = 0.0f; }
        const float* sa_row = p.fa + row * kb_count;
        float sa_next = row_ok ? __ldg(sa_row) : 0.0f;
        for (int kb0 = 0; kb0 < kb_count && ok; kb0 += FP8_ACCS) {
          // one round: up to four K blocks, block u in accumulator u, published together
          const int nkb = kb_count - kb0 < FP8_ACCS ? kb_count - kb0 : FP8_ACCS;
          if (lane == 0) ok = mbar_wait_spin(&sm.tmem_full[0], group & 1, p.status, 4);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          ++group;
          tc_fence_after();
          if (tr && kb0 == 0) trace_rec(p, 2, it, 0);
#pragma unroll 1
          for (int u = 0; u < nkb; ++u) {
            const int kb = kb0 + u;
            const float sa = sa_next;
            if (kb + 1 < kb_count && row_ok) sa_next = __ldg(sa_row + kb + 1);
            const uint64_t sa2 = pack_f32x2(sa, sa);
            // acc[i] += r[i] * (sa * table[i]).  The scale products are a packed fp32x2
            // multiply (both operands come as pairs: sb from shared memory, sa duplicated); the
            // accumulation is scalar, because the accumulator values arrive from tensor memory
            // in single registers and pairing them costs more moves than the packed form saves
            // (measured: all-packed 208 us, all-scalar 232 us, this 194 us on the QKV shape).
            auto promote = [&](float (&acc)[32], const uint32_t (&r)[32], const float* table) {
              const uint32_t taddr = smem_u32(table);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                uint64_t b0, b1;
                asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(b0), "=l"(b1) : "r"(taddr + v * 16));
                float s0, s1, s2, s3;
                unpack_f32x2(mul_f32x2(sa2, b0), s0, s1);
                unpack_f32x2(mul_f32x2(sa2, b1), s2, s3);
                acc[4 * v] = fmaf(__uint_as_float(r[4 * v]), s0, acc[4 * v]);
                acc[4 * v + 1] = fmaf(__uint_as_float(r[4 * v + 1]), s1, acc[4 * v + 1]);
                acc[4 * v + 2] = fmaf(__uint_as_float(r[4 * v + 2]), s2, acc[4 * v + 2]);
                acc[4 * v + 3] = fmaf(__uint_as_float(r[4 * v + 3]), s3, acc[4 * v + 3]);
              }
            };
            const uint32_t acc_addr = lane_addr + TM_ACC0 + u * 128 + col_base;
            uint32_t r[32];
            if constexpr (GLU) {
              if (has_work) {  // gate first, so that one register block serves both loads
                tc_ld_32x32b_x32(acc_addr + GATE_OFF, r);
                tc_wait_ld();
                promote(gate, r, sb_gate + kb * 32);
              }
            }
            if (has_work) {
              tc_ld_32x32b_x32(acc_addr, r);
              tc_wait_ld();
            }
            if ((u & 1) || u == nkb - 1) {
              // both accumulators of the pair are in registers: hand the pair back
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sm.tmem_empty[u >> 1]);
            }
            if (has_work) promote(z[0], r, sb_tab + kb * 32);
            if (tr && kb0 == 0) trace_rec(p, 2, it, 1 + u);
          }
        }
        if (!ok) break;
      } else {
        if (tr) trace_rec(p, 2, it, 0);
        // one polling lane per warp (512 polling threads would starve the MMA-issuing thread)
        const uint32_t acc = WIDE ? 0u : (group & 1);
        const uint32_t acc_addr = lane_addr + TM_ACC0 + acc * 128 + col_base;
        if (lane == 0) ok = mbar_wait_spin(&sm.tmem_full[acc], (WIDE ? group : (group >> 1)) & 1, p.status, 4);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        tc_fence_after();
        if (tr) trace_rec(p, 2, it, 1);
        {
          uint32_t r[32];
#pragma unroll
          for (int h = 0; h < (SEQ ? 1 : NCH); ++h) {
            tc_ld_32x32b_x32(acc_addr + h * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) z[h][i] = __uint_as_float(r[i]);
          }
          if constexpr (GLU) {
            tc_ld_32x32b_x32(acc_addr + GATE_OFF, r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) gate[i] = __uint_as_float(r[i]);
          }
        }
        if (tr) trace_rec(p, 2, it, 2);
        if constexpr (!SEQ) {
          // the accumulator is in registers: hand tensor memory back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.tmem_empty[acc]);
        }
        ++group;
      }

      if (has_work) {
#pragma unroll
        for (int h = 0; h < NCH; ++h) {
          if constexpr (SEQ) {
            // second chunk: read it now (its registers were free for the first chunk's
            // arithmetic), then hand tensor memory back
            if (h == 1) {
              uint32_t r[32];
              tc_ld_32x32b_x32(lane_addr + TM_ACC0 + col_base + 32, r);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) z[1][i] = __uint_as_float(r[i]);
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sm.tmem_empty[0]);
            }
          }
          const int64_t acc_col0 = static_cast<int64_t>(nb) * BNT + col_base + h * 32;       // accumulator / bias column
          const int64_t out_col0 = static_cast<int64_t>(nb) * OUT_TILE_COLS + col_base + h * 32;  // output column
          const bool box_ok = rows_ok && out_col0 < n_out;
          if constexpr (!FP8) {
            if (sf_unit) {
              // reference order: raw * row_scale * col_scale
              const float row_scale = row_ok ? ue8m0_to_float(__ldg(p.row_scale_u8 + row)) : 0.0f;
              const int64_t ncol = acc_col0 + lane;
              const float csv = ncol < p.N ? ue8m0_to_float(__ldg(p.col_scale_u8 + ncol)) : 0.0f;
#pragma unroll
              for (int i = 0; i < 32; ++i) z[h][i] = z[h][i] * row_scale * __shfl_sync(0xffffffffu, csv, i);
            } else if (kind_vec4(KIND) && p.a_amax) {
#pragma unroll
              for (int i = 0; i < 32; ++i) z[h][i] = __fmul_rn(z[h][i], g_ab);
              if constexpr (GLU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) gate[i] = __fmul_rn(gate[i], g_ab);
              }
            }
          }
          const uint8_t* res_smem = nullptr;
          uint8_t* const res_half = stage0 + (res_chunk & 1) * (STAGING_BYTES / 2);
          if constexpr (EPI == VX_EPI_BIAS_RESIDUAL) {
            if (res_inflight) {
              // first send for the next block (second chunk of this tile, or the first chunk of
              // the next tile): its half was last read by the store of the previous chunk
              const bool more = h + 1 < NCH || it + 1 < my_tiles;
              if (more) {
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                if (h + 1 < NCH) res_issue(res_chunk + 1, mb, out_col0 + 32);
                else res_issue(res_chunk + 1, mb_next, static_cast<int64_t>(nb_next) * OUT_TILE_COLS + col_base);
              }
              if (!mbar_wait(&sm.res_full[res_chunk & 1][ew], (res_chunk >> 1) & 1, p.status, 6)) { ok = false; break; }
              res_smem = res_half;
            }
          }
          if (tr && h == 0 && !FP8) trace_rec(p, 2, it, 3);
          ChunkOut<EPI, OUT == 1, kind_pow2_scales(KIND)>::apply(p, z[h], gate, row, bias_base ? bias_base + h * 32 : nullptr, bias_base + 32, out_col0,
                               row_ok, res_smem, lane);
          if (tr && h == 0 && !FP8) trace_rec(p, 2, it, 4);

          if constexpr (EPI == VX_EPI_BIAS_QKVPACK) {
            // Attention fold pack: this 32-column chunk lies inside one head of q, k or v.
            //   q: two boxes, bf16(bf16(q + u) * scale) and bf16(bf16(q + v) * scale) side by side;
            //   k: one box (the other half of the head row belongs to the positional projection);
            //   v: one box and a box of zeros.
            const int dk = p.head_dim;
            const int d_model = p.heads * dk;
            const int part = static_cast<int>(out_col0) / d_model;
            const int within = static_cast<int>(out_col0) - part * d_model;
            const int hh = within / dk, j0 = within - hh * dk;
            auto rnd = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };
            auto stage_bf16 = [&](uint8_t* buf, const float (&v)[32]) {
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                uint4 u;
                u.x = pack_bf16x2(v[8 * v4], v[8 * v4 + 1]);
                u.y = pack_bf16x2(v[8 * v4 + 2], v[8 * v4 + 3]);
                u.z = pack_bf16x2(v[8 * v4 + 4], v[8 * v4 + 5]);
                u.w = pack_bf16x2(v[8 * v4 + 6], v[8 * v4 + 7]);
                *reinterpret_cast<uint4*>(buf + lane * 64 + ((v4 ^ ((lane >> 1) & 3)) << 4)) = u;
              }
            };
            // bias vector (32 bf16, the same for every lane) -> fp32
            auto load_bias32 = [&](const __nv_bfloat16* src, float (&b)[32]) {
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(src) + v4);
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  b[8 * v4 + 2 * j] = __uint_as_float(ww[j] << 16);
                  b[8 * v4 + 2 * j + 1] = __uint_as_float(ww[j] & 0xffff0000u);
                }
              }
            };
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
            uint8_t* const buf_a = stage0;
            uint8_t* const buf_b = stage0 + STAGING_BYTES / 2;
            if (part == 0) {
              float b[32], o[32];
              load_bias32(p.pos_u + within, b);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __fmul_rn(rnd(__fadd_rn(rnd(z[h][i]), b[i])), p.qk_scale);
              stage_bf16(buf_a, o);
              load_bias32(p.pos_v + within, b);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __fmul_rn(rnd(__fadd_rn(rnd(z[h][i]), b[i])), p.qk_scale);
              stage_bf16(buf_b, o);
            } else {
              stage_bf16(buf_a, z[h]);
              if (part == 2) {
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) *reinterpret_cast<uint4*>(buf_b + lane * 64 + (v4 << 4)) = make_uint4(0, 0, 0, 0);
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && box_ok) {
              const int zc = part * p.heads + hh;
              tma_store_3d(&tmap_out, j0, mb * BM + q * 32, zc, buf_a);
              if (part != 1) tma_store_3d(&tmap_out, dk + j0, mb * BM + q * 32, zc, buf_b);
              tma_store_commit();
            }
          } else if constexpr (EPI == VX_EPI_BIAS_ARGMAX) {
            // key: order-preserving bits of bf16(z) (high half) | 0xFFFF - tile column (low half).  The chunk's
            // maximum is taken on the bf16-rounded values themselves (three-input max), then the first column
            // holding it is looked up: cheaper than forming a key per value (this epilogue is bound by its
            // integer arithmetic), and equal values -- -0 and +0 included -- resolve to the lowest column.
            const uint32_t cbase = 0xffffu - static_cast<uint32_t>(col_base + h * 32);
            const int valid = p.N - acc_col0 >= 32 ? 32 : static_cast<int>(p.N - acc_col0);
            float zr[32];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint32_t pk = pack_bf16x2(z[h][i], z[h][i + 1]);
              zr[i] = __uint_as_float(pk << 16);
              zr[i + 1] = __uint_as_float(pk & 0xffff0000u);
            }
            if (valid < 32) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i >= valid) zr[i] = -INFINITY;
            }
            float cm = zr[0];
#pragma unroll
            for (int i = 1; i < 32; i += 2) cm = i + 1 < 32 ? max3(cm, zr[i], zr[i + 1]) : fmaxf(cm, zr[i]);
            if (valid > 0) {
              int first = 31;
#pragma unroll
              for (int i = 30; i >= 0; --i)
                if (zr[i] == cm) first = i;
              const uint32_t x = __float_as_uint(__fadd_rn(cm, 0.0f));  // -0 -> +0: one key for both
              const uint32_t u = x ^ (static_cast<uint32_t>(static_cast<int32_t>(x) >> 31) | 0x80000000u);
              best_key = max(best_key, (u & 0xffff0000u) | (cbase - static_cast<uint32_t>(first)));
            }
            if (p.lse_part && valid > 0) {
              // log-sum-exp of the bf16-rounded logits, streaming: the chunk's sum relative to its maximum,
              // merged into the running pair of this 64-column group
              constexpr float L2E = 1.4426950408889634f;
              const float nb2 = -cm * L2E;
              float cs = 0.0f;
#pragma unroll
              for (int i = 0; i < 32; ++i) cs += ex2_ftz(fmaf(zr[i], L2E, nb2));
              const float nm = fmaxf(lse_m, cm);
              lse_s = lse_s * ex2_ftz((lse_m - nm) * L2E) + cs * ex2_ftz((cm - nm) * L2E);
              lse_m = nm;
              if (TOPK && row_ok) {
                // candidate pass of the top-k: append every logit of this chunk that reaches the row's threshold
                // (few chunks of a row hold one; the chunk maximum decides whether to look at all)
                const float thr = __ldg(p.topk_thr + row);
                if (cm >= thr) {
#pragma unroll
                  for (int i = 0; i < 32; ++i) {
                    if (zr[i] >= thr) {
                      const int slot = atomicAdd(p.topk_cnt + row, 1);
                      if (slot < p.topk_cap) {
                        const uint32_t x = __float_as_uint(zr[i]);
                        const uint32_t u = x ^ (static_cast<uint32_t>(static_cast<int32_t>(x) >> 31) | 0x80000000u);
                        p.topk_cand[row * p.topk_cap + slot] =
                            (static_cast<unsigned long long>(u) << 32) | (0xffffffffu - static_cast<uint32_t>(acc_col0 + i));
                      }
                    }
                  }
                }
              }
            }
          } else if (out_dtype == VX_FP4) {
            const uint32_t sb = store_chunk_fp4(p, out_fmt, z[h], row, out_col0, g_out, row_ok && out_col0 < n_out);
            if (out_col0 < n_out) {
              // this chunk's scale byte(s) inside the row's SF word(s); rows of the last tile
              // beyond M get zero scale factors (the SF atoms cover whole 128-row tiles)
              const uint32_t sbw = row_ok ? sb : 0u;
              const int64_t sf_row = (row >> 7) * p.out_sf_kg * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
              if (out_fmt == VX_FMT_MX32) {
                p.out_sf[sf_row + (out_col0 >> 7) * 512 + ((out_col0 >> 5) & 3)] = static_cast<uint8_t>(sbw);
                if (p.out_scales && row_ok) p.out_scales[row * (n_out >> 5) + (out_col0 >> 5)] = static_cast<uint8_t>(sbw);
              } else {
                *reinterpret_cast<uint16_t*>(p.out_sf + sf_row + (out_col0 >> 6) * 512 + ((out_col0 >> 5) & 1) * 2) =
                    static_cast<uint16_t>(sbw);
                if (p.out_scales && row_ok)
                  *reinterpret_cast<uint16_t*>(p.out_scales + row * (n_out >> 4) + (out_col0 >> 4)) =
                      static_cast<uint16_t>(sbw);
              }
            }
          } else if (tma_store) {
            // stage 32 rows x 32 columns (swizzled like the tensor map), then one TMA store
            uint8_t* buf = stage0;
            if (res_smem) {
              buf = res_half;  // in place over the residual block (same box layout); its previous
                               // store was waited for before that block was requested
            } else if (dbuf) {
              if (lane == 0) tma_store_wait_read<1>();  // the box staged two stores ago has left
              buf = stage0 + (store_count & 1) * (STAGING_BYTES / 2);
            } else {
              if (lane == 0) tma_store_wait_read<0>();
            }
            ++store_count;
            __syncwarp();
            if (out_dtype == VX_BF16) {
              // 64-byte rows, 64-byte swizzle: 16-byte slot index ^= (row >> 1) & 3
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 u;
                u.x = pack_bf16x2(z[h][8 * v], z[h][8 * v + 1]);
                u.y = pack_bf16x2(z[h][8 * v + 2], z[h][8 * v + 3]);
                u.z = pack_bf16x2(z[h][8 * v + 4], z[h][8 * v + 5]);
                u.w = pack_bf16x2(z[h][8 * v + 6], z[h][8 * v + 7]);
                *reinterpret_cast<uint4*>(buf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = u;
              }
            } else {
              // 128-byte rows, 128-byte swizzle: slot index ^= row & 7
#pragma unroll
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<float4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) =
                    make_float4(z[h][4 * v], z[h][4 * v + 1], z[h][4 * v + 2], z[h][4 * v + 3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (tr && h == 0 && !FP8) trace_rec(p, 2, it, 5);
            if (lane == 0 && box_ok) {
              if (p.heads > 0) {  // head-major: [head][row][head_col_off + column inside the head]
                const int hh = static_cast<int>(out_col0) / p.head_dim;
                tma_store_3d(&tmap_out, p.head_col_off + static_cast<int>(out_col0) - hh * p.head_dim, mb * BM + q * 32,
                             hh, buf);
              } else {
                tma_store_2d(&tmap_out, static_cast<int>(out_col0), mb * BM + q * 32, buf);
              }
              tma_store_commit();
            }
            if (tr && h == 0) trace_rec(p, 2, it, FP8 ? 7 : 6);
          } else if (row_ok) {
            store_chunk_direct(p, z[h], row, out_col0, n_out);
          }
          if (EPI == VX_EPI_BIAS_RESIDUAL && res_inflight) ++res_chunk;
        }
      }
      if constexpr (EPI == VX_EPI_BIAS_ARGMAX) {
        if (has_work && row_ok && best_key != 0) {
          const uint32_t gcol = static_cast<uint32_t>(nb) * BNT + (0xffffu - (best_key & 0xffffu));
          const unsigned long long key =
              (static_cast<unsigned long long>(best_key & 0xffff0000u) << 32) | (0xffffffffu - gcol);
          atomicMax(static_cast<unsigned long long*>(p.out) + row, key);
        }
        best_key = 0;
        if (p.lse_part) {
          if (has_work && row_ok) p.lse_part[(static_cast<int64_t>(nb) * 4 + cc) * p.M + row] = make_float2(lse_m, lse_s);
          lse_m = -INFINITY;
          lse_s = 0.0f;
        }
      }
      mb = mb_next;
      nb = nb_next;
    }
    if (tma_store && lane == 0) tma_store_wait_all<0>();
  }

  // ---- tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TM_COLS);
  }
}

// keys of the ARGMAX epilogue -> column ids (and the winning bf16 logit as fp32)
__global__ void argmax_ids_kernel(const unsigned long long* __restrict__ keys, int64_t M,
                                  int32_t* __restrict__ ids, float* __restrict__ max_out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= M) return;
  const unsigned long long k = keys[i];
  ids[i] = static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(k));
  if (max_out) {
    const uint32_t u = static_cast<uint32_t>(k >> 32);
    max_out[i] = __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u & 0xffff0000u);
  }
}

// Top-k of the CTC head, step 2 of 3: the k-th largest 64-column-group maximum of every row (the running
// maxima of the log-sum-exp partials).  At least k logits of the row reach it and each of the row's k largest
// does, so it is the threshold of the candidate pass.
__global__ void topk_threshold_kernel(const float2* __restrict__ parts, int nparts, int64_t M, int k, float* __restrict__ thr) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float top[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) top[i] = -INFINITY;
  for (int g = 0; g < nparts; ++g) {
    float v = parts[static_cast<int64_t>(g) * M + row].x;
    // insert into the descending list (registers only: fixed trip counts)
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float hi = fmaxf(top[i], v);
      v = fminf(top[i], v);
      top[i] = hi;
    }
  }
  float t = top[0];
#pragma unroll
  for (int i = 1; i < 16; ++i)
    if (i < k) t = top[i];
  thr[row] = t;
}

// Step 3 of 3: the k largest candidates of every row (equal logits: lowest column first -- the packed entry
// orders exactly that way), as ids and log-probabilities.
__global__ void topk_finish_kernel(const unsigned long long* __restrict__ cand, const int* __restrict__ cnt, int cap,
                                   const float2* __restrict__ parts, int nparts, int64_t M, int k, int32_t* __restrict__ ids,
                                   float* __restrict__ logp, int* __restrict__ overflow) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= M) return;
  constexpr float L2E = 1.4426950408889634f;
  // log-sum-exp exactly as ctc_finish_kernel forms it
  float m = -INFINITY, s = 0.0f;
  for (int g = 0; g < nparts; ++g) {
    const float2 pr = parts[static_cast<int64_t>(g) * M + row];
    if (pr.y > 0.0f) m = fmaxf(m, pr.x);
  }
  for (int g = 0; g < nparts; ++g) {
    const float2 pr = parts[static_cast<int64_t>(g) * M + row];
    if (pr.y > 0.0f) s += pr.y * exp2f((pr.x - m) * L2E);
  }
  const float lse = m + logf(s);
  const int n = cnt[row];
  if (n > cap || n < k) {  // overflowed list (or an inconsistent call): the caller goes back to the logits
    if (n > cap) atomicExch(overflow, 1);
    for (int j = 0; j < k; ++j) { ids[row * k + j] = -1; logp[row * k + j] = -INFINITY; }
    return;
  }
  const unsigned long long* c = cand + row * cap;
  unsigned long long below = ~0ull;  // entries are distinct (distinct columns): take the largest one below the last
  for (int j = 0; j < k; ++j) {
    unsigned long long best = 0;
    for (int i = 0; i < n; ++i) {
      const unsigned long long e = c[i];
      if (e < below && e > best) best = e;
    }
    below = best;
    const uint32_t u = static_cast<uint32_t>(best >> 32);
    const float z = __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u);
    ids[row * k + j] = static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(best));
    logp[row * k + j] = z - lse;
  }
}

// Greedy CTC tail: keys -> ids and winning logits, partial (max, sum) pairs -> log-sum-exp, and
// from both the log-probability of the winner, log_softmax(z)[argmax] = max - lse.
__global__ void ctc_finish_kernel(const unsigned long long* __restrict__ keys, const float2* __restrict__ parts,
                                  int n_parts, int64_t M, int32_t* __restrict__ ids, float* __restrict__ max_out,
                                  float* __restrict__ lse_out, float* __restrict__ logp_out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= M) return;
  const unsigned long long k = keys[i];
  if (ids) ids[i] = static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(k));
  const uint32_t u = static_cast<uint32_t>(k >> 32);
  const float vmax = __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u & 0xffff0000u);
  if (max_out) max_out[i] = vmax;
  if (!parts) return;
  constexpr float L2E = 1.4426950408889634f;
  float m = -INFINITY;
  for (int p = 0; p < n_parts; ++p) {
    const float2 v = parts[static_cast<int64_t>(p) * M + i];
    if (v.y > 0.0f) m = fmaxf(m, v.x);
  }
  float s = 0.0f;
  for (int p = 0; p < n_parts; ++p) {
    const float2 v = parts[static_cast<int64_t>(p) * M + i];
    if (v.y > 0.0f) s += v.y * exp2f((v.x - m) * L2E);
  }
  const float lse = m + logf(s);
  if (lse_out) lse_out[i] = lse;
  if (logp_out) logp_out[i] = vmax - lse;
}

// ---------------------------------------------------------------------------------------
// MMA peak probe: each CTA issues `iters` MMAs on resident (zero) operands, no memory traffic.
template <int KIND, int NT>
__global__ void __launch_bounds__(128, 1) mma_probe_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a = base;                   // 128 rows x 128 B
  uint8_t* b = base + TILE_BYTES;      // NT rows x 128 B
  uint8_t* sf = b + NT * 128;          // one SF atom (unit scales)
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < (TILE_BYTES + NT * 128) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(base)[i] = 0;
  for (int i = threadIdx.x; i < 128; i += blockDim.x) reinterpret_cast<uint32_t*>(sf)[i] = 0x7F7F7F7Fu;
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (threadIdx.x < 32) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t a_addr = smem_u32(a), b_addr = smem_u32(b);
    if (KIND != KIND_FP8) {
      const uint64_t d = make_desc_sf(smem_u32(sf));
      for (int c = 0; c < 8; ++c) tc_cp_32x128b_warpx4(tb + 480 + c * 4, d);
    }
    const uint32_t idesc = KIND == KIND_FP8 ? make_idesc_f8(128, NT) : make_idesc_mxf4(128, NT, true);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t d_tmem = tb;
        if (KIND == KIND_FP8)
          mma_f8(d_tmem, make_desc_k128(a_addr + j * 32), make_desc_k128(b_addr + j * 32), idesc, 1);
        else
          mma_mxf4<2>(d_tmem, make_desc_k128(a_addr + j * 32), make_desc_k128(b_addr + j * 32), idesc,
                      tb + 480, tb + 480, 1);
      }
    }
    tc_commit(&bar);
    mbar_wait(&bar, 0, status, 9);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tb, 512);
  }
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded wait: one thread waits on an mbarrier that nothing ever arrives at,
// with a caller-chosen limit.  The wait runs out, the status word is set, the kernel returns and
// the context stays usable -- the same path a lost arrival takes in the GEMM, in milliseconds
// instead of the production limit.  No tensor memory and no copy is in flight here.
__global__ void wait_selftest_kernel(unsigned long long limit_ns, int site, int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    abort_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait_slow(&bar, 0, status, site, &abort_flag, limit_ns);
  __syncthreads();
  // a second role of the same CTA sees the raised flag and leaves without writing a status of its own
  if (threadIdx.x == 32) mbar_wait_slow(&bar, 0, status, site + 1, &abort_flag, limit_ns);
}

// ---------------------------------------------------------------------------------------
// Host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Encoded tensor maps, cached by everything that goes into the encoding (base pointer, extents,
// pitch, box, element type, swizzle, rank).  A map is a pure function of those values -- it holds
// no reference to the allocation -- so an entry stays valid when the memory is freed and the
// address is handed out again.  The reference re-encodes its maps on every call
// (veloxvoice/kernels/csrc/dgx/dgx_mxfp4_gemm.cu:61-109); a steady-state caller (same buffers every
// step) pays the driver call once here.  Direct-mapped, one mutex: a lookup is a hash, a lock and a
// 48-byte compare.
struct TmapKey {
  const void* ptr;
  int64_t d0, d1, d2, pitch;
  int32_t box0, box1, dt, swizzle;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && pitch == o.pitch && box0 == o.box0 &&
           box1 == o.box1 && dt == o.dt && swizzle == o.swizzle;
  }
};
constexpr int kTmapCacheSlots = 1024;
struct TmapSlot { TmapKey key; CUtensorMap map; bool used; };
TmapSlot g_tmap_cache[kTmapCacheSlots];
std::mutex g_tmap_mutex;
std::atomic<uint64_t> g_tmap_hits{0}, g_tmap_misses{0};

inline uint32_t tmap_hash(const TmapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(k.d0) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(k.d1) * 0x165667B19E3779F9ull;
  h ^= static_cast<uint64_t>(k.d2) * 0x27D4EB2F165667C5ull + static_cast<uint64_t>(k.pitch) * 0x85EBCA77C2B2AE63ull;
  h ^= (static_cast<uint64_t>(k.box0) << 40) ^ (static_cast<uint64_t>(k.box1) << 24) ^ (static_cast<uint64_t>(k.dt) << 8) ^
       static_cast<uint64_t>(k.swizzle);
  h ^= h >> 29;
  h *= 0xBF58476D1CE4E5B9ull;
  h ^= h >> 32;
  return static_cast<uint32_t>(h) & (kTmapCacheSlots - 1);
}
bool tmap_lookup(const TmapKey& k, CUtensorMap* out) {
  TmapSlot& s = g_tmap_cache[tmap_hash(k)];
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  if (s.used && s.key == k) {
    *out = s.map;
    g_tmap_hits.fetch_add(1, std::memory_order_relaxed);
    return true;
  }
  return false;
}
void tmap_insert(const TmapKey& k, const CUtensorMap& m) {
  TmapSlot& s = g_tmap_cache[tmap_hash(k)];
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  s.key = k;
  s.map = m;
  s.used = true;
  g_tmap_misses.fetch_add(1, std::memory_order_relaxed);
}

// 2-D row-major tensor [rows, cols] of `elt`-byte elements, row pitch `pitch_bytes`; box =
// box_cols x box_rows; the inner extent in bytes equals the swizzle span (128 or 64).
int make_tmap(CUtensorMap* m, CUtensorMapDataType dt, int elt, const void* ptr, int64_t rows,
              int64_t cols, int64_t pitch_bytes, int box_cols, int box_rows,
              CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  const TmapKey key{ptr, cols, rows, 0, pitch_bytes, box_cols, box_rows, static_cast<int32_t>(dt),
                    static_cast<int32_t>(swizzle)};
  if (tmap_lookup(key, m)) return 0;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(-2, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  (void)elt;
  const CUresult r = fn(m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-3, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  tmap_insert(key, *m);
  return 0;
}

// 3-D bf16 tensor [z][rows][cols] (cols contiguous, row pitch `cols` elements): boxes of
// 32 columns x 32 rows x 1, 64-byte swizzle -- the head-major output of the attention fold pack.
int make_tmap_heads(CUtensorMap* m, const void* ptr, int64_t zdim, int64_t rows, int64_t cols) {
  const TmapKey key{ptr, cols, rows, zdim, cols * 2, 32, 32, static_cast<int32_t>(CU_TENSOR_MAP_DATA_TYPE_BFLOAT16),
                    static_cast<int32_t>(CU_TENSOR_MAP_SWIZZLE_64B)};
  if (tmap_lookup(key, m)) return 0;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(-2, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(zdim)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols * 2), static_cast<cuuint64_t>(rows * cols * 2)};
  const cuuint32_t box[3] = {32, 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-3, "cuTensorMapEncodeTiled (3-D) failed (%d)", static_cast<int>(r));
  tmap_insert(key, *m);
  return 0;
}

int* cached_status_ptr() {
  static int* cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return device_status_ptr();
  if (!cache[dev]) cache[dev] = device_status_ptr();
  return cache[dev];
}

constexpr size_t kSmemBytes = sizeof(SmemLayout) + 1024;

template <int KIND, int EPI, int OUT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr,
           GemmParams& p, bool allow_resident, cudaStream_t st) {
  int dev = 0, sms = 0;
  VX_CUDA_OK(cudaGetDevice(&dev));
  // The dynamic shared-memory opt-in belongs to the (function, device) pair: once per device
  // and template instance (a process may drive several GPUs).
  static std::atomic<uint64_t> attr_done{0};
  const bool dev_cached = dev >= 0 && dev < 64;
  if (!dev_cached || !(attr_done.load(std::memory_order_acquire) & (1ull << dev))) {
    const cudaError_t e = cudaFuncSetAttribute(bsgemm_kernel<KIND, EPI, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kSmemBytes));
    if (e != cudaSuccess) return fail(static_cast<int>(e), "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (dev_cached) attr_done.fetch_or(1ull << dev, std::memory_order_release);
  }
  static int sm_cache[64] = {};
  if (dev >= 0 && dev < 64 && sm_cache[dev]) sms = sm_cache[dev];
  else {
    VX_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (dev >= 0 && dev < 64) sm_cache[dev] = sms;
  }
  // shared-memory plan: keep B resident when all of its K stages fit beside a useful ring
  constexpr int BNT = kind_bn(KIND);
  constexpr int APS = kind_vec4(KIND) ? 4 : 2;
  const bool with_sf = KIND != KIND_FP8 && !p.sf_unit;
  p.a_slot_bytes = TILE_BYTES + (with_sf ? APS * 512 : 0);
  p.b_slot_bytes = BNT * STAGE_ROW_BYTES + (with_sf ? (BNT / 128) * APS * 512 : 0);
  // keep every slot 1024-byte aligned (128-byte swizzle atoms are 1 KB)
  p.a_slot_bytes = (p.a_slot_bytes + 1023) & ~1023;
  p.b_slot_bytes = (p.b_slot_bytes + 1023) & ~1023;
  const int tiles = p.m_tiles * p.n_tiles;
  int grid;
  // FP8: the end of the arena holds the epilogue's B-scale tables
  const int arena = ARENA_BYTES - (KIND == KIND_FP8 ? p.k_stages * FP8_SB_BYTES_PER_KB : 0);
  const int res_slots = (arena - p.k_stages * p.b_slot_bytes) / p.a_slot_bytes;
  p.b_resident = allow_resident && p.k_stages <= RESIDENT_MAX_KSTAGES && p.n_tiles <= sms && res_slots >= 2;
  p.group = 1;
  p.sfb_resident = 0;
  constexpr int SFB_STAGE_COLS = APS * (BNT / 128) * 4;  // TMEM columns of one stage of B scale factors
  if (!p.b_resident && allow_resident && with_sf && p.n_tiles <= sms && p.k_stages * SFB_STAGE_COLS <= 128 &&
      p.k_stages * (BNT / 128) * APS * 512 <= BNT * STAGE_ROW_BYTES) {
    // B is too large to stay in shared memory, its scale factors are not: one copy into
    // tensor memory per CTA instead of one per tile and stage
    p.sfb_resident = 1;
    p.b_slot_bytes = BNT * STAGE_ROW_BYTES;
  }
  if (p.b_resident) {
    p.num_slots = res_slots > MAX_STAGES ? MAX_STAGES : res_slots;
    // a whole K <= 512 FP4 tile (two stages) behind one barrier pair: the MMA-issuing thread
    // waits and commits once per tile instead of once per stage
    if (KIND != KIND_FP8 && p.k_stages == 2 && p.num_slots >= 4) {
      p.group = 2;
      p.num_slots &= ~1;
    }
    if (KIND == KIND_FP8 && p.k_stages % 2 == 0 && p.num_slots >= 4) {  // one ring barrier per pair of K blocks
      p.group = 2;
      p.num_slots &= ~1;
    }
    int groups = sms / p.n_tiles;
    if (groups > p.m_tiles) groups = p.m_tiles;
    grid = groups * p.n_tiles;
  } else {
    const int slots = arena / (p.a_slot_bytes + p.b_slot_bytes);
    p.num_slots = slots > MAX_STAGES ? MAX_STAGES : slots;
    if (KIND == KIND_FP8 && p.k_stages % 2 == 0 && p.num_slots >= 4) {
      p.group = 2;
      p.num_slots &= ~1;
    }
    grid = tiles < sms ? tiles : sms;
    if (p.sfb_resident) {
      int groups = sms / p.n_tiles;
      if (groups > p.m_tiles) groups = p.m_tiles;
      grid = groups * p.n_tiles;
    }
  }
  VX_CUDA_OK(launch_dependent(bsgemm_kernel<KIND, EPI, OUT>, dim3(grid), dim3(num_threads(KIND, EPI, OUT)), kSmemBytes, st, ta, tb,
                              to, tr, p));
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int KIND, int EPI>
int dispatch_out(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to,
                 const CUtensorMap& tr, GemmParams& p, bool res, cudaStream_t st) {
  constexpr bool fp4_out_ok = KIND != KIND_FP8 && (EPI == VX_EPI_NONE || EPI == VX_EPI_BIAS || EPI == VX_EPI_BIAS_SWISH);
  if constexpr (EPI != VX_EPI_BIAS_ARGMAX) {
    if (out == 1) return launch<KIND, EPI, 1>(ta, tb, to, tr, p, res, st);
    if constexpr (fp4_out_ok) {
      if (out == 2) return launch<KIND, EPI, 2>(ta, tb, to, tr, p, res, st);
    }
  }
  if constexpr (EPI == VX_EPI_BIAS_ARGMAX && KIND != KIND_FP8) {
    // the candidate pass of the top-k is an instance of its own: the plain arg-max kernel keeps its registers
    if (p.topk_thr) return launch<KIND, EPI, 3>(ta, tb, to, tr, p, res, st);
  }
  return launch<KIND, EPI, 0>(ta, tb, to, tr, p, res, st);
}

template <int KIND>
int dispatch_epi(int epi, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to,
                 const CUtensorMap& tr, GemmParams& p, bool res, cudaStream_t st) {
  switch (epi) {
    case VX_EPI_NONE: return dispatch_out<KIND, VX_EPI_NONE>(out, ta, tb, to, tr, p, res, st);
    case VX_EPI_BIAS: return dispatch_out<KIND, VX_EPI_BIAS>(out, ta, tb, to, tr, p, res, st);
    case VX_EPI_BIAS_SWISH: return dispatch_out<KIND, VX_EPI_BIAS_SWISH>(out, ta, tb, to, tr, p, res, st);
    case VX_EPI_BIAS_GLU: return dispatch_out<KIND, VX_EPI_BIAS_GLU>(out, ta, tb, to, tr, p, res, st);
    case VX_EPI_BIAS_RESIDUAL: return dispatch_out<KIND, VX_EPI_BIAS_RESIDUAL>(out, ta, tb, to, tr, p, res, st);
    case VX_EPI_BIAS_ARGMAX: return dispatch_out<KIND, VX_EPI_BIAS_ARGMAX>(out, ta, tb, to, tr, p, res, st);
    case VX_EPI_BIAS_QKVPACK: return launch<KIND, VX_EPI_BIAS_QKVPACK, 1>(ta, tb, to, tr, p, res, st);
    default: return fail(-1, "unknown epilogue %d", epi);
  }
}

}  // namespace

int make_tmap_2d(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int64_t rows, int64_t cols, int64_t pitch_bytes,
                 int box_cols, int box_rows) {
  return make_tmap(m, dt, 0, ptr, rows, cols, pitch_bytes, box_cols, box_rows);
}

}  // namespace vx

extern "C" {

int vx_bsgemm(const vx_gemm_desc* d, void* stream) {
  using namespace vx;
  if (!d) return fail(-1, "desc must not be NULL");
  if (d->struct_size != static_cast<int32_t>(sizeof(vx_gemm_desc)))
    return fail(-1, "vx_gemm_desc.struct_size=%d, expected %d", d->struct_size, (int)sizeof(vx_gemm_desc));
  const int fmt = d->fmt;
  if (!fmt_valid(fmt) || fmt == VX_FMT_BLK16_B) return fail(-1, "unsupported GEMM format %d", fmt);
  const int64_t M = d->M, N = d->N, K = d->K;
  if (M < 0 || N < 0 || K < 0) return fail(-1, "negative shape");
  if (M == 0 || N == 0) return 0;
  if (K == 0) return fail(-1, "K must be positive");
  const bool fp8 = fmt == VX_FMT_FP8_1X128;
  const int64_t row_bytes = fp8 ? K : K / 2;
  if (fp8 ? (K % 128 != 0) : (K % 32 != 0))
    return fail(-1, "K=%lld must be a multiple of %d", (long long)K, fp8 ? 128 : 32);
  if (fp8 && K > FP8_MAX_KB * 128) return fail(-1, "FP8 path supports K <= %d", FP8_MAX_KB * 128);
  if (!d->a_codes || !d->b_codes || !d->out) return fail(-1, "a_codes, b_codes and out must not be NULL");
  if (!aligned16(d->a_codes) || !aligned16(d->b_codes) || d->lda % 16 != 0 || d->ldb % 16 != 0 ||
      d->lda < row_bytes || d->ldb < row_bytes)
    return fail(-1, "operand rows must be 16-byte aligned and at least %lld bytes", (long long)row_bytes);
  if (!d->a_scales || !d->b_scales) return fail(-1, "a_scales and b_scales must not be NULL");
  if (fmt == VX_FMT_NV16 && (!d->a_amax || !d->b_amax)) return fail(-1, "NV16 needs a_amax and b_amax");
  if (fmt_has_sf(fmt) && (!aligned16(d->a_scales) || !aligned16(d->b_scales)))
    return fail(-1, "SF atoms must be 16-byte aligned");
  const int epi = d->epilogue;
  if (epi < VX_EPI_NONE || epi > VX_EPI_BIAS_QKVPACK) return fail(-1, "unknown epilogue %d", epi);
  const bool argmax = epi == VX_EPI_BIAS_ARGMAX;
  const bool qkvpack = epi == VX_EPI_BIAS_QKVPACK;
  const bool out_heads = (d->flags & VX_GEMM_OUT_HEADS) != 0;
  constexpr int32_t kKnownFlags = VX_GEMM_DIRECT_STORE | VX_GEMM_STREAM_B | VX_GEMM_WIDE_TILES | VX_GEMM_NARROW_TILES |
                                  VX_GEMM_OUT_HEADS;
  if (d->flags & ~kKnownFlags) return fail(-1, "unknown bits in flags (0x%x)", d->flags & ~kKnownFlags);
  if (qkvpack && fmt == VX_FMT_ROWSCALE)
    return fail(-1, "BIAS_QKVPACK is not available for the per-row-scaled format (use a block-scaled format or FP8)");
  if (qkvpack || out_heads) {
    if (d->heads <= 0 || d->head_dim <= 0 || d->head_dim % 32 != 0)
      return fail(-1, "head-major output needs heads > 0 and head_dim %% 32 == 0");
    if (d->out_dtype != VX_BF16 || !aligned16(d->out)) return fail(-1, "head-major output is bf16, 16-byte aligned");
    if (d->flags & VX_GEMM_DIRECT_STORE) return fail(-1, "head-major output goes through TMA stores only");
    if (qkvpack) {
      if (N != 3ll * d->heads * d->head_dim) return fail(-1, "BIAS_QKVPACK needs N = 3 * heads * head_dim");
      if (!d->pos_u || !d->pos_v || !aligned16(d->pos_u) || !aligned16(d->pos_v))
        return fail(-1, "BIAS_QKVPACK needs pos_u / pos_v (bf16, 16-byte aligned)");
      if (out_heads) return fail(-1, "VX_GEMM_OUT_HEADS does not combine with BIAS_QKVPACK");
    } else {
      if (epi != VX_EPI_NONE && epi != VX_EPI_BIAS) return fail(-1, "VX_GEMM_OUT_HEADS supports NONE / BIAS");
      if (N != static_cast<int64_t>(d->heads) * d->head_dim) return fail(-1, "VX_GEMM_OUT_HEADS needs N = heads * head_dim");
      if (d->head_col_off < 0 || d->head_col_off % 8 != 0 || d->ldo % 8 != 0 || d->ldo < d->head_col_off + d->head_dim)
        return fail(-1, "VX_GEMM_OUT_HEADS: head_col_off / ldo must be multiples of 8 and ldo >= head_col_off + head_dim");
    }
  }
  if (argmax && (reinterpret_cast<uintptr_t>(d->out) & 7)) return fail(-1, "argmax keys must be 8-byte aligned");
  if (argmax && N > 0xffffffffll) return fail(-1, "argmax needs N < 2^32");
  if (d->lse_partials && (!argmax || fp8 || (reinterpret_cast<uintptr_t>(d->lse_partials) & 7)))
    return fail(-1, "lse_partials goes with VX_EPI_BIAS_ARGMAX on the FP4 formats and must be 8-byte aligned");
  if (d->lse_partials && (d->flags & VX_GEMM_NARROW_TILES)) return fail(-1, "lse_partials needs the wide tile");
  if (d->topk_threshold || d->topk_candidates || d->topk_count) {
    if (!d->lse_partials || !d->topk_threshold || !d->topk_candidates || !d->topk_count || d->topk_capacity <= 0 ||
        d->topk_capacity > 256 || (reinterpret_cast<uintptr_t>(d->topk_candidates) & 7))
      return fail(-1, "the top-k candidate pass needs lse_partials, topk_threshold, topk_candidates (8-byte aligned), "
                      "topk_count and 0 < topk_capacity <= 256");
  }
  if (d->out_dtype != VX_F32 && d->out_dtype != VX_BF16 && d->out_dtype != VX_FP4)
    return fail(-1, "unknown out_dtype %d", d->out_dtype);
  if (d->bias && (reinterpret_cast<uintptr_t>(d->bias) & 15)) return fail(-1, "bias must be 16-byte aligned");
  const bool vec2 = fmt == VX_FMT_ROWSCALE || fmt == VX_FMT_MX32;
  int kind = fp8 ? KIND_FP8 : (vec2 ? KIND_FP4_VEC2 : KIND_FP4_VEC4);
  if (!fp8) {
    // Two 128-wide accumulators overlap the epilogue of one tile with the MMAs of the next.
    // Measured at M = 90000, K = 512: that wins for the residual epilogue (N = 512: 52 vs
    // 57 us) and loses where the output is wide (N = 1536: 83 vs 78 us; N = 5538 argmax: 388 vs
    // 327 us), because every 128-wide column block re-reads A.  It also wins whenever the
    // wide tiling would leave SMs without a tile.  Swish (bound by its own epilogue
    // arithmetic) and GLU (weights interleaved per 256 rows) stay on the wide tile, and so
    // does a long K, where the wide tile halves the re-reads of A.
    const int64_t stages = (K / 2 + STAGE_ROW_BYTES - 1) / STAGE_ROW_BYTES;
    const int64_t wide_tiles = ((M + BM - 1) / BM) * ((N + 255) / 256);
    bool narrow = stages <= 2 && epi != VX_EPI_BIAS_SWISH && epi != VX_EPI_BIAS_GLU &&
                  (epi == VX_EPI_BIAS_RESIDUAL || wide_tiles < 148);
    // Few rows (a shard of a job cut over several GPUs): CTAs own column blocks and walk the row
    // blocks in rounds of sms / column-blocks, so what counts is the number of rounds times the cost of
    // a tile -- a narrow tile costs about 0.55 of a wide one.  88 row blocks, N = 512: the wide tiling
    // takes 2 rounds on 74 groups, the narrow one 3 half-size rounds on 37.
    if (!narrow && epi != VX_EPI_BIAS_SWISH && epi != VX_EPI_BIAS_GLU) {
      static int sm_cache[64] = {};
      int sms = 148, dev = 0;
      if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
        if (!sm_cache[dev] && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
          sm_cache[dev] = sms;
        if (sm_cache[dev]) sms = sm_cache[dev];
      }
      const int64_t mt = (M + BM - 1) / BM, ntw = (N + 255) / 256, ntn = (N + 127) / 128;
      auto rounds = [&](int64_t nt) {
        int64_t groups = nt <= sms ? sms / nt : 1;
        if (groups > mt) groups = mt;
        return nt <= sms ? (mt + groups - 1) / groups : (mt * nt + sms - 1) / sms;
      };
      if (0.55 * static_cast<double>(rounds(ntn)) < 0.95 * static_cast<double>(rounds(ntw))) narrow = true;
    }
    // Swish + FP4 output (the FFN up-projection) stays on the wide tile: the narrow tile's
    // 28-warp round-robin epilogue is faster per value, but its N = 128 MMAs read A from shared
    // memory twice as often and that chain then bounds the tile (measured 144 vs 134 us at
    // T = 90000); VX_GEMM_NARROW_TILES selects it.
    if (d->flags & VX_GEMM_WIDE_TILES) narrow = false;
    if (argmax && d->lse_partials) narrow = false;  // the partials are laid out per 64-column group of the wide tile
    if ((d->flags & VX_GEMM_NARROW_TILES) && epi != VX_EPI_BIAS_GLU) narrow = true;
    if (narrow) kind = vec2 ? KIND_FP4_VEC2_N128 : KIND_FP4_VEC4_N128;
  }
  const int BN = kind_bn(kind);
  if (epi == VX_EPI_BIAS_GLU && (N % BN != 0))
    return fail(-1, "GLU needs N %% %d == 0 (value / gate halves interleaved per tile, see vx_glu_tile)", BN);
  if (epi == VX_EPI_BIAS_RESIDUAL) {
    if (!d->residual) return fail(-1, "residual must not be NULL");
    if (d->residual_dtype != VX_F32 && d->residual_dtype != VX_BF16) return fail(-1, "bad residual dtype");
  }
  const int64_t n_out = epi == VX_EPI_BIAS_GLU ? N / 2 : N;

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = static_cast<int>((M + BM - 1) / BM);
  p.n_tiles = static_cast<int>((N + BN - 1) / BN);
  p.k_stages = static_cast<int>((row_bytes + STAGE_ROW_BYTES - 1) / STAGE_ROW_BYTES);
  if (static_cast<int64_t>(p.m_tiles) * p.n_tiles > 0x7fffffff) return fail(-1, "too many tiles");
  p.sf_kg = fmt_has_sf(fmt) ? sf_kgroups(fmt, K) : 0;
  p.sf_unit = fmt == VX_FMT_ROWSCALE;
  p.sf_e8m0 = fmt != VX_FMT_NV16;
  if (fmt == VX_FMT_ROWSCALE) {
    p.row_scale_u8 = static_cast<const uint8_t*>(d->a_scales);
    p.col_scale_u8 = static_cast<const uint8_t*>(d->b_scales);
  } else if (fp8) {
    p.fa = static_cast<const float*>(d->a_scales);
    p.fb = static_cast<const float*>(d->b_scales);
  } else {
    p.sfa = static_cast<const uint8_t*>(d->a_scales);
    p.sfb = static_cast<const uint8_t*>(d->b_scales);
  }
  if (fmt == VX_FMT_NV16) { p.a_amax = d->a_amax; p.b_amax = d->b_amax; }
  p.out_dtype = d->out_dtype;
  p.out = d->out; p.ldo = d->ldo;
  p.bias = d->bias;
  p.residual = d->residual; p.residual_dtype = d->residual_dtype; p.ldr = d->ldr; p.alpha = d->alpha;
  p.status = cached_status_ptr();

  if (qkvpack || out_heads) {
    p.heads = d->heads;
    p.head_dim = d->head_dim;
    p.head_col_off = qkvpack ? 0 : d->head_col_off;
    p.pos_u = static_cast<const __nv_bfloat16*>(d->pos_u);
    p.pos_v = static_cast<const __nv_bfloat16*>(d->pos_v);
    p.qk_scale = d->qk_scale;
  } else if (argmax) {
    p.out_dtype = VX_F32;
    p.lse_part = static_cast<float2*>(d->lse_partials);
    p.topk_thr = d->topk_threshold;
    p.topk_cand = static_cast<unsigned long long*>(d->topk_candidates);
    p.topk_cnt = d->topk_count;
    p.topk_cap = d->topk_capacity;
  } else if (d->out_dtype == VX_FP4) {
    if (d->out_fmt != VX_FMT_MX32 && d->out_fmt != VX_FMT_NV16) return fail(-1, "FP4 output: out_fmt must be MX32 or NV16");
    if (epi == VX_EPI_BIAS_GLU || epi == VX_EPI_BIAS_RESIDUAL) return fail(-1, "FP4 output supports NONE / BIAS / BIAS_SWISH");
    if (!d->out_scales_sf || !aligned16(d->out_scales_sf)) return fail(-1, "FP4 output needs out_scales_sf (16-byte aligned)");
    if (d->out_fmt == VX_FMT_NV16 && !d->out_amax) return fail(-1, "NV16 output needs out_amax");
    if (N % 128 != 0) return fail(-1, "FP4 output needs N %% 128 == 0");
    if (!aligned16(d->out) || d->ldo % 16 != 0 || d->ldo < N / 2) return fail(-1, "FP4 output rows must be 16-byte aligned");
    p.out_fmt = d->out_fmt;
    p.out_sf = static_cast<uint8_t*>(d->out_scales_sf);
    p.out_scales = static_cast<uint8_t*>(d->out_scales);
    p.out_sf_kg = sf_kgroups(d->out_fmt, N);
    p.out_amax = d->out_amax;
    if (p.out_scales && (reinterpret_cast<uintptr_t>(p.out_scales) & 3)) return fail(-1, "out_scales must be 4-byte aligned");
  } else {
    if (d->ldo < n_out) return fail(-1, "ldo=%lld < output columns %lld", (long long)d->ldo, (long long)n_out);
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (argmax) VX_CUDA_OK(cudaMemsetAsync(d->out, 0, static_cast<size_t>(M) * 8, st));
  if (!argmax && d->out_dtype == VX_FP4 && p.out_sf_kg * (d->out_fmt == VX_FMT_MX32 ? 128 : 64) != N) {
    // k-groups beyond N must read as zero (rows of the last tile beyond M: written as zero by the epilogue)
    VX_CUDA_OK(cudaMemsetAsync(p.out_sf, 0, static_cast<size_t>(vx_sf_bytes(d->out_fmt, M, N)), st));
  }

  CUtensorMap ta, tb, to;
  int rc = make_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d->a_codes, M, row_bytes, d->lda, 128, BM);
  if (rc) return rc;
  rc = make_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d->b_codes, N, row_bytes, d->ldb, 128, BN);
  if (rc) return rc;
  const int oelt = d->out_dtype == VX_BF16 ? 2 : 4;
  p.tma_store = 0;
  if (qkvpack || out_heads) {
    rc = qkvpack ? make_tmap_heads(&to, d->out, 3ll * d->heads, M, 2ll * d->head_dim)
                 : make_tmap_heads(&to, d->out, d->heads, M, d->ldo);
    if (rc) return rc;
    p.tma_store = 1;
  } else if (!argmax && d->out_dtype != VX_FP4 && !(d->flags & VX_GEMM_DIRECT_STORE) && aligned16(d->out) &&
      (d->ldo * oelt) % 16 == 0) {
    rc = make_tmap(&to, d->out_dtype == VX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                   oelt, d->out, M, n_out, d->ldo * oelt, 32, 32,
                   d->out_dtype == VX_BF16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    p.tma_store = 1;
  } else {
    to = ta;  // unused by the kernel
  }
  CUtensorMap tr = ta;
  p.tma_residual = 0;
  if (epi == VX_EPI_BIAS_RESIDUAL && p.tma_store && d->out_dtype == VX_BF16 && d->residual_dtype == VX_BF16 &&
      aligned16(d->residual) && (d->ldr * 2) % 16 == 0) {
    rc = make_tmap(&tr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d->residual, M, N, d->ldr * 2, 32, 32,
                   CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    p.tma_residual = 1;
  }
  const bool res = !(d->flags & VX_GEMM_STREAM_B);
  p.trace = g_trace_buffer;
  // compile-time output route (see bsgemm_kernel): 1 and 2 cover the encoder's launches
  int out_route = 0;
  if (!p.sf_unit) {
    if (d->out_dtype == VX_BF16 && p.tma_store && (epi != VX_EPI_BIAS_RESIDUAL || p.tma_residual) && !argmax)
      out_route = 1;
    else if (d->out_dtype == VX_FP4 && !argmax && d->out_fmt == (vec2 ? VX_FMT_MX32 : VX_FMT_NV16))
      out_route = 2;
  }
  switch (kind) {
    case KIND_FP8: return dispatch_epi<KIND_FP8>(epi, out_route, ta, tb, to, tr, p, res, st);
    case KIND_FP4_VEC2: return dispatch_epi<KIND_FP4_VEC2>(epi, out_route, ta, tb, to, tr, p, res, st);
    case KIND_FP4_VEC4: return dispatch_epi<KIND_FP4_VEC4>(epi, out_route, ta, tb, to, tr, p, res, st);
    case KIND_FP4_VEC2_N128: return dispatch_epi<KIND_FP4_VEC2_N128>(epi, out_route, ta, tb, to, tr, p, res, st);
    default: return dispatch_epi<KIND_FP4_VEC4_N128>(epi, out_route, ta, tb, to, tr, p, res, st);
  }
}

int vx_argmax_ids(const void* keys, int64_t M, int32_t* ids, float* max_out, void* stream) {
  using namespace vx;
  if (M < 0) return fail(-1, "negative M");
  if (M == 0) return 0;
  if (!keys || !ids) return fail(-1, "keys and ids must not be NULL");
  const int grid = static_cast<int>((M + 255) / 256);
  argmax_ids_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(keys), M, ids, max_out);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int vx_ctc_topk_threshold(const void* lse_partials, int64_t N, int64_t M, int k, float* threshold, void* stream) {
  using namespace vx;
  if (M < 0 || N <= 0) return fail(-1, "bad shape");
  if (M == 0) return 0;
  if (!lse_partials || !threshold) return fail(-1, "lse_partials and threshold must not be NULL");
  const int nparts = static_cast<int>(vx_ctc_lse_parts(N));
  if (k <= 0 || k > 16 || k > nparts) return fail(-1, "k must be in 1..16 and at most the number of 64-column groups (%d)", nparts);
  topk_threshold_kernel<<<static_cast<int>((M + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float2*>(lse_partials), nparts, M, k, threshold);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int vx_ctc_topk_finish(const void* candidates, const int32_t* count, int capacity, const void* lse_partials, int64_t N,
                       int64_t M, int k, int32_t* ids, float* logp, int32_t* overflow, void* stream) {
  using namespace vx;
  if (M < 0 || N <= 0) return fail(-1, "bad shape");
  if (M == 0) return 0;
  if (!candidates || !count || !lse_partials || !ids || !logp || !overflow) return fail(-1, "NULL argument");
  if (k <= 0 || k > 16 || capacity < k || capacity > 256) return fail(-1, "k must be in 1..16, capacity in k..256");
  topk_finish_kernel<<<static_cast<int>((M + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(candidates), count, capacity, static_cast<const float2*>(lse_partials),
      static_cast<int>(vx_ctc_lse_parts(N)), M, k, ids, logp, overflow);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int vx_wait_selftest(int64_t limit_ns, int site, void* stream) {
  using namespace vx;
  if (limit_ns <= 0 || limit_ns > 100000000ll) return fail(-1, "limit_ns must be in (0, 1e8] (at most 100 ms)");
  if (site < 0 || site > 254) return fail(-1, "site must be in [0, 254]");
  int* status = cached_status_ptr();
  if (!status) return fail(-2, "device status word unavailable");
  wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned long long>(limit_ns), site, status);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int vx_tmap_cache_stats(int64_t* hits, int64_t* misses) {
  using namespace vx;
  if (hits) *hits = static_cast<int64_t>(g_tmap_hits.load());
  if (misses) *misses = static_cast<int64_t>(g_tmap_misses.load());
  return 0;
}

int64_t vx_ctc_lse_parts(int64_t N) { return N <= 0 ? 0 : 4 * ((N + 255) / 256); }

int vx_ctc_finish(const void* keys, const void* lse_partials, int64_t N, int64_t M, int32_t* ids, float* max_out,
                  float* lse_out, float* logp_out, void* stream) {
  using namespace vx;
  if (M < 0 || N < 0) return fail(-1, "negative shape");
  if (M == 0) return 0;
  if (!keys) return fail(-1, "keys must not be NULL");
  if ((lse_out || logp_out) && !lse_partials) return fail(-1, "lse_out / logp_out need lse_partials");
  const int grid = static_cast<int>((M + 255) / 256);
  ctc_finish_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(keys), static_cast<const float2*>(lse_partials),
      static_cast<int>(vx_ctc_lse_parts(N)), M, ids, max_out, lse_out, logp_out);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int vx_glu_tile(int fmt) { return vx::kind_bn(fmt == VX_FMT_FP8_1X128 ? vx::KIND_FP8 : vx::KIND_FP4_VEC2); }

int vx_set_trace_buffer(void* device_buffer, int64_t bytes) {
  using namespace vx;
  if (device_buffer && !kPhaseTrace) return fail(-4, "this build has no phase trace (compile with -DVX_PHASE_TRACE=1)");
  if (device_buffer && bytes < static_cast<int64_t>(3 * TRACE_TILES * TRACE_EVENTS * sizeof(unsigned long long)))
    return fail(-1, "trace buffer needs %d bytes", (int)(3 * TRACE_TILES * TRACE_EVENTS * sizeof(unsigned long long)));
  g_trace_buffer = static_cast<unsigned long long*>(device_buffer);
  return 0;
}

int vx_mma_peak_probe(int kind, int n_tile, int iters, float* tflops_out) {
  using namespace vx;
  if (!tflops_out || iters <= 0) return fail(-1, "bad arguments");
  if (kind != 0 && kind != 1) return fail(-1, "kind must be 0 (FP4) or 1 (FP8)");
  if (n_tile != 128 && n_tile != 256) return fail(-1, "n_tile must be 128 or 256");
  int dev = 0, sms = 0;
  VX_CUDA_OK(cudaGetDevice(&dev));
  VX_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const size_t smem = TILE_BYTES + 256 * 128 + 512 + 1024;
  void (*k)(int, int*) = nullptr;
  if (kind == 0) k = n_tile == 128 ? mma_probe_kernel<KIND_FP4_VEC2, 128> : mma_probe_kernel<KIND_FP4_VEC2, 256>;
  else k = n_tile == 128 ? mma_probe_kernel<KIND_FP8, 128> : mma_probe_kernel<KIND_FP8, 256>;
  VX_CUDA_OK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  cudaEvent_t e0, e1;
  VX_CUDA_OK(cudaEventCreate(&e0));
  VX_CUDA_OK(cudaEventCreate(&e1));
  int* status = cached_status_ptr();
  k<<<sms, 128, smem>>>(iters / 8 + 1, status);  // warm-up
  VX_CUDA_OK(cudaEventRecord(e0));
  k<<<sms, 128, smem>>>(iters, status);
  VX_CUDA_OK(cudaEventRecord(e1));
  VX_CUDA_OK(cudaEventSynchronize(e1));
  VX_CUDA_OK(cudaGetLastError());
  float ms = 0.f;
  VX_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  const double k_per_mma = kind == 0 ? 64.0 : 32.0;
  const double flops = 2.0 * 128.0 * n_tile * k_per_mma * 4.0 * iters * sms;
  *tflops_out = static_cast<float>(flops / (ms * 1e-3) / 1e12);
  return 0;
}

}  // extern "C"

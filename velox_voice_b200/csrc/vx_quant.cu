// Activation / weight quantize + pack kernels (optionally fused behind LayerNorm), the
// tensor amax reduction NV16 needs, and the natural -> SF-atom scale relayout.
//
// Rounding rules (bit-exact contract with the reference quantizers,
// veloxvoice/kernels/ops/triton_ops.py:34-89 and :228-258):
//   UE8M0:  s = max(amax / 6, 1e-6); e = ceil(log2 s) taken from the fp32 bit pattern;
//           byte = clamp(e + 127, 0, 255); values are normalised by exactly 2^e.
//   E2M1:   magnitude code = number of thresholds {0.25, 0.75, 1.25, 1.75, 2.5, 3.5} strictly
//           exceeded (largest code emitted is 6); sign bit = (q < 0); low nibble = even k.
// NV16 and FP8_1X128 have no reference counterpart; their arithmetic is spelled out at
// nv16_block() / fp8_block() and uses only correctly rounded IEEE operations so that a CPU
// restatement reproduces every byte.
//
// Work decomposition: one warp per row (per row PAIR for BLK16_A).  A row is cut into chunks
// of 256 elements; in a chunk lane l owns elements [8 l, 8 l + 8): a bf16 row is read with one
// 16-byte load per lane (512 contiguous bytes per warp), codes leave as one 32-bit store per
// lane (128 contiguous bytes per warp).  Block maxima are warp-shuffle reductions over the
// 2 / 4 / 16 lanes that share a scale.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vx_common.cuh"
#include "vx_ptx.cuh"
#include "vx_quant_math.cuh"

namespace vx {
namespace {

struct QuantParams {
  const void* x;
  int64_t M, K, ldx;
  uint8_t* codes;
  int64_t ldc;
  void* scales;   // natural layout or nullptr
  uint8_t* sf;    // SF atoms or nullptr
  int64_t sf_kg;  // atoms per 128-row tile
  const float* amax;
  const float* gamma;
  const float* beta;
  const float* gamma2;  // second LayerNorm applied to the stored y (nullptr: single LayerNorm)
  const float* beta2;
  float eps;
  void* y;
  int y_bf16;
  int64_t ldy;
  int* status;  // device status word (bounded waits of the bulk-copy row rings report here)
};

// Eight consecutive elements as loaded (not yet converted): lets a kernel issue the loads of
// rows it will work on later before it works on the current one.  Converted, the eight values
// are four packed fp32 pairs (element 2 i in the low half of pair i): the arithmetic below uses
// the packed fp32x2 instructions of sm_100, which round each half exactly like the scalar ones.
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> {
  uint4 u;
  // plain (coherent) loads: the LayerNorm kernels may store y over x while other rows are still read
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void zero() { u = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void get(uint64_t (&v)[4]) const {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = pack_f32x2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  }
};
template <> struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void get(uint64_t (&v)[4]) const {
    v[0] = pack_f32x2(a.x, a.y); v[1] = pack_f32x2(a.z, a.w);
    v[2] = pack_f32x2(b.x, b.y); v[3] = pack_f32x2(b.z, b.w);
  }
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float warp_max(float a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  return a;
}

template <typename I>
__device__ __forceinline__ I sf_offset(I row, I kgroup, I sf_kg) {
  return ((row >> 7) * sf_kg + kgroup) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
}

// Quantize one 256-element chunk of RP rows held in registers and store codes + scales.
// `row_rcp` is used by ROWSCALE only (the row maximum is known beforehand).
// I: index type -- 32-bit when every element / byte offset of the call fits (most tensors; half
// the integer instructions of the 64-bit form), else 64-bit.
// FAST: the common call shape, fixed at compile time -- K a whole number of 256-element chunks
// (a power of two behind LayerNorm), scale factors wanted as SF atoms only -- drops the
// per-chunk bounds predicates, the natural-layout stores and their tests from the inner loop.
// BF16IN: the values are bf16 numbers (straight from a bf16 tensor, no arithmetic in between),
// which lets the power-of-two-scaled formats skip the tie nudge (see e2m1_pack8p).
// CANON: turn a normalised value that is (or underflows to) -0 into +0 before the encode, as the
// reference's `q < 0` sign test does.  The quantizers of plain tensors keep it; behind LayerNorm
// it is dropped (a LayerNorm output is -0 only for beta = -0, and y / scale underflows only when a
// block holds a value more than 2^125 times smaller than its maximum).
template <int FMT, int RP, typename I, bool FAST, bool BF16IN, bool CANON = true>
__device__ __forceinline__ void quant_chunk(const QuantParams& p, I row0, int c, int lane,
                                            uint64_t (&v)[RP][4], float row_rcp, float g) {
  const I K = static_cast<I>(p.K), M = static_cast<I>(p.M), ldc = static_cast<I>(p.ldc);
  const I k0 = static_cast<I>(c) * 256 + lane * 8;
  const bool active = FAST || k0 < K;
  constexpr bool NUDGE = !BF16IN;

  if constexpr (FMT == VX_FMT_ROWSCALE) {
    if (active) {
      *reinterpret_cast<uint32_t*>(p.codes + row0 * ldc + (k0 >> 1)) = e2m1_pack8p<true, CANON, NUDGE>(v[0], row_rcp);
    }
  } else if constexpr (FMT == VX_FMT_FP8_1X128) {
    float a = amax8p(v[0]);
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float scale, rcp;
    fp8_block(a, scale, rcp);
    if (active) {
      *reinterpret_cast<uint2*>(p.codes + row0 * ldc + k0) = fp8_pack8p(v[0], rcp);
      if (p.scales && (lane & 15) == 0)
        static_cast<float*>(p.scales)[row0 * (K >> 7) + (k0 >> 7)] = scale;
    }
  } else {
    constexpr int BLK = (FMT == VX_FMT_MX32) ? 32 : 16;
    constexpr int LPB = BLK / 8;  // lanes per block
    float a = amax8p(v[0]);
    if constexpr (RP == 2) a = fmaxf(a, amax8p(v[1]));
#pragma unroll
    for (int o = 1; o < LPB; o <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    uint32_t byte;
    float rcp;
    if constexpr (FMT == VX_FMT_NV16) nv16_block(a, g, byte, rcp);
    else ue8m0_from_amax(a, byte, rcp);
    if (!active) byte = 0;
    const I kb = k0 / BLK;  // block index along K
#pragma unroll
    for (int r = 0; r < RP; ++r) {
      if (active) {
        uint32_t w;
        if constexpr (FMT == VX_FMT_NV16) w = e2m1_pack8p<false, CANON, true>(v[r], rcp);
        else w = e2m1_pack8p<true, CANON, NUDGE>(v[r], rcp);
        *reinterpret_cast<uint32_t*>(p.codes + (row0 + r) * ldc + (k0 >> 1)) = w;
      }
    }
    if (!FAST && p.scales && active && (lane % LPB) == 0) {
      uint8_t* s = static_cast<uint8_t*>(p.scales);
      if constexpr (FMT == VX_FMT_BLK16_A) s[kb * (M >> 1) + (row0 >> 1)] = byte;
      else if constexpr (FMT == VX_FMT_BLK16_B) s[kb * M + row0] = byte;
      else s[row0 * (K / BLK) + kb] = byte;
    }
    if (FAST || p.sf) {
      // one byte per block, stored by the first lane of the block (the byte sits at
      // [k-group atom][row slot][kb % 4]); the 8 / 16 byte stores of a chunk are one instruction
      if ((FAST || active) && (lane % LPB) == 0) {
        const I kg = kb >> 2;
#pragma unroll
        for (int r = 0; r < RP; ++r)
          p.sf[sf_offset<I>(row0 + r, kg, static_cast<I>(p.sf_kg)) + (kb & 3)] = static_cast<uint8_t>(byte);
      }
    }
  }
}

// Scale-factor atoms cover rows in tiles of 128: the rows between M and the next multiple of
// 128 must read as zero scale factors (the GEMM multiplies their zero-filled operand rows by
// them).  Every k-group word of those rows is cleared here, by the kernel that fills the rest.
template <typename I>
__device__ __forceinline__ void zero_pad_rows(const QuantParams& p, I gwarp, I warps, int lane) {
  const I M = static_cast<I>(p.M), sf_kg = static_cast<I>(p.sf_kg);
  if (!p.sf || (M & 127) == 0) return;
  const I m_pad = (M + 127) & ~static_cast<I>(127);
  for (I r = M + gwarp; r < m_pad; r += warps)
    for (I kg = lane; kg < sf_kg; kg += 32)
      *reinterpret_cast<uint32_t*>(p.sf + sf_offset<I>(r, kg, sf_kg)) = 0u;
}

// Streaming quantizer (no LayerNorm): any K % 8 == 0.  A warp walks its (row, chunk) items in
// order with the loads of the next QDEPTH items already in flight: the kernel is bound by
// memory latency, not by arithmetic, so what counts is the number of bytes each SM keeps
// outstanding (QDEPTH x 512 B per warp for bf16 input).
#ifndef VX_QUANT_DEPTH
#define VX_QUANT_DEPTH 4
#endif
#ifndef VX_QUANT_MIN_BLOCKS
#define VX_QUANT_MIN_BLOCKS 5
#endif
#ifndef VX_LNQ_MIN_BLOCKS
#define VX_LNQ_MIN_BLOCKS 4
#endif
#ifndef VX_LNQ_DEPTH
#define VX_LNQ_DEPTH 2
#endif

// Row source of the bf16 fast lanes (TMA = true): every warp owns a ring of VX_ROW_RING row slots
// in shared memory that its lane 0 keeps filled with bulk asynchronous copies (cp.async.bulk,
// completion on one mbarrier per slot), VX_ROW_RING rows ahead of the row the warp works on.  The
// copies need no registers and no load instructions, so the bytes an SM keeps in flight are set by
// shared memory (blocks x 8 warps x ring x row bytes), not by the register file -- which is what
// it takes to keep HBM busy from kernels that spend ~200 instructions on a 1 KB row.  A slot is
// handed back to the copy engine after a warp-wide barrier (all lanes have read it).
#ifndef VX_ROW_RING
#define VX_ROW_RING 4
#endif
constexpr int kRingRowBytes = 1024;  // one slot: a bf16 row of up to 512 elements

template <typename T, int FMT, typename I, bool FAST, bool TMA = false>
__global__ void __launch_bounds__(256, VX_QUANT_MIN_BLOCKS) quant_kernel(const QuantParams p) {
  constexpr int RP = (FMT == VX_FMT_BLK16_A) ? 2 : 1;
  constexpr bool BF16IN = sizeof(T) == 2;
  static_assert(!TMA || (BF16IN && RP == 1 && FMT != VX_FMT_ROWSCALE), "bulk-copy ring: bf16 rows, one row per unit");
  constexpr int DEPTH = (FMT == VX_FMT_ROWSCALE) ? 1 : (BF16IN ? (RP == 2 ? 2 : VX_QUANT_DEPTH) : (RP == 2 ? 1 : 2));
  const int lane = threadIdx.x & 31;
  const I warps = static_cast<I>(gridDim.x) * (blockDim.x >> 5);
  const I nunits = static_cast<I>(p.M) / RP;
  const int nchunks = static_cast<int>((static_cast<I>(p.K) + 255) >> 8);
  const T* x = static_cast<const T*>(p.x);
  float g = 1.0f;
  if constexpr (FMT == VX_FMT_NV16) g = nv16_global(__ldg(p.amax));
  const I u_first = static_cast<I>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);

  if constexpr (TMA) {
    __shared__ __align__(128) uint8_t ring_s[8 * VX_ROW_RING * kRingRowBytes];
    __shared__ uint64_t full_s[8 * VX_ROW_RING];
    const int w = threadIdx.x >> 5;
    uint8_t* const ring_w = ring_s + w * VX_ROW_RING * kRingRowBytes;
    uint64_t* const full_w = full_s + w * VX_ROW_RING;
    const uint32_t row_bytes = static_cast<uint32_t>(p.K) * 2;
    if (lane == 0) {
#pragma unroll
      for (int d = 0; d < VX_ROW_RING; ++d) mbar_init(&full_w[d], 1);
      mbar_fence_init();
    }
    __syncwarp();
    auto issue = [&](int slot, I u) {
      if (lane == 0) {
        mbar_expect_tx(&full_w[slot], row_bytes);
        bulk_load(ring_w + slot * kRingRowBytes, x + u * static_cast<I>(p.ldx), row_bytes, &full_w[slot]);
      }
    };
#pragma unroll
    for (int d = 0; d < VX_ROW_RING; ++d)
      if (u_first + d * warps < nunits) issue(d, u_first + d * warps);
    int slot = 0;
    uint32_t par = 0;
#pragma unroll 1
    for (I u = u_first; u < nunits; u += warps) {
      if (!mbar_wait(&full_w[slot], par, p.status, 8)) break;
      uint64_t v[2][1][4];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int k0 = c * 256 + lane * 8;
        Raw8<T> raw;
        if ((FAST && c < nchunks) || k0 < p.K) raw.u = *reinterpret_cast<const uint4*>(ring_w + slot * kRingRowBytes + k0 * 2);
        else raw.zero();
        raw.get(v[c][0]);
      }
      __syncwarp();  // every lane has read the slot: hand it back
      if (u + VX_ROW_RING * warps < nunits) issue(slot, u + VX_ROW_RING * warps);
      if (++slot == VX_ROW_RING) { slot = 0; par ^= 1; }
#pragma unroll
      for (int c = 0; c < 2; ++c)
        if (c < nchunks) quant_chunk<FMT, 1, I, FAST, BF16IN>(p, u, c, lane, v[c], 0.0f, g);
    }
  } else if constexpr (FMT == VX_FMT_ROWSCALE) {
    // the row maximum comes first: the row is read twice (the second time from L1 / L2)
    for (I u = u_first; u < nunits; u += warps) {
      float a = 0.0f;
      for (int c = 0; c < nchunks; ++c) {
        const I k0 = static_cast<I>(c) * 256 + lane * 8;
        if (k0 < static_cast<I>(p.K)) {
          float t[8];
          load8(x + u * static_cast<I>(p.ldx) + k0, t);
          a = fmaxf(a, amax8(t));
        }
      }
      a = warp_max(a);
      uint32_t byte;
      float row_rcp;
      ue8m0_from_amax(a, byte, row_rcp);
      if (p.scales && lane == 0) static_cast<uint8_t*>(p.scales)[u] = static_cast<uint8_t>(byte);
      for (int c = 0; c < nchunks; ++c) {
        const I k0 = static_cast<I>(c) * 256 + lane * 8;
        Raw8<T> raw;
        if (k0 < static_cast<I>(p.K)) raw.load(x + u * static_cast<I>(p.ldx) + k0);
        else raw.zero();
        uint64_t v[1][4];
        raw.get(v[0]);
        quant_chunk<FMT, 1, I, false, BF16IN>(p, u, c, lane, v, row_rcp, g);
      }
    }
  } else {
    Raw8<T> raw[DEPTH][RP];
    // cursor of the item whose loads are issued next
    I fu = u_first;
    int fc = 0;
    auto fetch = [&](int slot) {
      // (called with compile-time slot numbers only: `raw` stays in registers)
      const I k0 = static_cast<I>(fc) * 256 + lane * 8;
#pragma unroll
      for (int r = 0; r < RP; ++r) {
        if (fu < nunits && (FAST || k0 < static_cast<I>(p.K))) raw[slot][r].load(x + (fu * RP + r) * static_cast<I>(p.ldx) + k0);
        else raw[slot][r].zero();
      }
      if (++fc == nchunks) { fc = 0; fu += warps; }
    };
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) fetch(d);
    I u = u_first;
    int c = 0;
#pragma unroll 1
    while (u < nunits) {
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        if (u < nunits) {  // warp-uniform
          uint64_t v[RP][4];
#pragma unroll
          for (int r = 0; r < RP; ++r) raw[d][r].get(v[r]);
          fetch(d);
          quant_chunk<FMT, RP, I, FAST, BF16IN>(p, u * RP, c, lane, v, 0.0f, g);
          if (++c == nchunks) { c = 0; u += warps; }
        }
      }
    }
  }
  zero_pad_rows<I>(p, u_first, warps, lane);
}

// One 64-bit value across lanes (two 32-bit shuffles).
__device__ __forceinline__ uint64_t shfl_xor_b64(uint64_t v, int o) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(v), o);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(v >> 32), o);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// LayerNorm + quantize, row resident in registers (CH chunks of 256 elements, K <= 256 CH).
// Statistics follow the reference kernel's formula (velox_layernorm.cu:52-57): mean = sum / K,
// var = max(E[x^2] - mean^2, 0), y = (x - mean) * rstd * gamma + beta, evaluated with fused
// multiply-adds in this fixed order (so that a CPU restatement can reproduce every bit):
//   per lane, pair j of chunk c (elements 2 j, 2 j + 1 of the lane's eight), chunks in order:
//       S = S + v            Q = fma(v, v, Q)               (packed: even | odd elements)
//   s = S.even + S.odd, q = Q.even + Q.odd; butterfly over the lanes (xor 16, 8, 4, 2, 1);
//   mean = s / K, ex2 = q / K (a multiplication when K is a power of two: same rounding),
//   var = max(fma(-mean, mean, ex2), 0), rstd = 1 / sqrt(var + eps) correctly rounded in one step,
//   y = fma(fma(x, rstd, -mean * rstd), gamma, beta).
// gamma / beta of both LayerNorms sit in shared memory, laid out so that the 16-byte reads of a
// warp touch every bank once.  Rows are loaded VX_LNQ_DEPTH iterations ahead of their use.
// resident blocks per SM the register budget is set for: the row lives in registers (16 CH values
// per thread), so the wider rows get fewer, larger-budget blocks
constexpr int lnq_min_blocks(int ch) { return ch <= 2 ? VX_LNQ_MIN_BLOCKS : (ch <= 4 ? 2 : 1); }

template <typename T, int FMT, int CH, typename I, bool FAST, bool TMA = false>
__global__ void __launch_bounds__(256, lnq_min_blocks(CH)) ln_quant_kernel(const QuantParams p) {
  constexpr int RP = (FMT == VX_FMT_BLK16_A) ? 2 : 1;
  constexpr int DEPTH = (CH * RP * (sizeof(T) / 2) <= 2) ? VX_LNQ_DEPTH : 1;
  static_assert(!TMA || (sizeof(T) == 2 && RP == 1 && CH == 2), "bulk-copy ring: bf16 rows of up to 512 elements");
  const int lane = threadIdx.x & 31;
  const I warps = static_cast<I>(gridDim.x) * (blockDim.x >> 5);
  const I nunits = static_cast<I>(p.M) / RP;
  const T* x = static_cast<const T*>(p.x);
  const float k_f = static_cast<float>(p.K);
  const int npass = p.gamma2 ? 2 : 1;
  float g = 1.0f;
  if constexpr (FMT == VX_FMT_NV16) g = nv16_global(__ldg(p.amax));

  // [pass][gamma | beta][16-byte piece: chunk * 2 + half][lane]
  __shared__ float4 gb_s[2][2][CH * 2][32];
  for (int i = threadIdx.x; i < npass * 2 * CH * 2 * 32; i += blockDim.x) {
    const int l = i & 31, piece = (i >> 5) % (CH * 2), which = (i >> 5) / (CH * 2);  // which = pass * 2 + (0 gamma, 1 beta)
    const float* src = which == 0 ? p.gamma : (which == 1 ? p.beta : (which == 2 ? p.gamma2 : p.beta2));
    const int k0 = (piece >> 1) * 256 + l * 8 + (piece & 1) * 4;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k0 < p.K) val = __ldg(reinterpret_cast<const float4*>(src + k0));
    gb_s[which >> 1][which & 1][piece][l] = val;
  }
  __syncthreads();

  const I u_first = static_cast<I>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  // LayerNorm(s) + quantization of unit u, whose RP rows arrive converted in v
  auto process = [&](const I u, uint64_t (&v)[CH][RP][4]) {
      const I row0 = u * RP;
      // one pass per LayerNorm: the second one (if any) normalises the rows as pass 0 stored them
#pragma unroll 1
      for (int pass = 0; pass < npass; ++pass) {
#pragma unroll
        for (int r = 0; r < RP; ++r) {
          uint64_t S = pack_f32x2(0.0f, 0.0f), Q = S;
#pragma unroll
          for (int c = 0; c < CH; ++c) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              S = add_f32x2(S, v[c][r][j]);
              Q = fma_f32x2(v[c][r][j], v[c][r][j], Q);
            }
          }
          float s0, s1, q0, q1;
          unpack_f32x2(S, s0, s1);
          unpack_f32x2(Q, q0, q1);
          uint64_t SQ = pack_f32x2(__fadd_rn(s0, s1), __fadd_rn(q0, q1));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) SQ = add_f32x2(SQ, shfl_xor_b64(SQ, o));
          float s, sq;
          unpack_f32x2(SQ, s, sq);
          // FAST: K is a power of two, so multiplying by 1/K gives the same correctly rounded quotient
          const float mean = FAST ? __fmul_rn(s, 1.0f / (CH * 256)) : __fdiv_rn(s, k_f);
          const float ex2 = FAST ? __fmul_rn(sq, 1.0f / (CH * 256)) : __fdiv_rn(sq, k_f);
          const float var = fmaxf(__fmaf_rn(-mean, mean, ex2), 0.0f);
          const float rstd = __frsqrt_rn(__fadd_rn(var, p.eps));
          const float nmr = __fmul_rn(-mean, rstd);
          const uint64_t R2 = pack_f32x2(rstd, rstd), N2 = pack_f32x2(nmr, nmr);
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            const I k0 = static_cast<I>(c) * 256 + lane * 8;
            if (FAST || k0 < static_cast<I>(p.K)) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const float4 ga = gb_s[pass][0][c * 2 + h][lane];
                const float4 be = gb_s[pass][1][c * 2 + h][lane];
                v[c][r][2 * h] = fma_f32x2(fma_f32x2(v[c][r][2 * h], R2, N2), pack_f32x2(ga.x, ga.y), pack_f32x2(be.x, be.y));
                v[c][r][2 * h + 1] =
                    fma_f32x2(fma_f32x2(v[c][r][2 * h + 1], R2, N2), pack_f32x2(ga.z, ga.w), pack_f32x2(be.z, be.w));
              }
              if (p.y && pass == 0) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) unpack_f32x2(v[c][r][j], f[2 * j], f[2 * j + 1]);
                if (p.y_bf16) {
                  uint4 w4;
                  w4.x = pack2_bf16(f[0], f[1]);
                  w4.y = pack2_bf16(f[2], f[3]);
                  w4.z = pack2_bf16(f[4], f[5]);
                  w4.w = pack2_bf16(f[6], f[7]);
                  *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.y) + (row0 + r) * static_cast<I>(p.ldy) + k0) = w4;
                  if (npass > 1) {  // the next LayerNorm reads what was stored
                    const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                      v[c][r][j] = pack_f32x2(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xffff0000u));
                  }
                } else {
                  float4* yp = reinterpret_cast<float4*>(static_cast<float*>(p.y) + (row0 + r) * static_cast<I>(p.ldy) + k0);
                  yp[0] = make_float4(f[0], f[1], f[2], f[3]);
                  yp[1] = make_float4(f[4], f[5], f[6], f[7]);
                }
              }
            }
          }
        }
      }
      if (!FAST && !p.codes) return;  // plain LayerNorm
      float row_rcp = 0.0f;
      if constexpr (FMT == VX_FMT_ROWSCALE) {
        float a = 0.0f;
#pragma unroll
        for (int c = 0; c < CH; ++c) a = fmaxf(a, amax8p(v[c][0]));
        a = warp_max(a);
        uint32_t byte;
        ue8m0_from_amax(a, byte, row_rcp);
        if (p.scales && lane == 0) static_cast<uint8_t*>(p.scales)[row0] = static_cast<uint8_t>(byte);
      }
#pragma unroll
      for (int c = 0; c < CH; ++c) quant_chunk<FMT, RP, I, FAST, false, false>(p, row0, c, lane, v[c], row_rcp, g);
  };

  if constexpr (TMA) {
    __shared__ __align__(128) uint8_t ring_s[8 * VX_ROW_RING * kRingRowBytes];
    __shared__ uint64_t full_s[8 * VX_ROW_RING];
    const int w = threadIdx.x >> 5;
    uint8_t* const ring_w = ring_s + w * VX_ROW_RING * kRingRowBytes;
    uint64_t* const full_w = full_s + w * VX_ROW_RING;
    const uint32_t row_bytes = static_cast<uint32_t>(p.K) * 2;
    if (lane == 0) {
#pragma unroll
      for (int d = 0; d < VX_ROW_RING; ++d) mbar_init(&full_w[d], 1);
      mbar_fence_init();
    }
    __syncwarp();
    auto issue = [&](int slot, I u) {
      if (lane == 0) {
        mbar_expect_tx(&full_w[slot], row_bytes);
        bulk_load(ring_w + slot * kRingRowBytes, x + u * static_cast<I>(p.ldx), row_bytes, &full_w[slot]);
      }
    };
#pragma unroll
    for (int d = 0; d < VX_ROW_RING; ++d)
      if (u_first + d * warps < nunits) issue(d, u_first + d * warps);
    int slot = 0;
    uint32_t par = 0;
#pragma unroll 1
    for (I u = u_first; u < nunits; u += warps) {
      if (!mbar_wait(&full_w[slot], par, p.status, 8)) break;
      uint64_t v[CH][RP][4];
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int k0 = c * 256 + lane * 8;
        Raw8<T> raw;
        if constexpr (sizeof(T) == 2) {
          if (FAST || k0 < p.K) raw.u = *reinterpret_cast<const uint4*>(ring_w + slot * kRingRowBytes + k0 * 2);
          else raw.zero();
        }
        raw.get(v[c][0]);
      }
      __syncwarp();  // every lane has read the slot: hand it back
      if (u + VX_ROW_RING * warps < nunits) issue(slot, u + VX_ROW_RING * warps);
      if (++slot == VX_ROW_RING) { slot = 0; par ^= 1; }
      process(u, v);
    }
  } else {
    Raw8<T> raw[DEPTH][CH][RP];
    auto fetch = [&](int slot, I u) {
#pragma unroll
      for (int r = 0; r < RP; ++r)
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const I k0 = static_cast<I>(c) * 256 + lane * 8;
          if (FAST || k0 < static_cast<I>(p.K)) raw[slot][c][r].load(x + (u * RP + r) * static_cast<I>(p.ldx) + k0);
          else raw[slot][c][r].zero();
        }
    };
#pragma unroll
    for (int d = 0; d < DEPTH; ++d)
      if (u_first + d * warps < nunits) fetch(d, u_first + d * warps);
#pragma unroll 1
    for (I ub = u_first; ub < nunits; ub += DEPTH * warps) {
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        const I u = ub + d * warps;
        if (u >= nunits) break;  // warp-uniform
        uint64_t v[CH][RP][4];
#pragma unroll
        for (int r = 0; r < RP; ++r)
#pragma unroll
          for (int c = 0; c < CH; ++c) raw[d][c][r].get(v[c][r]);
        if (u + DEPTH * warps < nunits) fetch(d, u + DEPTH * warps);
        process(u, v);
      }
    }
  }
  zero_pad_rows<I>(p, u_first, warps, lane);
}

// ---------------------------------------------------------------------------------------------
// The hot shape -- bf16 rows of exactly 512 elements, SF-atom formats / FP8 -- on HALF a warp per
// row: lane j of a half owns elements [32 j, 32 j + 32), a whole MX32 block (two NV16 blocks, a
// quarter of an FP8 block).  Against the warp-per-row kernels above that halves what a row costs
// in instructions: the per-row work (statistics butterfly, rsqrt, loop and ring handling) is shared
// by two rows per warp instruction, a block maximum needs no shuffle, and a scale is computed once
// per 32 elements instead of once per 8 by each of four lanes.
//
// Rows arrive through the per-warp bulk-copy ring (two rows per slot).  A lane reads its 64 bytes
// as four 16-byte pieces in ROTATED order -- step c reads piece (c + rot) & 3, rot = (j >> 1) & 3 --
// so that the eight lanes of a shared-memory phase touch eight different 16-byte columns (lanes
// 64 bytes apart would otherwise collide four ways).  Codes are rotated back in registers and
// leave as one 16-byte store per lane; y leaves piece by piece.
//
// LayerNorm arithmetic: as in ln_quant_kernel, with the lane's 32 values accumulated in the order
// they are read (steps c = 0..3, pairs 0..3 of each piece, packed even | odd) and the butterfly
// over the 16 lanes of the half (xor 8, 4, 2, 1).
#ifndef VX_R2_RING
#define VX_R2_RING 2
#endif
#ifndef VX_R2_MIN_BLOCKS
#define VX_R2_MIN_BLOCKS 4
#endif
#ifndef VX_R2_MIN_BLOCKS_LN
#define VX_R2_MIN_BLOCKS_LN 3  // 85 registers per thread: the LayerNorm lanes spill at 64
#endif
constexpr int kR2SlotBytes = 2048;  // two bf16 rows of 512 elements

template <int FMT, bool LN>
__global__ void __launch_bounds__(256, LN ? VX_R2_MIN_BLOCKS_LN : VX_R2_MIN_BLOCKS) rows2_kernel(const QuantParams p) {
  static_assert(FMT == VX_FMT_MX32 || FMT == VX_FMT_NV16 || FMT == VX_FMT_FP8_1X128, "SF-atom FP4 formats and FP8");
  constexpr bool CANON = !LN;            // see quant_chunk
  constexpr bool NUDGE = LN;             // plain bf16 values with a power-of-two scale need no tie nudge
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int h = lane >> 4, j = lane & 15, rot = (j >> 1) & 3;
  const int M = static_cast<int>(p.M);
  const int warps = static_cast<int>(gridDim.x) * 8;
  const int nunits = (M + 1) >> 1;
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.x);
  const int ldx = static_cast<int>(p.ldx), ldc = static_cast<int>(p.ldc), ldy = static_cast<int>(p.ldy);
  const int npass = LN ? (p.gamma2 ? 2 : 1) : 0;
  pdl_launch_dependents();

  __shared__ __align__(128) uint8_t ring_s[8 * VX_R2_RING * kR2SlotBytes];
  __shared__ uint64_t full_s[8 * VX_R2_RING];
  // [pass][gamma | beta][step c * 2 + half of the piece][lane of the half]: the eight values lane j
  // needs at step c, i.e. those of piece (c + rot_j) & 3 of its block
  __shared__ float4 gb_s[LN ? 2 : 1][2][8][16];
  if constexpr (LN) {
    for (int i = threadIdx.x; i < npass * 2 * 8 * 16; i += blockDim.x) {
      const int l = i & 15, piece = (i >> 4) & 7, which = i >> 7;  // which = pass * 2 + (0 gamma, 1 beta)
      const float* src = which == 0 ? p.gamma : (which == 1 ? p.beta : (which == 2 ? p.gamma2 : p.beta2));
      const int k0 = l * 32 + ((((piece >> 1) + (l >> 1)) & 3) << 3) + (piece & 1) * 4;
      gb_s[which >> 1][which & 1][piece][l] = __ldg(reinterpret_cast<const float4*>(src + k0));
    }
  }
  uint8_t* const ring_w = ring_s + w * VX_R2_RING * kR2SlotBytes;
  uint64_t* const full_w = full_s + w * VX_R2_RING;
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < VX_R2_RING; ++d) mbar_init(&full_w[d], 1);
    mbar_fence_init();
  }
  __syncthreads();
  // set-up done (LayerNorm parameters are constants of the model): from here on the kernel touches what
  // the previous kernel of the stream produced
  pdl_wait();
  float g = 1.0f;
  if constexpr (FMT == VX_FMT_NV16) g = nv16_global(__ldg(p.amax));

  auto issue = [&](int slot, int u) {
    if (lane == 0) {
      const int r0 = 2 * u;
      const bool two = r0 + 1 < M;
      mbar_expect_tx(&full_w[slot], two ? 2048u : 1024u);
      bulk_load(ring_w + slot * kR2SlotBytes, x + static_cast<int64_t>(r0) * ldx, 1024u, &full_w[slot]);
      if (two) bulk_load(ring_w + slot * kR2SlotBytes + 1024, x + static_cast<int64_t>(r0 + 1) * ldx, 1024u, &full_w[slot]);
    }
  };
  const int u_first = static_cast<int>(blockIdx.x) * 8 + w;
#pragma unroll
  for (int d = 0; d < VX_R2_RING; ++d)
    if (u_first + d * warps < nunits) issue(d, u_first + d * warps);
  int poff[4];  // byte offset of the piece read at step c within the lane's 64 bytes
#pragma unroll
  for (int c = 0; c < 4; ++c) poff[c] = ((c + rot) & 3) << 4;
  int slot = 0;
  uint32_t par = 0;
#pragma unroll 1
  for (int u = u_first; u < nunits; u += warps) {
    if (!mbar_wait(&full_w[slot], par, p.status, 8)) break;
    const int row = 2 * u + h;
    const bool valid = row < M;
    uint64_t v[4][4];
    {
      // (a half without a row -- the last unit of an odd M -- works on the other half's row and stores nothing)
      const uint8_t* src = ring_w + slot * kR2SlotBytes + (valid ? h : 0) * 1024 + j * 64;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        Raw8<__nv_bfloat16> raw;
        raw.u = *reinterpret_cast<const uint4*>(src + poff[c]);
        raw.get(v[c]);
      }
    }
    __syncwarp();  // every lane has read the slot: hand it back
    if (u + VX_R2_RING * warps < nunits) issue(slot, u + VX_R2_RING * warps);
    if (++slot == VX_R2_RING) { slot = 0; par ^= 1; }

    if constexpr (LN) {
#pragma unroll 1
      for (int pass = 0; pass < npass; ++pass) {
#ifndef VX_R2_SPLIT_STATS
#define VX_R2_SPLIT_STATS 0
#endif
        uint64_t S = pack_f32x2(0.0f, 0.0f), Q = S;
#if VX_R2_SPLIT_STATS
        uint64_t Sb = S, Qb = S;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            S = add_f32x2(S, v[c][i]);
            Q = fma_f32x2(v[c][i], v[c][i], Q);
            Sb = add_f32x2(Sb, v[c + 2][i]);
            Qb = fma_f32x2(v[c + 2][i], v[c + 2][i], Qb);
          }
        }
        S = add_f32x2(S, Sb);
        Q = add_f32x2(Q, Qb);
#else
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            S = add_f32x2(S, v[c][i]);
            Q = fma_f32x2(v[c][i], v[c][i], Q);
          }
        }
#endif
        float s0, s1, q0, q1;
        unpack_f32x2(S, s0, s1);
        unpack_f32x2(Q, q0, q1);
        uint64_t SQ = pack_f32x2(__fadd_rn(s0, s1), __fadd_rn(q0, q1));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) SQ = add_f32x2(SQ, shfl_xor_b64(SQ, o));
        float sm, sq;
        unpack_f32x2(SQ, sm, sq);
        const float mean = __fmul_rn(sm, 1.0f / 512.0f);
        const float ex2 = __fmul_rn(sq, 1.0f / 512.0f);
        const float var = fmaxf(__fmaf_rn(-mean, mean, ex2), 0.0f);
        const float rstd = __frsqrt_rn(__fadd_rn(var, p.eps));
        const float nmr = __fmul_rn(-mean, rstd);
        const uint64_t R2 = pack_f32x2(rstd, rstd), N2 = pack_f32x2(nmr, nmr);
        auto normalise = [&](int c) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const float4 ga = gb_s[pass][0][c * 2 + hh][j];
            const float4 be = gb_s[pass][1][c * 2 + hh][j];
            v[c][2 * hh] = fma_f32x2(fma_f32x2(v[c][2 * hh], R2, N2), pack_f32x2(ga.x, ga.y), pack_f32x2(be.x, be.y));
            v[c][2 * hh + 1] = fma_f32x2(fma_f32x2(v[c][2 * hh + 1], R2, N2), pack_f32x2(ga.z, ga.w), pack_f32x2(be.z, be.w));
          }
        };
        if (!(p.y && pass == 0)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) normalise(c);
        } else if (p.y_bf16) {
          __nv_bfloat16* const yrow = static_cast<__nv_bfloat16*>(p.y) + static_cast<int64_t>(row) * ldy + j * 32;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            normalise(c);
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) unpack_f32x2(v[c][i], f[2 * i], f[2 * i + 1]);
            uint4 w4;
            w4.x = pack2_bf16(f[0], f[1]);
            w4.y = pack2_bf16(f[2], f[3]);
            w4.z = pack2_bf16(f[4], f[5]);
            w4.w = pack2_bf16(f[6], f[7]);
            if (valid) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(yrow) + poff[c]) = w4;
            // a LayerNorm that follows reads what was stored
            const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) v[c][i] = pack_f32x2(__uint_as_float(ww[i] << 16), __uint_as_float(ww[i] & 0xffff0000u));
          }
        } else {
          float* const yrow = static_cast<float*>(p.y) + static_cast<int64_t>(row) * ldy + j * 32;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            normalise(c);
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) unpack_f32x2(v[c][i], f[2 * i], f[2 * i + 1]);
            if (valid) {
              float4* yp = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(yrow) + 2 * poff[c]);
              yp[0] = make_float4(f[0], f[1], f[2], f[3]);
              yp[1] = make_float4(f[4], f[5], f[6], f[7]);
            }
          }
        }
      }
    }

    // ---- quantize the lane's 32 values ----
    if (LN && !p.codes) continue;  // plain LayerNorm
    float a[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) a[c] = amax8p(v[c]);
    if constexpr (FMT == VX_FMT_FP8_1X128) {
      float am = fmaxf(max3(a[0], a[1], a[2]), a[3]);
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
      float scale, rcp;
      fp8_block(am, scale, rcp);
      if (valid) {
        uint8_t* dst = p.codes + static_cast<int64_t>(row) * ldc + j * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint2*>(dst + (poff[c] >> 1)) = fp8_pack8p(v[c], rcp);
        if (p.scales && (j & 3) == 0) static_cast<float*>(p.scales)[row * 4 + (j >> 2)] = scale;
      }
    } else {
      uint32_t wd[4];
      if constexpr (FMT == VX_FMT_MX32) {
        uint32_t byte;
        float rcp;
        ue8m0_from_amax(fmaxf(max3(a[0], a[1], a[2]), a[3]), byte, rcp);
#pragma unroll
        for (int c = 0; c < 4; ++c) wd[c] = e2m1_pack8p<true, CANON, NUDGE>(v[c], rcp);
        if (valid) {
          if (p.sf) p.sf[sf_offset<int>(row, j >> 2, static_cast<int>(p.sf_kg)) + (j & 3)] = static_cast<uint8_t>(byte);
          if (p.scales) static_cast<uint8_t*>(p.scales)[row * 16 + j] = static_cast<uint8_t>(byte);
        }
      } else {
        // two 16-element blocks: pieces 0, 1 and pieces 2, 3; piece of step c is (c + rot) & 3
        float a_lo = 0.0f, a_hi = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const bool lo = ((c + rot) & 2) == 0;
          a_lo = fmaxf(a_lo, lo ? a[c] : 0.0f);
          a_hi = fmaxf(a_hi, lo ? 0.0f : a[c]);
        }
        uint32_t b_lo, b_hi;
        float r_lo, r_hi;
        nv16_block(a_lo, g, b_lo, r_lo);
        nv16_block(a_hi, g, b_hi, r_hi);
#pragma unroll
        for (int c = 0; c < 4; ++c) wd[c] = e2m1_pack8p<false, CANON, true>(v[c], ((c + rot) & 2) == 0 ? r_lo : r_hi);
        if (valid) {
          if (p.sf)
            *reinterpret_cast<uint16_t*>(p.sf + sf_offset<int>(row, j >> 1, static_cast<int>(p.sf_kg)) + (j & 1) * 2) =
                static_cast<uint16_t>(b_lo | (b_hi << 8));
          if (p.scales) {
            uint8_t* sc = static_cast<uint8_t*>(p.scales) + row * 32 + 2 * j;
            sc[0] = static_cast<uint8_t>(b_lo);
            sc[1] = static_cast<uint8_t>(b_hi);
          }
        }
      }
      // word of step c belongs to piece (c + rot) & 3: rotate the four words back by rot
      if (rot & 1) { const uint32_t t = wd[3]; wd[3] = wd[2]; wd[2] = wd[1]; wd[1] = wd[0]; wd[0] = t; }
      if (rot & 2) { uint32_t t = wd[0]; wd[0] = wd[2]; wd[2] = t; t = wd[1]; wd[1] = wd[3]; wd[3] = t; }
      if (valid) *reinterpret_cast<uint4*>(p.codes + static_cast<int64_t>(row) * ldc + j * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    }
  }
  zero_pad_rows<int>(p, u_first, warps, lane);
}

int grid_for_rows(int64_t units, int blocks_per_sm);

// rows2_kernel takes every bf16 call with rows of 512 elements in an SF-atom FP4 format or FP8 (whatever
// scale layouts, y and LayerNorms are asked for), provided offsets fit 32 bits and code rows are 16-byte
// aligned -- so that for those calls the LayerNorm summation order does not depend on the options.
template <int FMT>
bool launch_rows2(const QuantParams& p, bool ln, cudaStream_t st) {
  if constexpr (FMT == VX_FMT_MX32 || FMT == VX_FMT_NV16 || FMT == VX_FMT_FP8_1X128) {
    int64_t ld = p.ldx > p.ldy ? p.ldx : p.ldy;
    if (p.codes && p.ldc > ld) ld = p.ldc;
    const bool small = (p.M + 128) * ld < (1ll << 31) && (p.M + 128) * (p.sf_kg * 4 + 1) < (1ll << 31);
    if (p.K != 512 || !small) return false;
    if (p.codes && ((p.ldc & 15) || (reinterpret_cast<uintptr_t>(p.codes) & 15))) return false;
    if (!p.codes && !ln) return false;
    if (ln) launch_dependent(rows2_kernel<FMT, true>, dim3(grid_for_rows((p.M + 1) / 2, VX_R2_MIN_BLOCKS_LN)), dim3(256), 0, st, p);
    else launch_dependent(rows2_kernel<FMT, false>, dim3(grid_for_rows((p.M + 1) / 2, VX_R2_MIN_BLOCKS)), dim3(256), 0, st, p);
    return true;
  } else {
    return false;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) amax_kernel(const T* x, int64_t M, int64_t K, int64_t ldx,
                                                   float* out) {
  const int64_t per_row = K >> 3;
  const int64_t total = M * per_row;
  float a = 0.0f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / per_row, k0 = (i - r * per_row) << 3;
    float t[8];
    load8(x + r * ldx + k0, t);
    a = fmaxf(a, amax8(t));
  }
  a = warp_max(a);
  // non-negative floats order like their bit patterns
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(a));
}

// natural scale layout -> SF atoms.  One thread per (row, k-group).
__global__ void sf_relayout_kernel(int fmt, const uint8_t* __restrict__ s, int64_t R, int64_t nkb,
                                   uint8_t* __restrict__ sf, int64_t sf_kg) {
  const int64_t ngroups = (nkb + 3) >> 2;
  const int64_t total = R * ngroups;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i % R, kg = i / R;
    uint32_t w = 0;
    for (int j = 0; j < 4; ++j) {
      const int64_t kb = kg * 4 + j;
      if (kb >= nkb) break;
      uint32_t b;
      if (fmt == VX_FMT_BLK16_A) b = s[kb * (R >> 1) + (row >> 1)];
      else if (fmt == VX_FMT_BLK16_B) b = s[kb * R + row];
      else b = s[row * nkb + kb];
      w |= b << (8 * j);
    }
    *reinterpret_cast<uint32_t*>(sf + sf_offset(row, kg, sf_kg)) = w;
  }
}

int sm_count() {
  static int cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

int grid_for_rows(int64_t units, int blocks_per_sm) {
  // 8 warps per block, one row (pair) per warp and iteration; exactly the blocks that are
  // resident at once, grid-stride beyond (every warp then takes the same number of rows +- 1).
  const int64_t blocks = (units + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * blocks_per_sm;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T, int FMT, typename I, bool FAST>
void launch_quant_idx(const QuantParams& p, bool ln, cudaStream_t st) {
  constexpr int RP = (FMT == VX_FMT_BLK16_A) ? 2 : 1;
  const int ch = p.K <= 512 ? 2 : (p.K <= 1024 ? 4 : 8);
  const int grid = grid_for_rows(p.M / RP, ln ? lnq_min_blocks(ch) * (ch > 2 ? 2 : 1) : VX_QUANT_MIN_BLOCKS);
  // bf16 rows of up to 512 elements, one row per unit: rows come through the per-warp bulk-copy rings
  constexpr bool tma_ok = sizeof(T) == 2 && RP == 1;
  const bool tma = tma_ok && p.K <= 512;
  if (!ln) {
    if constexpr (tma_ok && FMT != VX_FMT_ROWSCALE) {
      if (tma) {
        quant_kernel<T, FMT, I, FAST, true><<<grid, 256, 0, st>>>(p);
        return;
      }
    }
    quant_kernel<T, FMT, I, FAST><<<grid, 256, 0, st>>>(p);
  } else if (p.K <= 512) {
    if constexpr (tma_ok) {
      ln_quant_kernel<T, FMT, 2, I, FAST, true><<<grid, 256, 0, st>>>(p);
      return;
    }
    ln_quant_kernel<T, FMT, 2, I, FAST><<<grid, 256, 0, st>>>(p);
  } else if (p.K <= 1024) {
    ln_quant_kernel<T, FMT, 4, I, FAST><<<grid, 256, 0, st>>>(p);
  } else {
    ln_quant_kernel<T, FMT, 8, I, FAST><<<grid, 256, 0, st>>>(p);
  }
}

template <typename T, int FMT>
void launch_quant(const QuantParams& p, bool ln, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    if (launch_rows2<FMT>(p, ln, st)) return;
  }
  // 32-bit indices when every offset the kernels form stays below 2^31 (rows padded to 128 for
  // the scale-factor atoms; strides in elements, y possibly fp32)
  int64_t ld = p.K;
  if (p.ldx > ld) ld = p.ldx;
  if (p.ldy > ld) ld = p.ldy;
  if (p.ldc > ld && p.codes) ld = p.ldc;
  const bool small = (p.M + 128) * ld < (1ll << 31) && (p.M + 128) * (p.sf_kg * 4 + 1) < (1ll << 31);
  // FAST (see quant_chunk): SF-atom formats, whole chunks, no natural-layout scales; behind
  // LayerNorm K must also fill its register chunks exactly (512, 1024 or 2048)
  constexpr bool sf_fmt = FMT == VX_FMT_MX32 || FMT == VX_FMT_NV16 || FMT == VX_FMT_BLK16_A || FMT == VX_FMT_BLK16_B;
  const bool fast = sf_fmt && small && p.codes && p.sf && !p.scales && p.K % 256 == 0 &&
                    (!ln || p.K == 512 || p.K == 1024 || p.K == 2048);
  if constexpr (sf_fmt) {
    if (fast) return launch_quant_idx<T, FMT, int32_t, true>(p, ln, st);
  }
  if (small) launch_quant_idx<T, FMT, int32_t, false>(p, ln, st);
  else launch_quant_idx<T, FMT, int64_t, false>(p, ln, st);
}

template <typename T>
int dispatch_fmt(int fmt, const QuantParams& p, bool ln, cudaStream_t st) {
  switch (fmt) {
    case VX_FMT_ROWSCALE: launch_quant<T, VX_FMT_ROWSCALE>(p, ln, st); break;
    case VX_FMT_BLK16_A: launch_quant<T, VX_FMT_BLK16_A>(p, ln, st); break;
    case VX_FMT_BLK16_B: launch_quant<T, VX_FMT_BLK16_B>(p, ln, st); break;
    case VX_FMT_MX32: launch_quant<T, VX_FMT_MX32>(p, ln, st); break;
    case VX_FMT_NV16: launch_quant<T, VX_FMT_NV16>(p, ln, st); break;
    case VX_FMT_FP8_1X128: launch_quant<T, VX_FMT_FP8_1X128>(p, ln, st); break;
    default: return fail(-1, "unknown format %d", fmt);
  }
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int quantize_common(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int fmt,
                    void* codes, int64_t ldc, void* scales, void* scales_sf, const float* amax,
                    bool ln, const float* gamma, const float* beta, float eps, void* y,
                    int y_dtype, int64_t ldy, void* stream, const float* gamma2 = nullptr,
                    const float* beta2 = nullptr) {
  if (!fmt_valid(fmt)) return fail(-1, "unknown format %d", fmt);
  if (x_dtype != VX_F32 && x_dtype != VX_BF16) return fail(-1, "x_dtype must be VX_F32 or VX_BF16");
  if (M < 0 || K < 0) return fail(-1, "negative shape");
  if (M == 0 || K == 0) return 0;
  if (!x) return fail(-1, "x must not be NULL");
  if (!codes && !(ln && y)) return fail(-1, "codes must not be NULL");
  if (!codes) { scales = nullptr; scales_sf = nullptr; if (fmt == VX_FMT_NV16) fmt = VX_FMT_MX32; ldc = 1 << 30; codes = nullptr; }
  const int blk = fmt_block(fmt);
  if (K % 8 != 0 || (blk && K % blk != 0))
    return fail(-1, "K=%lld must be a multiple of 8 and of the scale block (%d)", (long long)K, blk);
  if (fmt == VX_FMT_BLK16_A && (M & 1)) return fail(-1, "BLK16_A needs an even row count");
  const int64_t esz = x_dtype == VX_BF16 ? 2 : 4;
  if (ldx < K || !aligned16(x) || (ldx * esz) % 16 != 0)
    return fail(-1, "x rows must be 16-byte aligned (ldx=%lld)", (long long)ldx);
  const int64_t row_bytes = fmt == VX_FMT_FP8_1X128 ? K : K / 2;
  if (codes && (ldc < row_bytes || ldc % 4 != 0 || (reinterpret_cast<uintptr_t>(codes) & 7) != 0 ||
      (fmt == VX_FMT_FP8_1X128 && ldc % 8 != 0)))
    return fail(-1, "codes rows must be >= %lld bytes and 4/8-byte aligned (ldc=%lld)",
                (long long)row_bytes, (long long)ldc);
  if (fmt == VX_FMT_NV16 && !amax) return fail(-1, "NV16 needs the tensor amax");
  if (scales_sf && !fmt_has_sf(fmt)) return fail(-1, "format %d has no SF-atom layout", fmt);
  if (scales_sf && (reinterpret_cast<uintptr_t>(scales_sf) & 15))
    return fail(-1, "scales_sf must be 16-byte aligned");
  if (fmt == VX_FMT_FP8_1X128 && scales && (reinterpret_cast<uintptr_t>(scales) & 3))
    return fail(-1, "fp32 scales must be 4-byte aligned");
  if (ln) {
    if (!gamma || !beta) return fail(-1, "gamma and beta must not be NULL");
    if (K > 2048) return fail(-1, "fused LayerNorm supports K <= 2048 (K=%lld)", (long long)K);
    if (!aligned16(gamma) || !aligned16(beta)) return fail(-1, "gamma/beta must be 16-byte aligned");
    if (y && y_dtype != VX_F32 && y_dtype != VX_BF16) return fail(-1, "y_dtype must be VX_F32 or VX_BF16");
    if (y && (!aligned16(y) || ldy < K || (ldy * (y_dtype == VX_BF16 ? 2 : 4)) % 16 != 0))
      return fail(-1, "y rows must be 16-byte aligned");
    if ((gamma2 != nullptr) != (beta2 != nullptr)) return fail(-1, "gamma2 and beta2 go together");
    if (gamma2 && (!aligned16(gamma2) || !aligned16(beta2))) return fail(-1, "gamma2/beta2 must be 16-byte aligned");
    if (gamma2 && !codes) return fail(-1, "the second LayerNorm feeds the quantizer: codes must not be NULL");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  QuantParams p{};
  p.x = x; p.M = M; p.K = K; p.ldx = ldx;
  p.codes = static_cast<uint8_t*>(codes); p.ldc = ldc;
  p.scales = scales; p.sf = static_cast<uint8_t*>(scales_sf);
  p.sf_kg = sf_kgroups(fmt, K);
  p.status = device_status_ptr();
  p.amax = amax; p.gamma = gamma; p.beta = beta; p.gamma2 = gamma2; p.beta2 = beta2; p.eps = eps; p.y = y; p.y_bf16 = (y_dtype == VX_BF16); p.ldy = ldy;
  if (scales_sf) {
    // k-groups beyond K must read as zero scale factors (rows beyond M: cleared by the kernel)
    const int64_t nkb = K / blk;
    if (p.sf_kg * 4 != nkb)
      VX_CUDA_OK(cudaMemsetAsync(scales_sf, 0, static_cast<size_t>(vx_sf_bytes(fmt, M, K)), st));
  }
  return x_dtype == VX_BF16 ? dispatch_fmt<__nv_bfloat16>(fmt, p, ln, st)
                            : dispatch_fmt<float>(fmt, p, ln, st);
}

}  // namespace
}  // namespace vx

extern "C" {

int64_t vx_sf_kgroups(int fmt, int64_t K) { return vx::fmt_has_sf(fmt) ? vx::sf_kgroups(fmt, K) : 0; }

int64_t vx_sf_bytes(int fmt, int64_t R, int64_t K) {
  if (!vx::fmt_has_sf(fmt)) return 0;
  return ((R + 127) / 128) * vx::sf_kgroups(fmt, K) * 512;
}

int vx_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int fmt,
                     void* codes, int64_t ldc, void* scales, void* scales_sf, const float* amax,
                     void* stream) {
  return vx::quantize_common(x, x_dtype, M, K, ldx, fmt, codes, ldc, scales, scales_sf, amax, false,
                             nullptr, nullptr, 0.f, nullptr, 0, 0, stream);
}

int vx_ln_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                        const float* gamma, const float* beta, float eps, int fmt, void* codes,
                        int64_t ldc, void* scales, void* scales_sf, const float* amax, void* y,
                        int y_dtype, int64_t ldy, void* stream) {
  return vx::quantize_common(x, x_dtype, M, K, ldx, fmt, codes, ldc, scales, scales_sf, amax, true,
                             gamma, beta, eps, y, y_dtype, ldy, stream);
}

int vx_ln2_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                         const float* gamma1, const float* beta1, const float* gamma2,
                         const float* beta2, float eps, int fmt, void* codes, int64_t ldc,
                         void* scales, void* scales_sf, const float* amax, void* y, int y_dtype,
                         int64_t ldy, void* stream) {
  if (!gamma2 || !beta2) return vx::fail(-1, "gamma2 and beta2 must not be NULL");
  return vx::quantize_common(x, x_dtype, M, K, ldx, fmt, codes, ldc, scales, scales_sf, amax, true,
                             gamma1, beta1, eps, y, y_dtype, ldy, stream, gamma2, beta2);
}

int vx_amax(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, float* amax_out,
            void* stream) {
  using namespace vx;
  if (x_dtype != VX_F32 && x_dtype != VX_BF16) return fail(-1, "x_dtype must be VX_F32 or VX_BF16");
  if (!amax_out) return fail(-1, "amax_out must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VX_CUDA_OK(cudaMemsetAsync(amax_out, 0, sizeof(float), st));
  if (M <= 0 || K <= 0) return 0;
  const int64_t esz = x_dtype == VX_BF16 ? 2 : 4;
  if (!x || K % 8 != 0 || !aligned16(x) || (ldx * esz) % 16 != 0 || ldx < K)
    return fail(-1, "x must be 16-byte aligned rows with K %% 8 == 0");
  const int64_t threads = M * (K >> 3);
  int grid = static_cast<int>((threads + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  if (x_dtype == VX_BF16)
    amax_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), M, K, ldx, amax_out);
  else
    amax_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(x), M, K, ldx, amax_out);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

int vx_sf_from_natural(int fmt, const void* scales, int64_t R, int64_t K, void* scales_sf,
                       void* stream) {
  using namespace vx;
  if (!fmt_has_sf(fmt)) return fail(-1, "format %d has no SF-atom layout", fmt);
  if (R <= 0 || K <= 0) return 0;
  if (!scales || !scales_sf || (reinterpret_cast<uintptr_t>(scales_sf) & 15))
    return fail(-1, "scales / scales_sf must be non-NULL, scales_sf 16-byte aligned");
  const int blk = fmt_block(fmt);
  if (K % blk != 0) return fail(-1, "K must be a multiple of %d", blk);
  if (fmt == VX_FMT_BLK16_A && (R & 1)) return fail(-1, "BLK16_A needs an even row count");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VX_CUDA_OK(cudaMemsetAsync(scales_sf, 0, static_cast<size_t>(vx_sf_bytes(fmt, R, K)), st));
  const int64_t nkb = K / blk;
  const int64_t total = R * ((nkb + 3) / 4);
  int grid = static_cast<int>((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  sf_relayout_kernel<<<grid, 256, 0, st>>>(fmt, static_cast<const uint8_t*>(scales), R, nkb,
                                           static_cast<uint8_t*>(scales_sf), sf_kgroups(fmt, K));
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"

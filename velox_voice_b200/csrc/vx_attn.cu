// Relative-position attention of the Conformer encoder on the folded operands of the attention
// fold pack (vx_qkv_pack / the QKV GEMM's fold-pack epilogue):
//
//   q2[h, t, :] = ((q + pos_u) | (q + pos_v)) / sqrt(dk)      k2[h, t, :] = k | p      v2[h, t, 0:dk] = v
//   out[t, h dk : (h + 1) dk] = softmax_j(q2[h, t, :] . k2[h, j, :]) v[h, j, :]        (keys j < kv_len)
//
// i.e. what the model computes with scaled_dot_product_attention(q2, k2, v2, scale = 1)[..., :dk] followed
// by transpose(1, 2).reshape (veloxvoice/models/wenet/torch_conformer.py:514-519; the reference's own
// CUDA kernel for the chunked case is veloxvoice/kernels/csrc/velox_chunk_rel_pos_attn.cu:23-114).  The zero
// half of v2 is never read and the result lands token-major, ready for the output projection's quantizer.
//
// One CTA = 128 queries of one head, all on the 5th-generation tensor cores (tcgen05.mma kind::f16, bf16
// operands, fp32 accumulators in tensor memory):
//   warp 0      TMA producer: Q once, then K (and V) tiles of 128 keys through a three-stage ring;
//   warp 1      MMA issuer: S = Q K^T (128 x 128 x 128) into one of two S accumulators, O += P V
//               (128 x 64 x 128; V is read in its natural [key][dv] layout as an MN-major operand);
//   warps 2..9  softmax, one query row per thread straight out of tensor memory; two warps share a row
//               (64 of a tile's 128 keys each) and exchange their maxima / sums through shared memory once.
// One pass over the keys with a lazily updated reference maximum: p = 2^((s - m_ref) log2 e) is formed
// against the reference m_ref the row has used so far, which only moves when a tile's maximum exceeds it by
// more than 2^8 (so p never exceeds 256 and nothing overflows in bf16 or fp32).  When it moves -- typically in
// the first tiles of a row only -- the row sum and the row's part of the O accumulator in tensor memory are
// multiplied by 2^((m_old - m_new) log2 e) (tcgen05.ld / tcgen05.st of 32 columns per warp) before the next
// P V product is released.  P is written as bf16 into the swizzled K-major tile the P V product reads; O is
// divided by the row sum once at the end.
// Every mbarrier wait is bounded.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "vx_common.cuh"
#include "vx_ptx.cuh"
#include "vx_tmap.cuh"

namespace vx {
namespace {

constexpr int AT_BM = 128;   // queries per CTA = TMEM lanes
constexpr int AT_BN = 128;   // keys per tile
constexpr int AT_D = 128;    // folded head dimension (2 dk)
constexpr int AT_DV = 64;    // value dimension (dk)
constexpr int AT_PANEL = AT_BM * 128;            // one 64-column bf16 panel of 128 rows: 16 KB
constexpr int AT_Q_BYTES = 2 * AT_PANEL;          // 32 KB
constexpr int AT_K_BYTES = 2 * AT_PANEL;          // 32 KB
constexpr int AT_V_BYTES = AT_BN * AT_DV * 2;     // 16 KB
constexpr int AT_STAGE = AT_K_BYTES + AT_V_BYTES; // 48 KB
constexpr int AT_P_BYTES = 2 * AT_PANEL;          // 32 KB
constexpr int AT_NS = 3;                          // K / V stages in flight
constexpr int AT_SMEM = AT_Q_BYTES + AT_NS * AT_STAGE + AT_P_BYTES + 1024;
constexpr int AT_SOFTMAX_WARPS = 8;  // two per 32-row quadrant of tensor memory: 64 of a tile's 128 keys each
constexpr int AT_THREADS = (2 + AT_SOFTMAX_WARPS) * 32;
constexpr uint32_t AT_TM_S = 0, AT_TM_O = 256;    // S0 | S1 (128 columns each) | O (64 columns)

struct AttnParams {
  int64_t T;        // queries and keys per head
  int64_t kv_len;   // keys j >= kv_len are masked
  int heads;
  __nv_bfloat16* out;
  int64_t ldo;
  int* status;
};

struct AttnBarriers {
  uint64_t q_full, kv_full[AT_NS], kv_empty[AT_NS], s_full[2], s_empty[2], p_full, p_empty, o_full;
  uint32_t tmem_base;
  float xch[2][2][AT_BM];  // [tile parity][half][row]: tile maxima (finally row sums) of the two warps that share a row
};

// bf16 x bf16 -> fp32, A K-major; B K-major or MN-major (b_mn)
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// shared-memory descriptor with the 128-byte swizzle and explicit leading / stride byte offsets
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ void tc_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(AT_THREADS, 1)
relpos_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* const q_s = base;
  uint8_t* const st_s = base + AT_Q_BYTES;        // AT_NS stages of [K | V]
  uint8_t* const p_s = st_s + AT_NS * AT_STAGE;
  __shared__ AttnBarriers bar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int64_t q0 = static_cast<int64_t>(blockIdx.x) * AT_BM;
  const int nkb = static_cast<int>((p.kv_len + AT_BN - 1) / AT_BN);
  const int iters = nkb;
  const int row_base = static_cast<int>(head * p.T);  // this head's token 0 in the [heads * T, 128] views

  if (threadIdx.x == 0) {
    mbar_init(&bar.q_full, 1);
    for (int s = 0; s < AT_NS; ++s) {
      mbar_init(&bar.kv_full[s], 1);
      mbar_init(&bar.kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar.s_full[s], 1);
      mbar_init(&bar.s_empty[s], AT_SOFTMAX_WARPS);
    }
    mbar_init(&bar.p_full, AT_SOFTMAX_WARPS);
    mbar_init(&bar.p_empty, 1);
    mbar_init(&bar.o_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(&bar.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar.tmem_base;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      mbar_expect_tx(&bar.q_full, AT_Q_BYTES);
      tma_load_2d(q_s, &tm_q, 0, row_base + static_cast<int>(q0), &bar.q_full);
      tma_load_2d(q_s + AT_PANEL, &tm_q, 64, row_base + static_cast<int>(q0), &bar.q_full);
      for (int it = 0; it < iters; ++it) {
        const int s = it % AT_NS, j = it;
        if (!mbar_wait(&bar.kv_empty[s], ((it / AT_NS) & 1) ^ 1, p.status, 20)) break;
        uint8_t* const dst = st_s + s * AT_STAGE;
        mbar_expect_tx(&bar.kv_full[s], AT_K_BYTES + AT_V_BYTES);
        tma_load_2d(dst, &tm_k, 0, row_base + j * AT_BN, &bar.kv_full[s]);
        tma_load_2d(dst + AT_PANEL, &tm_k, 64, row_base + j * AT_BN, &bar.kv_full[s]);
        tma_load_2d(dst + AT_K_BYTES, &tm_v, 0, row_base + j * AT_BN, &bar.kv_full[s]);
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_bf16(AT_BM, AT_BN, false);
    const uint32_t idesc_o = make_idesc_bf16(AT_BM, AT_DV, true);
    const uint32_t q_u32 = smem_u32(q_s), st_u32 = smem_u32(st_s), p_u32 = smem_u32(p_s);
    bool ok = mbar_wait_spin(&bar.q_full, 0, p.status, 21);
    // S(it) = Q K_j^T into accumulator it & 1
    auto issue_s = [&](int it) {
      const int s = it & 1, ks = it % AT_NS;  // S accumulator, K / V stage
      if (!mbar_wait_spin(&bar.kv_full[ks], (it / AT_NS) & 1, p.status, 22)) return false;
      if (!mbar_wait_spin(&bar.s_empty[s], ((it >> 1) & 1) ^ 1, p.status, 23)) return false;
      tc_fence_after();
      if (leader) {
        const uint32_t k_u32 = st_u32 + ks * AT_STAGE;
#pragma unroll
        for (int i = 0; i < AT_D / 16; ++i) {
          const uint32_t off = (i >> 2) * AT_PANEL + (i & 3) * 32;
          mma_bf16(tmem_base + AT_TM_S + s * 128, make_desc_k128(q_u32 + off), make_desc_k128(k_u32 + off), idesc_s, i != 0);
        }
        tc_commit(&bar.s_full[s]);
      }
      __syncwarp();
      return true;
    };
    if (ok && iters > 0) ok = issue_s(0);
    for (int it = 0; it < iters && ok; ++it) {
      if (it + 1 < iters) ok = issue_s(it + 1);
      if (!ok) break;
      {
        const int n = it;
        if (!mbar_wait_spin(&bar.p_full, n & 1, p.status, 24)) { ok = false; break; }
        tc_fence_after();
        if (leader) {
          const uint32_t v_u32 = st_u32 + (it % AT_NS) * AT_STAGE + AT_K_BYTES;
#pragma unroll
          for (int i = 0; i < AT_BN / 16; ++i) {
            const uint32_t aoff = (i >> 2) * AT_PANEL + (i & 3) * 32;
            // V tile as TMA wrote it: one 128-byte row of 64 dv values per key, 8-key swizzle atoms 1 KB apart
            // (the stride offset of the MN-major operand); 64 dv values are one group along N, so the leading
            // offset is not used.  A K = 16 step is two atoms.
            mma_bf16(tmem_base + AT_TM_O, make_desc_k128(p_u32 + aoff), make_desc_sw128(v_u32 + i * 16 * 128, 0, 1024),
                     idesc_o, (n | i) != 0);
          }
          tc_commit(&bar.p_empty);
          tc_commit(&bar.kv_empty[it % AT_NS]);
          if (it == iters - 1) tc_commit(&bar.o_full);
        }
        __syncwarp();
      }
    }
  } else {
    // =========================== softmax: warps 2..9 ===========================
    // warp -> (quadrant q of tensor memory = rows 32 q .. 32 q + 31, half of the tile's keys / of O's columns)
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    constexpr float L2E = 1.4426950408889634f;
    const float NEG_INF = __int_as_float(0xff800000);
    float m_ref = NEG_INF;  // reference maximum of the row, in units of log2 (s * log2 e)
    float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    auto softmax_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX_WARPS * 32) : "memory"); };
    bool ok = true;
    int syncs = 0;  // named barriers this thread has executed (every softmax thread executes nkb + 1 of them)
    for (int it = 0; it < iters && ok; ++it) {
      const int b = it & 1;
      if (lane == 0) ok = mbar_wait(&bar.s_full[b], (it >> 1) & 1, p.status, 25);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const int n_valid = static_cast<int>(p.kv_len - static_cast<int64_t>(it) * AT_BN);  // >= 128: the whole tile
      // this warp's 64 keys of the tile, scaled to log2 units
      float t[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t r[32];
        tc_ld_32x32b_x32(lane_addr + AT_TM_S + b * 128 + (half * 2 + cc) * 32, r);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) t[cc][i] = __uint_as_float(r[i]) * L2E;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.s_empty[b]);  // S is in registers: the accumulator may be overwritten
      if (n_valid < AT_BN) {
        // the last tile of a span whose length is not a multiple of 128: keys beyond kv_len count as -inf
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((half * 2 + cc) * 32 + i >= n_valid) t[cc][i] = NEG_INF;
      }
      float m4[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
#pragma unroll
        for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], t[cc][i]);
      const float mine = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      bar.xch[it & 1][half][row] = mine;
      softmax_sync();
      ++syncs;
      const float m_tile = fmaxf(mine, bar.xch[it & 1][half ^ 1][row]);
      // The reference of a row moves when the tile's maximum exceeds it by more than 8 (both warps of a row
      // decide alike: same lanes, same values).  Then the row sum and this warp's 32 columns of O are scaled by
      // 2^(m_ref - m_tile).  The tensor-memory accesses are warp-wide, so the warp goes through them when any of
      // its rows moves; the other rows scale by one.  Before the first P V product there is nothing to scale.
      const bool moves = m_tile > m_ref + 8.0f;
      const bool any_moves = __any_sync(0xffffffffu, moves);
      const float alpha = moves ? ex2f(m_ref - m_tile) : 1.0f;  // 0 for m_ref = -inf
      if (moves) m_ref = m_tile;
#pragma unroll
      for (int i = 0; i < 4; ++i) l4[i] *= alpha;
      // the exponentials (the special-function unit is the busiest pipe here) run while the tensor core is still
      // on the previous tile's P V product
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          t[cc][i] = ex2f(t[cc][i] - m_ref);
          l4[i & 3] += t[cc][i];
        }
      // P V of the previous tile complete: the P tile may be overwritten and O may be corrected
      if (lane == 0) ok = mbar_wait(&bar.p_empty, (it & 1) ^ 1, p.status, 26);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (any_moves && it > 0) {
        tc_fence_after();
        uint32_t o[32];
        tc_ld_32x32b_x32(lane_addr + AT_TM_O + half * 32, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tc_st_32x32b_x32(lane_addr + AT_TM_O + half * 32, o);
        tc_wait_st();
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float* e = &t[cc][g * 8];
          const int c8 = c * 4 + g;  // 16-byte chunk of the row: 8 keys
          uint8_t* dst = p_s + (c8 >> 3) * AT_PANEL + row * 128 + (((c8 & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(bf16x2(e[0], e[1]), bf16x2(e[2], e[3]), bf16x2(e[4], e[5]), bf16x2(e[6], e[7]));
        }
      }
      tc_fence_before();         // O corrections before the P V product that the arrival below releases
      fence_proxy_async_smem();  // P written by the generic proxy -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.p_full);
    }
    // O / l -> bf16 -> out[t, head * dk + :]; this warp stores 32 of the 64 value columns
    if (ok) {
      if (lane == 0) ok = mbar_wait(&bar.o_full, 0, p.status, 27);
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    // Every softmax thread executes the same number of named barriers whatever happened above: a warp whose
    // bounded wait ran out makes up for the ones it skipped, so that the others cannot be left waiting for it.
    while (syncs < iters) { softmax_sync(); ++syncs; }
    const float lmine = (l4[0] + l4[1]) + (l4[2] + l4[3]);
    bar.xch[iters & 1][half][row] = lmine;
    softmax_sync();
    const float inv = 1.0f / (lmine + bar.xch[iters & 1][half ^ 1][row]);
    if (ok) {
      tc_fence_after();
      const int64_t tq = q0 + row;
      uint32_t r[32];
      tc_ld_32x32b_x32(lane_addr + AT_TM_O + half * 32, r);
      tc_wait_ld();
      if (tq < p.T) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + tq * p.ldo + head * AT_DV + half * 32);
#pragma unroll
        for (int g = 0; g < 4; ++g)
          dst[g] = make_uint4(bf16x2(__uint_as_float(r[8 * g]) * inv, __uint_as_float(r[8 * g + 1]) * inv),
                              bf16x2(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv),
                              bf16x2(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv),
                              bf16x2(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace
}  // namespace vx

extern "C" int vx_relpos_attention(const void* q2, const void* k2, const void* v2, int64_t T, int heads, int head_dim,
                                   int64_t kv_len, void* out, int64_t ldo, void* stream) {
  using namespace vx;
  if (T < 0 || heads <= 0) return fail(-1, "bad shape T=%lld heads=%d", (long long)T, heads);
  if (T == 0) return 0;
  if (head_dim != AT_DV) return fail(-1, "head_dim must be %d (got %d)", AT_DV, head_dim);
  if (!q2 || !k2 || !v2 || !out) return fail(-1, "q2, k2, v2 and out must not be NULL");
  if (kv_len <= 0 || kv_len > T) kv_len = T;
  if (static_cast<int64_t>(heads) * T + AT_BM >= (1ll << 31)) return fail(-1, "heads * T must stay below 2^31");
  if (!aligned16(q2) || !aligned16(k2) || !aligned16(v2) || !aligned16(out) || ldo < static_cast<int64_t>(heads) * AT_DV || (ldo * 2) % 16 != 0)
    return fail(-1, "operands must be 16-byte aligned, out rows at least heads * head_dim wide");
  CUtensorMap tq, tk, tv;
  const int64_t rows = static_cast<int64_t>(heads) * T;
  int rc = make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, q2, rows, AT_D, AT_D * 2, 64, AT_BM);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k2, rows, AT_D, AT_D * 2, 64, AT_BN);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, v2, rows, AT_D, AT_D * 2, 64, AT_BN);
  if (rc) return rc;
  AttnParams p{};
  p.T = T; p.kv_len = kv_len; p.heads = heads;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.status = device_status_ptr();
  int dev = 0;
  VX_CUDA_OK(cudaGetDevice(&dev));
  static std::atomic<uint64_t> attr_done{0};
  const bool dev_cached = dev >= 0 && dev < 64;
  if (!dev_cached || !(attr_done.load(std::memory_order_acquire) & (1ull << dev))) {
    VX_CUDA_OK(cudaFuncSetAttribute(relpos_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM));
    if (dev_cached) attr_done.fetch_or(1ull << dev, std::memory_order_release);
  }
  const dim3 grid(static_cast<unsigned>((T + AT_BM - 1) / AT_BM), static_cast<unsigned>(heads));
  relpos_attn_kernel<<<grid, AT_THREADS, AT_SMEM, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

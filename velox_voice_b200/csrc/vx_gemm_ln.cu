// Residual GEMM with the next layer's LayerNorm + MX32 quantizer in its epilogue, d_model = 512.
//
//   x[M,512]   = bf16( alpha * (A[M,K] . B[512,K]^T + bias) + residual )        (stored; may alias residual)
//   codes, sf  = quantize_mx32( LayerNorm(x as stored; gamma, beta, eps) )       (the operand of the next GEMM)
//
// A LayerNorm needs whole rows, and one CTA cannot hold a 128 x 512 fp32 accumulator next to the scale
// factors of a block-scaled MMA in tensor memory.  So a CLUSTER OF TWO CTAs owns each block of 128 rows:
// CTA r computes columns [256 r, 256 r + 256) with 128 x 256 x 64 MXF4 MMAs, and the two exchange the
// per-row partial sums of the LayerNorm statistics through distributed shared memory (st.async with
// mbarrier completion into a table double-buffered per tile, one barrier per lane quadrant).  Per CTA, 18 warps:
//   warp 0      TMA producer: A tiles (128-byte swizzle) + scale-factor atoms into a ring; the CTA's half of B stays
//               resident in shared memory when K <= 512, else it streams through the ring with A;
//   warp 1      owns tensor memory, copies scale factors shared -> tensor memory and issues the MMAs;
//   warps 2..17 epilogue, warp (q, g) = TMEM lane quadrant q, 32-column blocks 2 g and 2 g + 1 of the CTA:
//     pass 1  accumulator -> + bias, alpha, residual (its 32 x 64 block prefetched by TMA into the warp's
//             staging buffer) -> bf16, formed in place and stored by TMA; the bf16 pairs also go back to
//             tensor memory (128 columns next to the accumulator), the accumulator is released to the
//             MMAs of the next tile; per-block (sum, sum of squares) sent to both CTAs;
//     pass 2  after the exchange: mean / rstd, normalise the bf16 values read back from tensor memory,
//             block maximum, E2M1 codes and the UE8M0 scale byte -> global.
// The statistics are summed in exactly the order of the stand-alone half-warp-per-row LayerNorm
// quantizer (rows2_kernel in vx_quant.cu): block j of 16 accumulates its four 8-element pieces in the
// rotated order (c + (j >> 1)) & 3 with separate even / odd sums, and the 16 block sums are combined by
// the xor 8, 4, 2, 1 butterfly tree -- so x, codes and scale factors equal, bit for bit, those of the
// residual GEMM followed by that kernel.
// A second instance (LN2) covers the end of a Conformer block, where norm_final is followed by the next block's
// first LayerNorm: x is not stored, a middle pass forms y = bf16(LayerNorm(x)) (stored instead of x) and its
// statistics, a second exchange follows, and the last pass quantizes LayerNorm(y) -- the bits of
// vx_ln2_quantize_pack behind the residual GEMM.
// Every mbarrier wait is bounded; both CTAs reach the closing cluster barrier on every path.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vx_common.cuh"
#include "vx_ptx.cuh"
#include "vx_quant_math.cuh"
#include "vx_tmap.cuh"

namespace vx {
namespace {

constexpr int LN_BM = 128, LN_BN = 256, LN_D = 512;
constexpr int LN_A_TILE = LN_BM * 128;        // 16 KB: 128 rows x 128 bytes (256 FP4 elements of K)
constexpr int LN_SFA = 2 * 512;               // two SF atoms per stage (UE8M0 per 32)
constexpr int LN_B_TILE = LN_BN * 128;        // 32 KB
constexpr int LN_SFB = 2 * 2 * 512;           // two 128-row tiles x two atoms
constexpr int LN_B_OFF = LN_A_TILE + LN_SFA;  // 17 KB: keeps the B tile 1024-byte aligned
constexpr int LN_A_SLOT = LN_B_OFF;                     // 17 KB: A tile + its scale factors
constexpr int LN_B_SLOT = LN_B_TILE + LN_SFB;           // 34 KB: B tile + its scale factors
constexpr int LN_SLOT = LN_A_SLOT + LN_B_SLOT;          // 51 KB
// Operand arena, two plans (as in vx_gemm.cu):
//   B resident (K <= 512)  [B stage 0 | B stage 1] then three ring slots [A | SFA];
//   streaming              two ring slots [A | SFA | B | SFB].
constexpr int LN_RESIDENT_MAX_STAGES = 2;
constexpr int LN_ARENA = LN_RESIDENT_MAX_STAGES * LN_B_SLOT + 3 * LN_A_SLOT;  // 119 KB
constexpr int LN_MAX_SLOTS = 3;
constexpr int LN_STAGING = 32 * 128;                    // per epilogue warp: 32 rows x 64 bf16 columns, 128-byte swizzle
constexpr int LN_THREADS = 18 * 32;
constexpr uint32_t LN_XCH_BYTES = 2 * 4 * 32 * 16;  // per CTA, tile and lane quadrant: 2 CTAs x 4 warps x 32 lanes x 16 bytes
// tensor-memory columns
constexpr uint32_t LN_TM_ACC = 0, LN_TM_XP = 256, LN_TM_SFA = 384, LN_TM_SFB = 448;

struct LnParams {
  int64_t M, K;
  int m_tiles, k_stages;
  int b_resident;  // 1: the CTA keeps its half of B (all K stages) in shared memory
  const uint8_t* sfa;
  const uint8_t* sfb;
  int64_t sf_kg;
  const float* bias;
  const __nv_bfloat16* residual;
  int64_t ldr;
  __nv_bfloat16* out;
  int64_t ldo;
  float alpha;
  const float* gamma;
  const float* beta;
  const float* gamma2;  // two LayerNorms in a row (LN2 instance): parameters of the second one
  const float* beta2;
  float eps;
  uint8_t* codes;
  int64_t ldc;
  uint8_t* sf_out;
  int* status;
};

struct __align__(1024) LnSmem {
  uint8_t arena[LN_ARENA];
  uint8_t staging[16][LN_STAGING];  // residual block in (TMA), x block out (TMA), per epilogue warp
  float4 part[2][8][LN_BM];  // [tile parity][block pair of the row][row] = (S, Q) of blocks 2 i and 2 i + 1
  float bias[LN_BN], gamma[LN_BN], beta[LN_BN], gamma2[LN_BN], beta2[LN_BN];
  uint64_t full[LN_MAX_SLOTS], empty[LN_MAX_SLOTS];
  uint64_t tmem_full, tmem_empty, b_full;
  uint64_t res_full[16];
  uint64_t xch[2][4];  // [tile parity][lane quadrant]: the rows of a quadrant depend on that quadrant's warps only
  uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address of this CTA -> shared::cluster address of the same variable in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// 16 bytes into (possibly another CTA's) shared memory; the write completes 16 tx bytes on `bar`
// (an mbarrier of the same CTA as `addr`) when it has landed.
__device__ __forceinline__ void st_async_f4(uint32_t addr, float a, float b, float c, float d, uint32_t bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st_all() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t bf16_pair(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// LN2 = false: out = x, codes = quantize(LN(x)).
// LN2 = true (the end of a Conformer block): out = y = bf16(LN(x; gamma, beta)) -- x itself is not stored -- and
// codes = quantize(LN(y as stored; gamma2, beta2)): a second exchange of row statistics and a third pass.
template <bool LN2>
__global__ void __launch_bounds__(LN_THREADS, 1)
bsgemm_residual_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_res, const __grid_constant__ CUtensorMap tmap_out,
                          const LnParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  // (the same offset in both CTAs of the cluster: map_to_cta relies on it)
  LnSmem& sm = *reinterpret_cast<LnSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // column half of this CTA
  const int cluster = static_cast<int>(blockIdx.x >> 1), nclusters = static_cast<int>(gridDim.x >> 1);
  const int my_tiles = cluster < p.m_tiles ? (p.m_tiles - cluster + nclusters - 1) / nclusters : 0;
  const bool resident = p.b_resident != 0;
  const int nslots = resident ? 3 : 2;
  const uint32_t slot_bytes = resident ? LN_A_SLOT : LN_SLOT;
  const uint32_t ring_off = resident ? p.k_stages * LN_B_SLOT : 0;

  // ---- set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < LN_MAX_SLOTS; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.tmem_full, 1);
    mbar_init(&sm.tmem_empty, 16);  // one arrival per epilogue warp
    mbar_init(&sm.b_full, 1);
    for (int w = 0; w < 16; ++w) mbar_init(&sm.res_full[w], 1);
    // exchange barriers: the one arrival is the arming below / after each use; the partial sums arrive as bytes
    for (int b = 0; b < 2; ++b)
      for (int qq = 0; qq < 4; ++qq) {
        mbar_init(&sm.xch[b][qq], 1);
        mbar_expect_tx(&sm.xch[b][qq], LN_XCH_BYTES);
      }
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_res);
    prefetch_tmap(&tmap_out);
  }
  for (int i = threadIdx.x; i < LN_BN; i += blockDim.x) {  // constants of the model
    sm.bias[i] = p.bias ? __ldg(p.bias + rank * LN_BN + i) : 0.0f;
    sm.gamma[i] = __ldg(p.gamma + rank * LN_BN + i);
    sm.beta[i] = __ldg(p.beta + rank * LN_BN + i);
    if constexpr (LN2) {
      sm.gamma2[i] = __ldg(p.gamma2 + rank * LN_BN + i);
      sm.beta2[i] = __ldg(p.beta2 + rank * LN_BN + i);
    }
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  const uint32_t tmem_base = sm.tmem_base;
  const bool producer_thread = warp == 0 && lane == 0 && my_tiles > 0;
  if (!producer_thread) pdl_wait();

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0 && my_tiles > 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      // B tile + scale factors of K stage ks -> dst
      auto load_b = [&](uint8_t* dst, int ks, uint64_t* bar) {
        tma_load_2d(dst, &tmap_b, ks * 128, static_cast<int>(rank) * LN_BN, bar);
#pragma unroll
        for (int rt = 0; rt < 2; ++rt)
          bulk_load(dst + LN_B_TILE + rt * 1024,
                    p.sfb + (static_cast<int64_t>(rank * 2 + rt) * p.sf_kg) * 512 + static_cast<int64_t>(ks) * 1024, 1024, bar);
      };
      if (resident) {  // weights: constants of the model, loaded before the wait for the previous kernel
        mbar_expect_tx(&sm.b_full, p.k_stages * LN_B_SLOT);
        for (int ks = 0; ks < p.k_stages; ++ks) load_b(sm.arena + ks * LN_B_SLOT, ks, &sm.b_full);
      }
      pdl_wait();
      int mb = cluster;
      for (int i = 0; i < my_tiles && ok; ++i, mb += nclusters) {
        const uint8_t* sfa_row = p.sfa + (static_cast<int64_t>(mb) * p.sf_kg) * 512;
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!mbar_wait(&sm.empty[s], ph ^ 1, p.status, 21)) { ok = false; break; }
          uint8_t* dst = sm.arena + ring_off + s * slot_bytes;
          mbar_expect_tx(&sm.full[s], slot_bytes);
          tma_load_2d(dst, &tmap_a, ks * 128, mb * LN_BM, &sm.full[s]);
          bulk_load(dst + LN_A_TILE, sfa_row + static_cast<int64_t>(ks) * LN_SFA, LN_SFA, &sm.full[s]);
          if (!resident) load_b(dst + LN_A_SLOT, ks, &sm.full[s]);
          if (++s == static_cast<uint32_t>(nslots)) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (my_tiles > 0) {
      const bool leader = elect_one();
      uint32_t s = 0, ph = 0, sfsel = 0;
      bool ok = true;
      const uint32_t idesc_base = make_idesc_mxf4(LN_BM, LN_BN, true);
      const uint32_t k128_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t sf_hi = (128u >> 4) | (1u << 14);
      auto desc = [](uint32_t lo, uint32_t hi) -> uint64_t { return (static_cast<uint64_t>(hi) << 32) | (lo & 0x3fffu); };
      const uint32_t arena_lo = smem_u32(sm.arena) >> 4;
      const uint32_t ring_lo = arena_lo + (ring_off >> 4);
      // B scale factors of one stage: shared (b_lo = B tile >> 4) -> 16 TMEM columns at col0
      auto cp_sfb = [&](uint32_t b_lo, uint32_t col0) {
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int rt = 0; rt < 2; ++rt)
            tc_cp_32x128b_warpx4(col0 + a * 8 + rt * 4, desc(b_lo + (LN_B_TILE >> 4) + (rt * 2 + a) * 32, sf_hi));
      };
      if (resident) {
        if (!mbar_wait(&sm.b_full, 0, p.status, 26)) ok = false;
        tc_fence_after();
        if (ok && leader)  // B's scale factors stay in tensor memory for the whole kernel
          for (int ks = 0; ks < p.k_stages; ++ks) cp_sfb(arena_lo + ks * (LN_B_SLOT >> 4), tmem_base + LN_TM_SFB + ks * 16);
        __syncwarp();
      }
      for (int i = 0; i < my_tiles && ok; ++i) {
        // the epilogue has read the previous accumulator out (pass 1 of tile i - 1)
        if (!mbar_wait_spin(&sm.tmem_empty, (i & 1) ^ 1, p.status, 22)) { ok = false; break; }
        tc_fence_after();
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!mbar_wait_spin(&sm.full[s], ph, p.status, 23)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = ring_lo + s * (slot_bytes >> 4);
          const uint32_t b_lo = resident ? arena_lo + ks * (LN_B_SLOT >> 4) : a_lo + (LN_A_SLOT >> 4);
          const uint32_t sfa_buf = tmem_base + LN_TM_SFA + sfsel * 32;
          const uint32_t sfb_buf = tmem_base + LN_TM_SFB + (resident ? ks * 16 : sfsel * 32);
          if (leader) {
#pragma unroll
            for (int a = 0; a < 2; ++a) tc_cp_32x128b_warpx4(sfa_buf + a * 4, desc(a_lo + (LN_A_TILE >> 4) + a * 32, sf_hi));
            if (!resident) cp_sfb(b_lo, sfb_buf);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t atom = j >> 1, sf_id = (j & 1) * 2;
              mma_mxf4<2>(tmem_base + LN_TM_ACC, desc(a_lo + 2 * j, k128_hi), desc(b_lo + 2 * j, k128_hi),
                          idesc_with_sf_id(idesc_base, sf_id, sf_id), sfa_buf + atom * 4, sfb_buf + atom * 8,
                          static_cast<uint32_t>((ks | j) != 0));
            }
            tc_commit(&sm.empty[s]);
            if (ks == p.k_stages - 1) tc_commit(&sm.tmem_full);
          }
          __syncwarp();
          sfsel ^= 1;
          if (++s == static_cast<uint32_t>(nslots)) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // =========================== epilogue ===========================
    const int q = warp & 3, g = (warp - 2) >> 2;  // TMEM lane quadrant; blocks 2 g, 2 g + 1 of this CTA's eight
    const int ew = warp - 2;
    const int row_in = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    // piece (8 columns) handled at step c of a block: (c + rot) & 3, rot = (block >> 1) & 3 = g for both blocks
    int piece[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) piece[c] = (c + g) & 3;
    const uint32_t part0 = smem_u32(&sm.part[0][rank * 4 + g][row_in]);
    const uint32_t bar0 = smem_u32(&sm.xch[0][q]);
    const uint32_t dst_part[2] = {map_to_cta(part0, 0), map_to_cta(part0, 1)};
    const uint32_t dst_bar[2] = {map_to_cta(bar0, 0), map_to_cta(bar0, 1)};
    constexpr uint32_t PART_STRIDE = 8 * LN_BM * 16;
    const int sf_kg_out = 4;  // SF atoms per 128 rows of a 512-wide MX32 operand
    // Staging block of this warp: rows [32 q, +32) x columns [256 rank + 64 g, +64) of the tile as bf16, rows of
    // 128 bytes with the 128-byte swizzle: 16-byte unit u of row r sits at unit u ^ (r & 7).  The residual block
    // lands here by TMA, x is formed in place and leaves by TMA (rows beyond M: zero-filled / clipped).
    uint8_t* const stage_row = sm.staging[ew] + lane * 128;
    const int sw = lane & 7;
    const int tile_col = static_cast<int>(rank) * LN_BN + g * 64;
    const uint64_t A2 = pack_f32x2(p.alpha, p.alpha);
    bool ok = true;
    int mb = cluster;
    if (lane == 0 && my_tiles > 0) {
      mbar_expect_tx(&sm.res_full[ew], LN_STAGING);
      tma_load_2d(sm.staging[ew], &tmap_res, tile_col, mb * LN_BM + q * 32, &sm.res_full[ew]);
    }
    for (int i = 0; i < my_tiles && ok; ++i, mb += nclusters) {
      const int64_t row = static_cast<int64_t>(mb) * LN_BM + row_in;
      const bool row_ok = row < p.M;
      if (!mbar_wait(&sm.tmem_full, i & 1, p.status, 24)) { ok = false; break; }
      tc_fence_after();
      if (!mbar_wait(&sm.res_full[ew], i & 1, p.status, 27)) { ok = false; break; }
      // ---- pass 1: x = bf16(alpha (acc + bias) + residual), block statistics
      float SQ[4];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int k = 2 * g + t;
        uint32_t z[4][8];
#pragma unroll
        for (int c = 0; c < 4; ++c) tc_ld_x8(lane_addr + LN_TM_ACC + k * 32 + piece[c] * 8, z[c]);
        tc_wait_ld();
        if (t == 1) {
          // the warp's part of the accumulator is in registers: free it for the MMAs of the next tile now, not
          // after the arithmetic below (with K = 2048 those MMAs are what the next tile waits for)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.tmem_empty);
        }
        uint32_t xp[16];
        uint64_t S = pack_f32x2(0.0f, 0.0f), Q = S;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float* bs = sm.bias + k * 32 + piece[c] * 8;
          const float4 b0 = *reinterpret_cast<const float4*>(bs), b1 = *reinterpret_cast<const float4*>(bs + 4);
          const uint64_t bb[4] = {pack_f32x2(b0.x, b0.y), pack_f32x2(b0.z, b0.w), pack_f32x2(b1.x, b1.y), pack_f32x2(b1.z, b1.w)};
          uint4* const slot = reinterpret_cast<uint4*>(stage_row + (((4 * t + piece[c]) ^ sw) << 4));
          const uint4 res = *slot;
          const uint32_t rw[4] = {res.x, res.y, res.z, res.w};
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // (packed fp32 pairs: each half rounds exactly like the scalar add / fused multiply-add)
            const uint64_t zz = add_f32x2(pack_f32x2(__uint_as_float(z[c][2 * e]), __uint_as_float(z[c][2 * e + 1])), bb[e]);
            const uint64_t xx = fma_f32x2(A2, zz, pack_f32x2(__uint_as_float(rw[e] << 16), __uint_as_float(rw[e] & 0xffff0000u)));
            float lo, hi;
            unpack_f32x2(xx, lo, hi);
            w[e] = bf16_pair(lo, hi);
            xp[4 * c + e] = w[e];
            const uint64_t v = pack_f32x2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
            S = add_f32x2(S, v);
            Q = fma_f32x2(v, v, Q);
          }
          if constexpr (!LN2) *slot = make_uint4(w[0], w[1], w[2], w[3]);
        }
        tc_st_x16(lane_addr + LN_TM_XP + k * 16, xp);
        float s0, s1, q0, q1;
        unpack_f32x2(S, s0, s1);
        unpack_f32x2(Q, q0, q1);
        SQ[2 * t] = __fadd_rn(s0, s1);
        SQ[2 * t + 1] = __fadd_rn(q0, q1);
      }
      // ---- exchange: this thread's two block sums to both CTAs (first: the peer waits for them).
      // One LayerNorm: table / barrier i & 1, used every second tile.  Two: table 0 for the first, 1 for the
      // second, both used every tile (a peer can only write the next tile's sums of a table after every thread
      // here has sent the sums of the exchange in between, which it does after reading this one).
      auto send = [&](uint32_t b, const float (&sq)[4]) {
#pragma unroll
        for (int d = 0; d < 2; ++d) st_async_f4(dst_part[d] + b * PART_STRIDE, sq[0], sq[1], sq[2], sq[3], dst_bar[d] + b * 32);
      };
      // x (or y) leaves by TMA from the staging block
      auto store_block = [&]() {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmap_out, tile_col, mb * LN_BM + q * 32, sm.staging[ew]);
          tma_store_commit();
        }
      };
      // waits for the sums of exchange b, arms its barrier for the next use, fetches the next residual block when
      // the staging block is free, and reduces the 16 block sums of the row: (rstd, -mean rstd) as packed pairs
      auto finish_stats = [&](uint32_t b, uint32_t parity, bool staging_free, uint64_t& R2, uint64_t& N2) -> bool {
        // (plain polling: at this point every epilogue warp of the quadrant waits, nobody is robbed of issue slots)
        const bool landed = mbar_wait_spin(&sm.xch[b][q], parity, p.status, 25);
        tc_wait_st_all();  // the bf16 copy is in tensor memory before the next pass reads it back
        if (!landed) return false;
        if (g == 0 && lane == 0) mbar_expect_tx(&sm.xch[b][q], LN_XCH_BYTES);  // armed for the next use
        if (staging_free && lane == 0 && i + 1 < my_tiles) {
          // By now the store has read the staging block (waiting for that right behind the store would hold the
          // whole warp for the read): the residual block of the next tile may land in it.
          tma_store_wait_read<0>();
          mbar_expect_tx(&sm.res_full[ew], LN_STAGING);
          tma_load_2d(sm.staging[ew], &tmap_res, tile_col, (mb + nclusters) * LN_BM + q * 32, &sm.res_full[ew]);
        }
        // block sums j and j ^ 8 first (blocks 2 e, 2 e + 1 sit in entry e: entries e and e + 4), then xor 4, 2, 1
        float s[8], qq[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float4 lo = sm.part[b][e][row_in], hi = sm.part[b][e + 4][row_in];
          s[2 * e] = __fadd_rn(lo.x, hi.x); qq[2 * e] = __fadd_rn(lo.y, hi.y);
          s[2 * e + 1] = __fadd_rn(lo.z, hi.z); qq[2 * e + 1] = __fadd_rn(lo.w, hi.w);
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
#pragma unroll
          for (int e = 0; e < o; ++e) {
            s[e] = __fadd_rn(s[e], s[e + o]);
            qq[e] = __fadd_rn(qq[e], qq[e + o]);
          }
        }
        const float mean = __fmul_rn(s[0], 1.0f / 512.0f);
        const float ex2 = __fmul_rn(qq[0], 1.0f / 512.0f);
        const float var = fmaxf(__fmaf_rn(-mean, mean, ex2), 0.0f);
        const float rstd = __frsqrt_rn(__fadd_rn(var, p.eps));
        const float nmr = __fmul_rn(-mean, rstd);
        R2 = pack_f32x2(rstd, rstd);
        N2 = pack_f32x2(nmr, nmr);
        return true;
      };
      uint64_t R2, N2;
      if constexpr (!LN2) {
        send(i & 1, SQ);
        store_block();
        if (!finish_stats(i & 1, (i >> 1) & 1, true, R2, N2)) { ok = false; break; }
      } else {
        send(0, SQ);
        if (!finish_stats(0, i & 1, false, R2, N2)) { ok = false; break; }
        // ---- pass 2 of 3: y = bf16(LN(x)) into the staging block and back into tensor memory, statistics of y
        float SQ2[4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int k = 2 * g + t;
          uint32_t xp[16];
          tc_ld_x16(lane_addr + LN_TM_XP + k * 16, xp);
          tc_wait_ld();
          uint64_t S = pack_f32x2(0.0f, 0.0f), Q = S;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float4* ga = reinterpret_cast<const float4*>(sm.gamma + k * 32 + piece[c] * 8);
            const float4* be = reinterpret_cast<const float4*>(sm.beta + k * 32 + piece[c] * 8);
            uint32_t w[4];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const float4 gv = ga[hh], bv = be[hh];
              const uint32_t w0 = xp[4 * c + 2 * hh], w1 = xp[4 * c + 2 * hh + 1];
              const uint64_t x0 = pack_f32x2(__uint_as_float(w0 << 16), __uint_as_float(w0 & 0xffff0000u));
              const uint64_t x1 = pack_f32x2(__uint_as_float(w1 << 16), __uint_as_float(w1 & 0xffff0000u));
              const uint64_t y0 = fma_f32x2(fma_f32x2(x0, R2, N2), pack_f32x2(gv.x, gv.y), pack_f32x2(bv.x, bv.y));
              const uint64_t y1 = fma_f32x2(fma_f32x2(x1, R2, N2), pack_f32x2(gv.z, gv.w), pack_f32x2(bv.z, bv.w));
              float a0, a1, a2, a3;
              unpack_f32x2(y0, a0, a1);
              unpack_f32x2(y1, a2, a3);
              w[2 * hh] = bf16_pair(a0, a1);
              w[2 * hh + 1] = bf16_pair(a2, a3);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {  // the second LayerNorm reads what is stored
              xp[4 * c + e] = w[e];
              const uint64_t v = pack_f32x2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
              S = add_f32x2(S, v);
              Q = fma_f32x2(v, v, Q);
            }
            *reinterpret_cast<uint4*>(stage_row + (((4 * t + piece[c]) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          tc_st_x16(lane_addr + LN_TM_XP + k * 16, xp);
          float s0, s1, q0, q1;
          unpack_f32x2(S, s0, s1);
          unpack_f32x2(Q, q0, q1);
          SQ2[2 * t] = __fadd_rn(s0, s1);
          SQ2[2 * t + 1] = __fadd_rn(q0, q1);
        }
        send(1, SQ2);
        store_block();
        if (!finish_stats(1, i & 1, true, R2, N2)) { ok = false; break; }
      }
      const float* const gamma_q = LN2 ? sm.gamma2 : sm.gamma;  // parameters of the LayerNorm in front of the quantizer
      const float* const beta_q = LN2 ? sm.beta2 : sm.beta;
      // ---- last pass: normalise, quantize
      uint32_t sf2 = 0;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int k = 2 * g + t;
        uint32_t xp[16];
        tc_ld_x16(lane_addr + LN_TM_XP + k * 16, xp);
        tc_wait_ld();
        uint64_t v[4][4];
        float a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float4* ga = reinterpret_cast<const float4*>(gamma_q + k * 32 + piece[c] * 8);
          const float4* be = reinterpret_cast<const float4*>(beta_q + k * 32 + piece[c] * 8);
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const float4 gv = ga[hh], bv = be[hh];
            const uint32_t w0 = xp[4 * c + 2 * hh], w1 = xp[4 * c + 2 * hh + 1];
            const uint64_t x0 = pack_f32x2(__uint_as_float(w0 << 16), __uint_as_float(w0 & 0xffff0000u));
            const uint64_t x1 = pack_f32x2(__uint_as_float(w1 << 16), __uint_as_float(w1 & 0xffff0000u));
            v[c][2 * hh] = fma_f32x2(fma_f32x2(x0, R2, N2), pack_f32x2(gv.x, gv.y), pack_f32x2(bv.x, bv.y));
            v[c][2 * hh + 1] = fma_f32x2(fma_f32x2(x1, R2, N2), pack_f32x2(gv.z, gv.w), pack_f32x2(bv.z, bv.w));
          }
          a[c] = amax8p(v[c]);
        }
        uint32_t byte;
        float rcp;
        ue8m0_from_amax(fmaxf(max3(a[0], a[1], a[2]), a[3]), byte, rcp);
        uint32_t wd[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) wd[c] = e2m1_pack8p<true, false, true>(v[c], rcp);
        // word of step c belongs to piece (c + g) & 3: rotate the four words back by g
        if (g & 1) { const uint32_t tt = wd[3]; wd[3] = wd[2]; wd[2] = wd[1]; wd[1] = wd[0]; wd[0] = tt; }
        if (g & 2) { uint32_t tt = wd[0]; wd[0] = wd[2]; wd[2] = tt; tt = wd[1]; wd[1] = wd[3]; wd[3] = tt; }
        if (row_ok)
          *reinterpret_cast<uint4*>(p.codes + row * p.ldc + (rank * 8 + k) * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
        sf2 |= byte << (8 * t);
      }
      // scale bytes of blocks j = 8 rank + 2 g, + 1: k-group j >> 2, bytes (j & 3), (j & 3) + 1 of its word;
      // rows beyond M in the last tile read as zero scale factors
      {
        const int64_t off = ((row >> 7) * sf_kg_out + (rank * 2 + (g >> 1))) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
                            (g & 1) * 2;
        *reinterpret_cast<uint16_t*>(p.sf_out + off) = static_cast<uint16_t>(row_ok ? sf2 : 0u);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ---- tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still write into its shared memory
}

// Every condition of the fused kernel that depends on the problem only (not on pointers).
bool ln_shape_ok(int fmt, int64_t N, int64_t K) { return fmt == VX_FMT_MX32 && N == LN_D && K >= 256 && K % 256 == 0; }

}  // namespace
}  // namespace vx

extern "C" {

int vx_bsgemm_residual_ln_supported(int fmt, int64_t N, int64_t K) { return vx::ln_shape_ok(fmt, N, K) ? 1 : 0; }

}  // extern "C"

namespace vx {
namespace {

// Shared by the one- and the two-LayerNorm entry points (gamma2 / beta2 == nullptr: one).
int launch_residual_ln(const vx_gemm_desc* d, const float* gamma, const float* beta, const float* gamma2, const float* beta2,
                       float eps, void* codes, int64_t ldc, void* scales_sf, void* stream, const char* who) {
  if (!d) return fail(-1, "desc must not be NULL");
  if (d->struct_size != static_cast<int32_t>(sizeof(vx_gemm_desc)))
    return fail(-1, "vx_gemm_desc.struct_size=%d, expected %d", d->struct_size, (int)sizeof(vx_gemm_desc));
  if (!ln_shape_ok(d->fmt, d->N, d->K))
    return fail(-1, "%s needs fmt = MX32, N = 512 and K a multiple of 256 (see vx_bsgemm_residual_ln_supported)", who);
  const int64_t M = d->M, K = d->K;
  if (M < 0) return fail(-1, "negative shape");
  if (d->epilogue != VX_EPI_BIAS_RESIDUAL || d->out_dtype != VX_BF16 || d->residual_dtype != VX_BF16 || d->flags != 0)
    return fail(-1, "%s: epilogue BIAS_RESIDUAL with bf16 output and bf16 residual, no flags", who);
  if (M == 0) return 0;
  const int64_t row_bytes = K / 2;
  if (!d->a_codes || !d->b_codes || !d->out || !d->residual || !d->a_scales || !d->b_scales)
    return fail(-1, "a_codes, b_codes, a_scales, b_scales, residual and out must not be NULL");
  if (!aligned16(d->a_codes) || !aligned16(d->b_codes) || d->lda % 16 != 0 || d->ldb % 16 != 0 || d->lda < row_bytes ||
      d->ldb < row_bytes)
    return fail(-1, "operand rows must be 16-byte aligned and at least %lld bytes", (long long)row_bytes);
  if (!aligned16(d->a_scales) || !aligned16(d->b_scales)) return fail(-1, "SF atoms must be 16-byte aligned");
  if (!aligned16(d->out) || !aligned16(d->residual) || d->ldo % 8 != 0 || d->ldr % 8 != 0 || d->ldo < LN_D || d->ldr < LN_D)
    return fail(-1, "out / residual rows must be 16-byte aligned and at least 512 elements");
  if (d->bias && (reinterpret_cast<uintptr_t>(d->bias) & 15)) return fail(-1, "bias must be 16-byte aligned");
  if (!gamma || !beta) return fail(-1, "gamma and beta must not be NULL");
  if ((gamma2 == nullptr) != (beta2 == nullptr)) return fail(-1, "gamma2 and beta2 go together");
  if (!codes || !aligned16(codes) || ldc % 16 != 0 || ldc < LN_D / 2) return fail(-1, "codes rows must be 16-byte aligned, ldc >= 256");
  if (!scales_sf || !aligned16(scales_sf)) return fail(-1, "scales_sf must be 16-byte aligned");
  if ((M + LN_BM - 1) / LN_BM > 0x7fffffff / LN_BM) return fail(-1, "too many rows");

  LnParams p{};
  p.M = M; p.K = K;
  p.m_tiles = static_cast<int>((M + LN_BM - 1) / LN_BM);
  p.k_stages = static_cast<int>(K / 256);
  p.b_resident = p.k_stages <= LN_RESIDENT_MAX_STAGES;
  p.sfa = static_cast<const uint8_t*>(d->a_scales);
  p.sfb = static_cast<const uint8_t*>(d->b_scales);
  p.sf_kg = sf_kgroups(VX_FMT_MX32, K);
  p.bias = d->bias;
  p.residual = static_cast<const __nv_bfloat16*>(d->residual);
  p.ldr = d->ldr;
  p.out = static_cast<__nv_bfloat16*>(d->out);
  p.ldo = d->ldo;
  p.alpha = d->alpha;
  p.gamma = gamma; p.beta = beta; p.gamma2 = gamma2; p.beta2 = beta2; p.eps = eps;
  p.codes = static_cast<uint8_t*>(codes);
  p.ldc = ldc;
  p.sf_out = static_cast<uint8_t*>(scales_sf);
  p.status = device_status_ptr();

  CUtensorMap ta, tb, tr, to;
  int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, d->a_codes, M, row_bytes, d->lda, 128, LN_BM);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, d->b_codes, LN_D, row_bytes, d->ldb, 128, LN_BN);
  if (rc) return rc;
  // residual in / x out: blocks of 32 rows x 64 bf16 columns (128-byte rows), one per epilogue warp and tile
  rc = make_tmap_2d(&tr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d->residual, M, LN_D, d->ldr * 2, 64, 32);
  if (rc) return rc;
  rc = make_tmap_2d(&to, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d->out, M, LN_D, d->ldo * 2, 64, 32);
  if (rc) return rc;

  static int sm_cache[64] = {};
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    if (!sm_cache[dev] && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
      sm_cache[dev] = sms;
    if (sm_cache[dev]) sms = sm_cache[dev];
  }
  int clusters = sms / 2;
  if (clusters > p.m_tiles) clusters = p.m_tiles;
  if (clusters < 1) clusters = 1;
  const size_t smem = sizeof(LnSmem) + 1024;
  const bool two = gamma2 != nullptr;
  auto* kernel = two ? bsgemm_residual_ln_kernel<true> : bsgemm_residual_ln_kernel<false>;
  static bool attr_set[2][64] = {};  // the opt-in belongs to the device (and the kernel instance)
  if (dev >= 0 && dev < 64 && !attr_set[two][dev]) {
    VX_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr_set[two][dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(LN_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  VX_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tr, to, p));
  return 0;
}

}  // namespace
}  // namespace vx

extern "C" {

int vx_bsgemm_residual_ln(const vx_gemm_desc* d, const float* gamma, const float* beta, float eps, void* codes, int64_t ldc,
                          void* scales_sf, void* stream) {
  return vx::launch_residual_ln(d, gamma, beta, nullptr, nullptr, eps, codes, ldc, scales_sf, stream, "vx_bsgemm_residual_ln");
}

int vx_bsgemm_residual_ln2(const vx_gemm_desc* d, const float* gamma1, const float* beta1, const float* gamma2,
                           const float* beta2, float eps, void* codes, int64_t ldc, void* scales_sf, void* stream) {
  if (!gamma2 || !beta2) return vx::fail(-1, "gamma2 and beta2 must not be NULL");
  return vx::launch_residual_ln(d, gamma1, beta1, gamma2, beta2, eps, codes, ldc, scales_sf, stream, "vx_bsgemm_residual_ln2");
}

}  // extern "C"

// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (bulk tensor and plain bulk copies),
// tensor memory (tcgen05.alloc/ld/cp/commit) and the tcgen05.mma forms this library issues.
//
// Every wait on an mbarrier is BOUNDED: after a wall-clock limit the waiter records a
// status word in global memory and returns false, so a lost arrival ends the kernel with
// an error instead of hanging the GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace vx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the thread until the phase
// completes (or the hint, in nanoseconds, runs out) instead of spinning: sixteen epilogue
// warps polling in a tight loop take the issue slots the single MMA-issuing thread needs.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}

// Wall-clock limit of one wait.  Whole kernels here run for well under 100 ms.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// status word layout: 0 = ok; else (code << 24) | (site << 16) | (blockIdx.x & 0xffff)
// Slow path of a wait (kept inline: an out-of-line call was measured slower in most kernels): polls against the
// wall clock (%globaltimer, slow to read) and gives up after `limit_ns`.  `abort` (optional) is a
// flag in shared memory that the first role of a CTA to give up raises: the other roles of that
// CTA then leave their own waits at once instead of running out their own limits one after another.
__device__ __forceinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int* status, int site,
                                               volatile int* abort = nullptr, uint64_t limit_ns = kWaitLimitNs) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3f) == 0) {
      if (abort && *abort) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, (1 << 24) | ((site & 0xff) << 16) | (blockIdx.x & 0xffff));
        if (abort) *abort = 1;
        return false;
      }
    }
  }
}

// Parked wait: each poll may suspend the thread for up to 20 us, so a wait that succeeds
// within 64 polls never reads the clock.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int site,
                                          volatile int* abort = nullptr) {
#pragma unroll 1
  for (uint32_t spins = 0; spins < 64; ++spins)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, status, site, abort);
}

// Same contract, plain polling without the suspend hint: for the MMA-issuing warp and the
// epilogue's polling lane, whose reaction time is on the critical path of every tile.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, int* status, int site,
                                               volatile int* abort = nullptr) {
#pragma unroll 1
  for (uint32_t spins = 0; spins < 100000; ++spins) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return mbar_wait_slow(bar, parity, status, site, abort);
}

// ------------------------------------------------------------------ proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ TMA
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load global -> shared, completion on an mbarrier.  x = innermost coordinate
// (elements of the map's data type; x * element size must be a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// 2-D tiled store shared -> global (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const void* tmap, int x, int y, const void* smem_src) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
          reinterpret_cast<uint64_t>(tmap)),
      "r"(x), "r"(y), "r"(smem_u32(smem_src))
      : "memory");
}
// 3-D tiled store shared -> global (x innermost).
__device__ __forceinline__ void tma_store_3d(const void* tmap, int x, int y, int z, const void* smem_src) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
          reinterpret_cast<uint64_t>(tmap)),
      "r"(x), "r"(y), "r"(z), "r"(smem_u32(smem_src))
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ------------------------------------------------------------------ tensor memory
// Allocate `ncols` (power of two >= 32) TMEM columns; one full warp executes this.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// mbarrier arrival once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// shared -> tensor memory copy of one 32-row x 16-byte block, replicated to the four
// 32-lane quadrants (the layout block-scaled MMAs read scale factors from).
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive columns, one fp32 per (lane, column); thread i gets lane i.
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with the programmatic-serialization attribute may start while its predecessor
// in the stream is still running; it must execute pdl_wait() before it touches anything the
// predecessor reads or writes (the wait returns once the predecessor grid has completed and its
// memory is visible).  pdl_launch_dependents() lets the successor's blocks be scheduled as soon as
// this grid's blocks have all issued it (or exited).  Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ------------------------------------------------------------------ descriptors
// 64-bit shared-memory matrix descriptor, K-major operand stored as rows of 128 bytes with
// the 128-byte swizzle (what a TMA load with SWIZZLE_128B writes): 8-row groups are 1024
// bytes apart (stride byte offset), version 1 (sm_100), layout type 2 (128B swizzle).
__device__ __forceinline__ uint64_t make_desc_k128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                     // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                     // SWIZZLE_128B
  return d;
}
// Descriptor of one 512-byte scale-factor atom (32 rows x 16 bytes, no swizzle).
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // 8 rows x 16 bytes between row groups
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// 32-bit instruction descriptor, block-scaled kinds.  E2M1 x E2M1 (format id 1 for
// kind::mxf4nvf4), both operands K-major, fp32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_mxf4(int M, int N, bool scale_is_e8m0) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         ((scale_is_e8m0 ? 1u : 0u) << 23) | (static_cast<uint32_t>(M >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_with_sf_id(uint32_t idesc, uint32_t a_id,
                                                        uint32_t b_id) {
  return idesc | (b_id << 4) | (a_id << 29);
}
// kind::f8f6f4, E4M3 x E4M3 (format id 0), fp32 accumulate (c_format = 1), K-major.
__host__ __device__ constexpr uint32_t make_idesc_f8(int M, int N) {
  return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ------------------------------------------------------------------ MMA issue (one thread)
// D[tmem] (+)= A[smem] * B[smem]^T with per-block scale factors read from tensor memory.
// VEC = 2: one UE8M0 scale per 32 K-elements; VEC = 4: one scale per 16 K-elements.
template <int VEC>
__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                         uint32_t accumulate) {
  if constexpr (VEC == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

}  // namespace vx

// Filterbank projection of the audio front-end: power spectrum -> mel GEMM -> log -> CMVN, one pass.
//
//   out[t, m] = (log(max(sum_f (re[t,f]^2 + im[t,f]^2) * mel[m, f], 2^-23)) - mean[m]) * istd[m]
//
// Replaces power_mel_log (veloxvoice/kernels/ops/cuda_ops.py:82-135) and its kernel
// (veloxvoice/kernels/csrc/dgx/dgx_power_mel_log.cu:20-79, dgx/block/nv_block_power_mel_log.h:35-190:
// mma.sync m16n8k8 tf32, at most 48 CTAs).  Here the product runs on the 5th-generation tensor cores
// (tcgen05.mma kind::tf32, accumulator in tensor memory) and the kernel is shaped by what bounds it,
// the 2 KB of complex spectrum per frame that have to come out of HBM:
//
//   warps 0..3    epilogue: tcgen05.ld of the fp32 accumulator (one frame per thread), log, CMVN, store;
//   warps 4..11   loaders: read the spectrum with coalesced 8-byte loads (one complex bin per lane, sixteen
//                 rows per stage, the loads of the next stage in flight while the current one is
//                 processed), form re^2 + im^2 and write it straight into the 128-byte-swizzled
//                 K-major tile layout the MMA reads -- the power spectrum never exists in global memory;
//   warp 12       MMA issuer: four K = 8 MMAs per 32-bin stage, tcgen05.commit hands ring slots back and
//                 publishes finished accumulators (two of them, so the epilogue of frame tile i runs under the
//                 loads and MMAs of tile i + 1).
// The filterbank (at most 256 mel rows, zero-padded to a multiple of 16) stays resident in shared memory in
// the same swizzled layout for the whole kernel.  fp32 operands are read by the tensor core as tf32 (the low
// 13 mantissa bits are ignored), which is the reference kernel's precision contract
// (tests/kernels/test_power_mel_log.py:1-16).  Every mbarrier wait is bounded.

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "vx_common.cuh"
#include "vx_ptx.cuh"

namespace vx {
namespace {

constexpr int MEL_BM = 128;             // frames per tile = TMEM lanes
constexpr int MEL_KS = 32;              // spectrum bins per K stage (128 bytes of fp32)
constexpr int MEL_SLOT = MEL_BM * 128;  // bytes of one A stage
constexpr int MEL_RING_MAX = 4;         // A stages in flight: as many (2..4) as fit beside the filterbank
constexpr int MEL_LOADERS = 8;          // loader warps, 16 frames each
constexpr int MEL_THREADS = (4 + MEL_LOADERS + 1) * 32;
constexpr int MEL_MAX_SMEM = 220 * 1024;

struct MelParams {
  const float2* spec;
  int64_t T, F, ld_spec;
  const float* mel;
  int64_t M, ld_mel;
  const float* mean;
  const float* istd;
  float* out;
  int64_t ldo;
  int n_pad, stages, tiles, ring;
  int* status;
};

// byte offset of element (row, k) of a K-major tile of 128-byte rows with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int k) {
  return static_cast<uint32_t>(row) * 128u + ((static_cast<uint32_t>(k >> 2) ^ (static_cast<uint32_t>(row) & 7u)) << 4) +
         (static_cast<uint32_t>(k & 3) << 2);
}

__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N) {
  // fp32 accumulate (c_format 1), A and B tf32 (format 2), both K-major
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

struct MelBarriers {
  uint64_t full[MEL_RING_MAX];
  uint64_t empty[MEL_RING_MAX];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(MEL_THREADS, 1) power_mel_log_kernel(const MelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* const ring = base;                                  // p.ring x 16 KB
  uint8_t* const bres = base + p.ring * MEL_SLOT;              // stages x n_pad x 128 B (n_pad % 8 == 0: 1 KB atoms hold)
  __shared__ MelBarriers bar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* const abortp = &bar.abort_flag;
  const int my_tiles = static_cast<int>(blockIdx.x) < p.tiles ? (p.tiles - static_cast<int>(blockIdx.x) + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t b_stage_bytes = static_cast<uint32_t>(p.n_pad) * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.ring; ++s) {
      mbar_init(&bar.full[s], MEL_LOADERS);
      mbar_init(&bar.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bar.acc_full[a], 1);
      mbar_init(&bar.acc_empty[a], 4);
    }
    bar.abort_flag = 0;
    mbar_fence_init();
  }
  // the filterbank, zero-padded, into its resident swizzled tiles: element (n, k) of stage k / 32
  for (int64_t i = threadIdx.x; i < static_cast<int64_t>(p.stages) * p.n_pad * MEL_KS; i += blockDim.x) {
    const int kk = static_cast<int>(i % MEL_KS);
    const int n = static_cast<int>((i / MEL_KS) % p.n_pad);
    const int ks = static_cast<int>(i / (static_cast<int64_t>(MEL_KS) * p.n_pad));
    const int64_t k = static_cast<int64_t>(ks) * MEL_KS + kk;
    const float v = (n < p.M && k < p.F) ? __ldg(p.mel + n * p.ld_mel + k) : 0.0f;
    *reinterpret_cast<float*>(bres + ks * b_stage_bytes + sw128(n, kk)) = v;
  }
  fence_proxy_async_smem();
  if (warp == 4 + MEL_LOADERS) {
    tmem_alloc(&bar.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar.tmem_base;

  if (warp >= 4 && warp < 4 + MEL_LOADERS) {
    // =========================== loaders ===========================
    // The (tile, stage) items of this CTA form one sequence; the sixteen loads of item n + 1 are in
    // flight while item n is squared and written to its ring slot.
    const int lw = warp - 4;
    const int64_t items = static_cast<int64_t>(my_tiles) * p.stages;
    auto fetch = [&](int64_t n, float2 (&c)[16]) {
      const int64_t tile = static_cast<int64_t>(blockIdx.x) + (n / p.stages) * gridDim.x;
      const int64_t row0 = tile * MEL_BM + lw * 16;
      const int64_t f = (n % p.stages) * MEL_KS + lane;
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const int64_t row = row0 + r;
        c[r] = (n < items && row < p.T && f < p.F) ? __ldg(p.spec + row * p.ld_spec + f) : make_float2(0.0f, 0.0f);
      }
    };
    auto publish = [&](uint32_t s, const float2 (&c)[16]) {
      uint8_t* const slot = ring + s * MEL_SLOT;
#pragma unroll
      for (int r = 0; r < 16; ++r)  // two rounded squares and one rounded add, as spec.real**2 + spec.imag**2
        *reinterpret_cast<float*>(slot + sw128(lw * 16 + r, lane)) = __fadd_rn(__fmul_rn(c[r].x, c[r].x), __fmul_rn(c[r].y, c[r].y));
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.full[s]);
    };
    uint32_t s = 0, ph = 0;
    bool ok = true;
    float2 ca[16], cb[16];
    fetch(0, ca);
    for (int64_t n = 0; n < items && ok; n += 2) {
      fetch(n + 1, cb);
      if (lane == 0) ok = mbar_wait(&bar.empty[s], ph ^ 1, p.status, 11, abortp);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      publish(s, ca);
      if (++s == static_cast<uint32_t>(p.ring)) { s = 0; ph ^= 1; }
      if (n + 1 >= items) break;
      fetch(n + 2, ca);
      if (lane == 0) ok = mbar_wait(&bar.empty[s], ph ^ 1, p.status, 11, abortp);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      publish(s, cb);
      if (++s == static_cast<uint32_t>(p.ring)) { s = 0; ph ^= 1; }
    }
    if (!ok) bar.abort_flag = 1;
  } else if (warp == 4 + MEL_LOADERS) {
    // =========================== MMA issuer ===========================
    if (my_tiles > 0) {
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_tf32(MEL_BM, p.n_pad);
      const uint32_t ring_u32 = smem_u32(ring), b_u32 = smem_u32(bres);
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const uint32_t a = i & 1;
        if (!mbar_wait_spin(&bar.acc_empty[a], ((i >> 1) & 1) ^ 1, p.status, 12, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * 256;
        for (int ks = 0; ks < p.stages; ++ks) {
          if (!mbar_wait_spin(&bar.full[s], ph, p.status, 13, abortp)) { ok = false; break; }
          tc_fence_after();
          if (leader) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              mma_tf32(d_tmem, make_desc_k128(ring_u32 + s * MEL_SLOT + j * 32), make_desc_k128(b_u32 + ks * b_stage_bytes + j * 32), idesc,
                       (ks | j) != 0);
            tc_commit(&bar.empty[s]);
          }
          __syncwarp();
          if (++s == static_cast<uint32_t>(p.ring)) { s = 0; ph ^= 1; }
        }
        if (ok && leader) tc_commit(&bar.acc_full[a]);
        __syncwarp();
      }
      if (!ok && leader) bar.abort_flag = 1;
    }
  } else {
    // =========================== epilogue (warps 0..3 = lane quadrants 0..3) ===========================
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      const uint32_t a = i & 1;
      if (lane == 0) ok = mbar_wait(&bar.acc_full[a], (i >> 1) & 1, p.status, 14, abortp);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const int64_t row = (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(i) * gridDim.x) * MEL_BM + warp * 32 + lane;
      const uint32_t taddr = tmem_base + a * 256 + (static_cast<uint32_t>(warp * 32) << 16);
      for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
        uint32_t r[16];
        tc_ld_32x32b_x16(taddr + c0, r);
        tc_wait_ld();
        if (row < p.T) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c0 + j;
            if (m < p.M) {
              float v = __logf(fmaxf(__uint_as_float(r[j]), 1.1920929e-7f));
              if (p.mean) v = (v - __ldg(p.mean + m)) * __ldg(p.istd + m);
              p.out[row * p.ldo + m] = v;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_empty[a]);
    }
    if (!ok) bar.abort_flag = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4 + MEL_LOADERS) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace
}  // namespace vx

namespace vx {
namespace {
// shared memory the kernel needs for an M x F filterbank with `ring` A stages; 0 when M is too large
size_t mel_smem_bytes(int64_t F, int64_t M, int ring) {
  if (M <= 0 || F <= 0 || M > 256) return 0;
  const size_t n_pad = static_cast<size_t>((M + 15) / 16 * 16), stages = static_cast<size_t>((F + MEL_KS - 1) / MEL_KS);
  return stages * n_pad * 128 + 1024 + static_cast<size_t>(ring) * MEL_SLOT;
}
}  // namespace
}  // namespace vx

extern "C" int vx_power_mel_log_supported(int64_t F, int64_t M) {
  const size_t need = vx::mel_smem_bytes(F, M, 2);
  return need != 0 && need <= static_cast<size_t>(vx::MEL_MAX_SMEM);
}

extern "C" int vx_power_mel_log(const void* spec, int64_t T, int64_t F, int64_t ld_spec, const float* mel, int64_t M,
                                int64_t ld_mel, const float* cmvn_mean, const float* cmvn_istd, float* out, int64_t ldo,
                                void* stream) {
  using namespace vx;
  if (T < 0 || F <= 0 || M <= 0) return fail(-1, "bad shape T=%lld F=%lld M=%lld", (long long)T, (long long)F, (long long)M);
  if (T == 0) return 0;
  if (!spec || !mel || !out) return fail(-1, "spec, mel and out must not be NULL");
  if ((cmvn_mean == nullptr) != (cmvn_istd == nullptr)) return fail(-1, "cmvn_mean and cmvn_istd go together");
  if (reinterpret_cast<uintptr_t>(spec) & 7) return fail(-1, "spec must be 8-byte aligned (complex64)");
  if (ld_spec < F || ld_mel < F || ldo < M) return fail(-1, "row strides are smaller than the rows");
  if (M > 256) return fail(-1, "at most 256 mel rows (M=%lld)", (long long)M);
  MelParams p{};
  p.spec = static_cast<const float2*>(spec);
  p.T = T; p.F = F; p.ld_spec = ld_spec;
  p.mel = mel; p.M = M; p.ld_mel = ld_mel;
  p.mean = cmvn_mean; p.istd = cmvn_istd;
  p.out = out; p.ldo = ldo;
  p.n_pad = static_cast<int>((M + 15) / 16 * 16);
  p.stages = static_cast<int>((F + MEL_KS - 1) / MEL_KS);
  p.tiles = static_cast<int>((T + MEL_BM - 1) / MEL_BM);
  const size_t bank = static_cast<size_t>(p.stages) * p.n_pad * 128 + 1024;
  p.ring = MEL_RING_MAX;
  while (p.ring > 2 && bank + static_cast<size_t>(p.ring) * MEL_SLOT > static_cast<size_t>(MEL_MAX_SMEM)) --p.ring;
  const size_t smem = bank + static_cast<size_t>(p.ring) * MEL_SLOT;
  if (smem > static_cast<size_t>(MEL_MAX_SMEM))
    return fail(-1, "filterbank of %lld x %lld does not fit in shared memory (%zu bytes needed, %d available)", (long long)M,
                (long long)F, smem, MEL_MAX_SMEM);
  p.status = device_status_ptr();
  int dev = 0, sms = 0;
  VX_CUDA_OK(cudaGetDevice(&dev));
  VX_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  static std::atomic<uint64_t> attr_done{0};
  const bool dev_cached = dev >= 0 && dev < 64;
  if (!dev_cached || !(attr_done.load(std::memory_order_acquire) & (1ull << dev))) {
    VX_CUDA_OK(cudaFuncSetAttribute(power_mel_log_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MEL_MAX_SMEM));
    if (dev_cached) attr_done.fetch_or(1ull << dev, std::memory_order_release);
  }
  const int grid = p.tiles < sms ? p.tiles : sms;
  power_mel_log_kernel<<<grid, MEL_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
  VX_CUDA_OK(cudaGetLastError());
  return 0;
}

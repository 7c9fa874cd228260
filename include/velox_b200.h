/*
 * velox_b200 -- C ABI of the B200 (sm_100a) quantized-linear library.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless stated otherwise,
 * `stream` is a cudaStream_t passed as void*.  The caller owns every buffer; the library
 * allocates no device memory.  All entry points enqueue work on `stream` and return without
 * synchronising.
 *
 * Return value: 0 = OK; negative = argument error (nothing was launched, see vx_last_error());
 * positive = CUDA runtime error code.
 *
 * Each entry point names the interface of the reference project (velox-voice) it replaces.
 */
#ifndef VELOX_B200_H_
#define VELOX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VX_ABI_VERSION 6

/* Quantization formats.  values / scale / natural scale layout
 *  ROWSCALE   E2M1, one UE8M0 per row                      u8 [R]
 *  BLK16_A    E2M1, UE8M0 per 16 cols shared by a row pair u8 [K/16][R/2]  (kb-major)
 *  BLK16_B    E2M1, UE8M0 per 16 cols per row              u8 [K/16][R]    (kb-major)
 *  MX32       E2M1, UE8M0 per 32 cols                      u8 [R][K/32]
 *  NV16       E2M1, E4M3 per 16 cols + fp32 tensor scale   u8 [R][K/16], amax f32[1]
 *  FP8_1X128  E4M3 values, fp32 scale per 1x128            f32 [R][K/128]
 * E2M1 codes are packed two per byte, low nibble = even k, nibble = sign<<3 | magnitude.
 */
enum vx_fmt {
  VX_FMT_ROWSCALE = 0,
  VX_FMT_BLK16_A = 1,
  VX_FMT_BLK16_B = 2,
  VX_FMT_MX32 = 3,
  VX_FMT_NV16 = 4,
  VX_FMT_FP8_1X128 = 5
};

enum vx_dtype { VX_F32 = 0, VX_BF16 = 1, VX_FP4 = 2 /* fused re-quantized output */ };

enum vx_epilogue {
  VX_EPI_NONE = 0,      /* out = acc (* scales)                      */
  VX_EPI_BIAS = 1,      /* out = acc + bias[n]                       */
  VX_EPI_BIAS_SWISH = 2,/* out = silu(acc + bias[n])                 */
  VX_EPI_BIAS_GLU = 3,  /* out[:, j] = (acc_a + b_a) * sigmoid(acc_b + b_b), GLU-interleaved weights */
  VX_EPI_BIAS_RESIDUAL = 4, /* out = residual + alpha * (acc + bias[n]) */
  VX_EPI_BIAS_ARGMAX = 5, /* no [M, N] output: per row the first column holding the maximum of
                            bf16(acc + bias[n]); `out` = u64 keys [M], see vx_argmax_ids */
  VX_EPI_BIAS_QKVPACK = 6 /* fused QKV projection written as the attention fold pack (vx_qkv_pack):
                            N = 3 * heads * head_dim, `out` = bf16 [3 * heads, M, 2 * head_dim]
                            (q2 | k2 | v2); the second half of k2 is left for the positional
                            projection, see VX_GEMM_OUT_HEADS */
};

/* Scale factors in the layout the block-scaled tensor-core MMA consumes ("SF atoms"):
 * tiles of 128 rows x 4 consecutive K-blocks, 512 bytes each, byte offset inside a tile
 *   (r % 32) * 16 + ((r / 32) % 4) * 4 + (kb % 4);
 * tiles ordered [ceil(R/128)][kg] with kg = vx_sf_kgroups(fmt, K); unused bytes are zero.
 */
int64_t vx_sf_kgroups(int fmt, int64_t K);
int64_t vx_sf_bytes(int fmt, int64_t R, int64_t K);

/* Quantize + pack the rows of x [M,K] (row stride ldx elements, dtype VX_F32 or VX_BF16).
 * Replaces per_row_col_quantize / triton_quantize_w (veloxvoice/kernels/ops/triton_ops.py:92-129)
 * and mxfp4_block_quantize (triton_ops.py:261-293); MX32 / NV16 / FP8_1X128 extend the same rules.
 *   codes      u8 [M, K/2] (E2M1 formats) or u8 [M, K] (FP8), row stride ldc BYTES
 *   scales     natural layout (table above), may be NULL
 *   scales_sf  SF-atom layout (block E2M1 formats only), may be NULL
 *   amax       NV16 only: f32[1] holding the tensor's max |x| (see vx_amax); read, not written
 * K % 8 == 0 (and the format's block size must divide K); x rows 16-byte aligned.
 */
int vx_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int fmt,
                     void* codes, int64_t ldc, void* scales, void* scales_sf, const float* amax,
                     void* stream);

/* LayerNorm (fp32 statistics, eps, gamma/beta f32[K]) fused in front of vx_quantize_pack:
 * replaces the LayerNorm launch (veloxvoice/kernels/csrc/velox_layernorm.cu:13-58,
 * fused_layernorm in veloxvoice/kernels/ops/cuda_ops.py:204-210) followed by the quantizer
 * launch (veloxvoice/models/wenet/torch_conformer.py:251-262).  K <= 2048.
 *   y      optional [M,K] copy of the normalised rows (y_dtype VX_F32 or VX_BF16, row stride
 *          ldy elements), may be NULL;
 *   codes  may be NULL when y is given: plain LayerNorm, nothing is quantized.
 */
int vx_ln_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                        const float* gamma, const float* beta, float eps, int fmt, void* codes,
                        int64_t ldc, void* scales, void* scales_sf, const float* amax, void* y,
                        int y_dtype, int64_t ldy, void* stream);

/* Two LayerNorms in a row, then the quantizer, in one pass over x:
 *   y = LN(x; gamma1, beta1) stored (may alias x), codes = quantize(LN(y as stored; gamma2, beta2)).
 * This is the end of one Conformer block (norm_final, torch_conformer.py:713) running into the
 * first LayerNorm of the next block (:706) or into after_norm (:745): the reference runs two
 * LayerNorm launches and a quantizer launch.  Same eps for both; y may be NULL (then the second
 * LayerNorm reads the unrounded fp32 result of the first).  Other arguments as above. */
int vx_ln2_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                         const float* gamma1, const float* beta1, const float* gamma2,
                         const float* beta2, float eps, int fmt, void* codes, int64_t ldc,
                         void* scales, void* scales_sf, const float* amax, void* y, int y_dtype,
                         int64_t ldy, void* stream);

/* max |x| over a tensor into amax_out[0] (f32, overwritten).  No reference counterpart
 * (the reference has no per-tensor scale); needed by NV16. */
int vx_amax(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, float* amax_out,
            void* stream);

/* Natural-layout block scales -> SF atoms (weights quantized elsewhere, or scales produced
 * by the reference's quantizers).  fmt in {BLK16_A, BLK16_B, MX32, NV16}. */
int vx_sf_from_natural(int fmt, const void* scales, int64_t R, int64_t K, void* scales_sf,
                       void* stream);

/* Block-scaled GEMM  D[M,N] = epilogue( A[M,K] . B[N,K]^T ).
 * Replaces velox_dgx_mxfp4_gemm / velox_dgx_mxfp4_blkscale_gemm
 * (veloxvoice/kernels/csrc/dgx/dgx_mxfp4_gemm.cu:61-111,135-180; Python wrappers
 * dgx_mxfp4_gemm / dgx_mxfp4_blkscale_gemm in veloxvoice/kernels/ops/cuda_ops.py:626-645,679-702)
 * plus the bias / SiLU / GLU / residual launches that follow them in the model
 * (veloxvoice/models/wenet/torch_conformer.py:265-266,657-658,706,594-633).
 */
typedef struct vx_gemm_desc {
  int32_t struct_size; /* sizeof(vx_gemm_desc) */
  int32_t fmt;         /* vx_fmt of both operands (BLK16_A means A side "A", B side "B") */
  int64_t M, N, K;
  const void* a_codes; /* u8 [M, K/2] or [M, K] (FP8) */
  int64_t lda;         /* bytes per row, multiple of 16 */
  const void* b_codes; /* u8 [N, K/2] or [N, K] */
  int64_t ldb;
  const void* a_scales; /* ROWSCALE: u8 [M]; block E2M1 formats: SF atoms; FP8: f32 [M,K/128] */
  const void* b_scales; /* same for the N side */
  const float* a_amax;  /* NV16: f32[1] tensor amax of A (global scale = amax / 2688) */
  const float* b_amax;
  int32_t epilogue;     /* vx_epilogue */
  int32_t out_dtype;    /* vx_dtype */
  void* out;            /* [M, N'] (N' = N/2 for GLU); FP4: u8 [M, N'/2] */
  int64_t ldo;          /* elements (bytes for FP4 codes) */
  const float* bias;    /* f32 [N] or NULL */
  const void* residual; /* [M, N] or NULL */
  int32_t residual_dtype;
  int32_t out_fmt;      /* FP4 output: MX32 or NV16 */
  int64_t ldr;          /* elements */
  float alpha;          /* BIAS_RESIDUAL */
  int32_t flags;        /* VX_GEMM_* */
  void* out_scales_sf;  /* FP4 output: SF atoms of the output rows */
  void* out_scales;     /* FP4 output: natural layout, may be NULL */
  const float* out_amax;/* FP4 NV16 output: f32[1] static tensor amax */
  int32_t heads;        /* BIAS_QKVPACK / VX_GEMM_OUT_HEADS: number of attention heads */
  int32_t head_dim;     /*   columns per head (multiple of 32) */
  const void* pos_u;    /* BIAS_QKVPACK: bf16 [heads, head_dim] positional biases */
  const void* pos_v;
  float qk_scale;       /* BIAS_QKVPACK: scale applied to q + bias */
  int32_t head_col_off; /* VX_GEMM_OUT_HEADS: first column inside the head row (0 or head_dim) */
  void* lse_partials;   /* BIAS_ARGMAX, FP4 formats: optional f32 pairs [vx_ctc_lse_parts(N)][M], see vx_ctc_finish */
  const float* topk_threshold; /* BIAS_ARGMAX with lse_partials: optional f32 [M]; every bf16-rounded logit >= its row's    */
  void* topk_candidates;       /*   threshold is appended to that row's list: u64 [M][topk_capacity] =                      */
  int32_t* topk_count;         /*   (order-preserving logit bits << 32) | (0xFFFFFFFF - column); i32 [M], zeroed by the caller */
  int32_t topk_capacity;       /*   entries per row; appends beyond it are counted but not stored (see vx_ctc_topk_finish)  */
  int32_t reserved0;
} vx_gemm_desc;

/* VX_EPI_BIAS_GLU expects the rows of B (and the bias) interleaved per tile of vx_glu_tile(fmt)
 * rows: tile/2 rows of the value half followed by the matching tile/2 rows of the gate half.
 * (The reference's bf16 GLU kernel loads both halves' tiles per stage instead,
 * veloxvoice/kernels/csrc/hopper/block/wasp_producer.h:47-72.) */
int vx_glu_tile(int fmt);

#define VX_GEMM_DIRECT_STORE 1 /* bypass the shared-memory staged TMA store */
#define VX_GEMM_STREAM_B 2     /* never keep the B tile resident in shared memory */
#define VX_GEMM_WIDE_TILES 4   /* FP4: force the 128 x 256 single-accumulator tile */
#define VX_GEMM_NARROW_TILES 8 /* FP4: force the 128 x 128 double-accumulator tile (not for GLU) */
#define VX_GEMM_OUT_HEADS 16   /* bf16 output written head-major: `out` = [heads, M, ldo], column n goes to
                                  out[n / head_dim][m][head_col_off + n % head_dim]; N = heads * head_dim.
                                  With head_col_off = head_dim and out = the k2 third of a BIAS_QKVPACK
                                  buffer this is where lp(pos_emb) belongs (torch_conformer.py:472,507) */

int vx_bsgemm(const vx_gemm_desc* desc, void* stream);

/* The residual GEMM that ends a Conformer module together with the LayerNorm + quantizer that opens the
 * next one, in one launch: replaces vx_bsgemm(BIAS_RESIDUAL, bf16) followed by vx_ln_quantize_pack(fmt = MX32)
 * -- in the reference a GEMM, a bias / residual add, a LayerNorm launch and a quantizer launch
 * (veloxvoice/models/wenet/torch_conformer.py:706, 251-262; velox_layernorm.cu:13-58).
 *   desc       as for vx_bsgemm with fmt = MX32, N = 512, K % 256 == 0, epilogue = BIAS_RESIDUAL, bf16 output and
 *              bf16 residual (rows 16-byte aligned; out may alias residual), flags = 0;
 *   out        x = bf16(alpha (A B^T + bias) + residual), stored as by vx_bsgemm;
 *   codes / scales_sf   MX32 codes u8 [M, 256] (row stride ldc bytes) and SF atoms (vx_sf_bytes(MX32, M, 512)) of
 *              LayerNorm(x as stored; gamma, beta, eps) -- the same bits as vx_ln_quantize_pack on x.
 * A cluster of two CTAs owns each block of 128 rows (256 columns each) and exchanges the row statistics
 * through distributed shared memory.  vx_bsgemm_residual_ln_supported: 1 when (fmt, N, K) is covered. */
int vx_bsgemm_residual_ln_supported(int fmt, int64_t N, int64_t K);
int vx_bsgemm_residual_ln(const vx_gemm_desc* desc, const float* gamma, const float* beta, float eps, void* codes,
                          int64_t ldc, void* scales_sf, void* stream);
/* The same launch at the end of a Conformer block, where norm_final is followed by the first LayerNorm of the next
 * block or by after_norm (veloxvoice/models/wenet/torch_conformer.py:713 -> :706 / :745): replaces
 * vx_bsgemm(BIAS_RESIDUAL, bf16) + vx_ln2_quantize_pack(fmt = MX32, y = x).
 *   out        y = bf16(LayerNorm(x; gamma1, beta1)), x = bf16(alpha (A B^T + bias) + residual) as above (x itself is
 *              not stored; out may alias residual);
 *   codes / scales_sf   of LayerNorm(y as stored; gamma2, beta2) -- the same bits as the two calls.
 * Two exchanges of row statistics between the CTAs of a cluster instead of one. */
int vx_bsgemm_residual_ln2(const vx_gemm_desc* desc, const float* gamma1, const float* beta1, const float* gamma2,
                           const float* beta2, float eps, void* codes, int64_t ldc, void* scales_sf, void* stream);

/* Greedy (argmax) head without materialising the logits: what the reference computes as
 * ctc_lo(x).argmax(-1) on [T, vocab] logits (veloxvoice/models/wenet/torch_conformer.py:810-814).
 * vx_bsgemm with VX_EPI_BIAS_ARGMAX clears and fills `out` = u64 [M]: key = (order-preserving
 * bits of the bf16-rounded logit) << 32 | (0xFFFFFFFF - column), maximised over the columns, so
 * equal bf16 logits resolve to the lowest column like torch.argmax.  vx_argmax_ids turns keys
 * into ids i32 [M] and, when max_out != NULL, the winning logits f32 [M]. */
int vx_argmax_ids(const void* keys, int64_t M, int32_t* ids, float* max_out, void* stream);

/* The CTC tail without the logits: log-softmax needs log sum_n exp(z[m, n]) per frame
 * (z - logsumexp(z), veloxvoice/models/wenet/torch_conformer.py:945-949).  With `lse_partials`
 * set, the BIAS_ARGMAX epilogue also keeps, per row and 64-column group, the running maximum and
 * the sum of exp(z - max) of the bf16-rounded logits (8 bytes per row and group instead of 128
 * bytes of logits).  vx_ctc_finish merges them: lse_out[m] = log sum exp, logp_out[m] =
 * log_softmax(z[m])[argmax] = max - lse, next to the ids / winning logits of vx_argmax_ids.
 * ids, max_out, lse_out, logp_out may each be NULL.  vx_ctc_lse_parts(N) = groups to allocate. */
int64_t vx_ctc_lse_parts(int64_t N);
int vx_ctc_finish(const void* keys, const void* lse_partials, int64_t N, int64_t M, int32_t* ids, float* max_out,
                  float* lse_out, float* logp_out, void* stream);

/* Relative-position attention on the folded operands of the attention fold pack (vx_qkv_pack or the
 * fold-pack epilogue of the QKV GEMM): replaces
 *   scaled_dot_product_attention(q2, k2, v2, scale = 1.0)[..., :dk].transpose(1, 2).reshape(T, d)
 * of the encoder's attention (veloxvoice/models/wenet/torch_conformer.py:514-519; the reference's own
 * kernel for its chunked lane is veloxvoice/kernels/csrc/velox_chunk_rel_pos_attn.cu:23-114).
 *   q2, k2, v2: bf16 [heads, T, 2 head_dim] contiguous; the second half of v2 is not read;
 *   out[t, h head_dim + c] = sum_j softmax_j(q2[h, t, :] . k2[h, j, :]) v2[h, j, c], keys j < kv_len
 *   (kv_len <= 0 or > T: all T keys); out bf16 [T, >= heads head_dim], row stride ldo elements.
 * tcgen05 bf16 MMAs with fp32 accumulation, probabilities rounded to bf16 for the second product, like
 * the fused attention kernels torch dispatches to.  head_dim must be 64. */
int vx_relpos_attention(const void* q2, const void* k2, const void* v2, int64_t T, int heads, int head_dim,
                        int64_t kv_len, void* out, int64_t ldo, void* stream);

/* Filterbank projection of the audio front-end in one pass: replaces power_mel_log
 * (veloxvoice/kernels/ops/cuda_ops.py:95-135; kernel veloxvoice/kernels/csrc/dgx/dgx_power_mel_log.cu:20-79,
 * dgx/block/nv_block_power_mel_log.h:35-190) and the formula of reference_power_mel_log (cuda_ops.py:195-202):
 *   out[t, m] = (log(max(sum_f (re[t,f]^2 + im[t,f]^2) * mel[m, f], 2^-23)) - mean[m]) * istd[m]
 * spec: complex64 [T, F] (interleaved re, im as torch.fft.rfft returns it; 8-byte aligned; row stride ld_spec
 * complex elements), mel f32 [M, F] (row stride ld_mel), cmvn_mean / cmvn_istd f32 [M] or both NULL,
 * out f32 [T, M] (row stride ldo).  The product runs on the tensor cores with tf32 operands (the low 13
 * mantissa bits of power and mel are dropped) and fp32 accumulation -- the reference kernel's precision
 * contract (tests/kernels/test_power_mel_log.py:1-16).  Any T >= 0; M <= 256 and the filterbank must fit in
 * shared memory next to two input stages: vx_power_mel_log_supported(F, M) says whether it does (the
 * reference falls back to cuBLAS above M = 80 or below T = 64, cuda_ops.py:110-134). */
int vx_power_mel_log_supported(int64_t F, int64_t M);
int vx_power_mel_log(const void* spec, int64_t T, int64_t F, int64_t ld_spec, const float* mel, int64_t M, int64_t ld_mel,
                     const float* cmvn_mean, const float* cmvn_istd, float* out, int64_t ldo, void* stream);

/* Top-k of the CTC log-probabilities without the logits: what torch.topk(log_softmax(ctc_lo(x)), k) feeds the
 * prefix beam search with (veloxvoice/stream/rescore.py:252-262, veloxvoice/kernels/ops/cuda_ops.py:836-893).
 * Two launches of the CTC GEMM: the first as for vx_ctc_finish (arg-max keys + lse_partials, whose running
 * maxima are the maxima of every 64-column group); vx_ctc_topk_threshold takes the k-th largest group maximum
 * of each row -- at least k logits of the row are >= it and every one of the row's k largest is; the second
 * launch, with topk_threshold / topk_candidates / topk_count set, appends every logit >= the threshold to its
 * row's list; vx_ctc_topk_finish picks the k largest of each list (equal values: lowest column first) and
 * writes ids i32 [M, k] and logp f32 [M, k] = logit - logsumexp.  A row whose list overflowed topk_capacity
 * (many equal bf16 logits) sets overflow[0] (i32, zeroed by the caller) and gets ids -1: the caller falls
 * back to the logits for those rows.  k <= 16, topk_capacity <= 256. */
int vx_ctc_topk_threshold(const void* lse_partials, int64_t N, int64_t M, int k, float* threshold, void* stream);
int vx_ctc_topk_finish(const void* candidates, const int32_t* count, int capacity, const void* lse_partials, int64_t N,
                       int64_t M, int k, int32_t* ids, float* logp, int32_t* overflow, void* stream);

/* Attention fold pack in one pass: replaces velox_qkv_pack
 * (veloxvoice/kernels/csrc/velox_qkv_pack.cu:34-97; Python wrapper qkv_pack in
 * veloxvoice/kernels/ops/cuda_ops.py:554-581), i.e. the torch fold chain of
 * veloxvoice/models/wenet/torch_conformer.py:488-510.
 *   qkv bf16 [T, 3d] (q | k | v per token, row stride ld_qkv elements), p0 bf16 [T, d] (lp(pos_emb)),
 *   pos_u / pos_v bf16 [heads, head_dim], scale f32;
 *   q2 = bf16(bf16(q + u) * scale) | bf16(bf16(q + v) * scale),  k2 = k | p0,  v2 = v | 0,
 *   each bf16 [heads, T, 2 head_dim] contiguous.  d = heads * head_dim, head_dim % 8 == 0. */
int vx_qkv_pack(const void* qkv, int64_t ld_qkv, const void* p0, int64_t ld_p0, const void* pos_u,
                const void* pos_v, float scale, int64_t T, int heads, int head_dim, void* q2, void* k2,
                void* v2, void* stream);

/* Block-scaled FP4 GEMM for callers that cannot allocate device memory.  (No counterpart in
 * the reference: its Python wrappers allocate through torch.)
 *
 * Same product as dgx_mxfp4_blkscale_gemm: out f32 [M,N] (dense, ld = N) from packed codes
 * pack_a u8 [M,K/2], pack_b u8 [N,K/2] (dense) and UE8M0 scales in the reference's layout,
 * scale_a u8 [K/16][M/2], scale_b u8 [K/16][N].  The tensor-core copy of the scales, which
 * the regular route keeps in two caller-provided buffers, lives here in a fixed array inside
 * the library: VX_NOALLOC_SF_MAX_BYTES per operand on every GPU that loads the library, held
 * until the process exits.  Problems whose scale factors do not fit (vx_sf_bytes(fmt, rows, K) >
 * the limit, i.e. roughly rows * K > 32 Mi) are rejected with a negative return code.
 *
 * Meant for hosts that gave all device memory to their own pool at start-up or run on a
 * latency-critical thread: cudaMalloc would fail there or stall every stream.  The call itself
 * never calls cudaMalloc / cudaFree or any allocating routine.
 *
 * The first call on each device looks up the array's device address (one-time set-up); make
 * that first call before starting any stream capture.  All calls on a device share the
 * array and overwrite it: two calls whose GPU work may overlap (different streams, or
 * threads) race on it -- serialise them, e.g. issue them on one stream. */
#define VX_NOALLOC_SF_MAX_BYTES (2 * 1024 * 1024)
int vx_blkscale_gemm_noalloc(const void* pack_a, const void* pack_b, const void* scale_a,
                             const void* scale_b, float* out, int64_t M, int64_t N, int64_t K,
                             void* stream);

/* Phase trace of the GEMM pipeline (the reference has a compile-time %globaltimer trace of its
 * Hopper QKV kernel, veloxvoice/kernels/csrc/hopper/block/wasp_producer.h:20-34).  While a
 * device buffer of 3 * 32 * 8 u64 is registered, CTA 0 of every vx_bsgemm launch stamps the SM
 * cycle counter at [role][tile][event]: role 0 = TMA producer (event k: slot for K stage k
 * acquired), 1 = MMA issuer (0 accumulator free, 1 + k stage k landed, 6 tile committed),
 * 2 = epilogue warp 0 (0 waiting, 1 accumulator ready, 2 TMEM read, 3 / 4 before / after the
 * epilogue math, 5 staged, 6 store issued).  NULL switches it off.  The stamps are compiled in only
 * when the library is built with -DVX_PHASE_TRACE=1; otherwise registering a buffer returns -4. */
int vx_set_trace_buffer(void* device_buffer, int64_t bytes);

/* Tensor-core peak probe: times `iters` back-to-back MMAs (no memory traffic) per SM.
 * kind 0 = FP4 block-scaled (kind::mxf4nvf4), 1 = FP8 (kind::f8f6f4).  Host pointer out. */
int vx_mma_peak_probe(int kind, int n_tile, int iters, float* tflops_out);

/* Self-test of the bounded device-side waits (the reference's waits spin without a limit,
 * veloxvoice/kernels/csrc/dgx/arch/tma/tma_lite.h:82-91): launches one small kernel whose only
 * mbarrier is never arrived at, with a wait limit of `limit_ns` nanoseconds (at most 1e8).  The
 * wait gives up, vx_device_status then reports (1 << 24) | (site << 16) | 0 once, and the GPU
 * context stays usable.  Nothing faults, traps or hangs. */
int vx_wait_selftest(int64_t limit_ns, int site, void* stream);

/* Counters of the tensor-map cache (host pointers, either may be NULL): vx_bsgemm encodes a
 * CUtensorMap per operand / output once per distinct (pointer, extents, pitch, box) and re-uses
 * it afterwards; the reference encodes on every call (dgx_mxfp4_gemm.cu:61-109). */
int vx_tmap_cache_stats(int64_t* hits, int64_t* misses);

/* Device-side status word of the last kernels (0 = OK; nonzero = a bounded wait expired:
 * (code<<24)|(site<<16)|block).  Synchronises the device.  Host pointer out. */
int vx_device_status(int* status_out);

const char* vx_last_error(void);
int vx_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* VELOX_B200_H_ */

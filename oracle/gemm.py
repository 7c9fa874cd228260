"""GEMM, epilogue and LayerNorm references (numpy / torch-CPU).  TEST INFRASTRUCTURE.

Follows, in the reference project:

* GEMM result of the per-row-scaled FP4 path: ``raw = unpack(xq) @ unpack(wq).T`` then
  ``raw * 2**(sa-127)[:, None] * 2**(sb-127)[None, :]``
  (``tests/kernels/test_dgx_mxfp4_gemm.py:35-61``).
* every other format: dequantize, then an fp32 matmul (the acceptance rule of the path).
* bias add ``veloxvoice/models/wenet/torch_conformer.py:265-266``; FFN ``w2(silu(w1 x))``
  ``:657-658``; half-step residual ``x + 0.5 * ff(...)`` ``:706,712``; GLU ``a * sigmoid(b)``
  with ``b`` the second half of the channels ``:633`` and
  ``veloxvoice/kernels/csrc/hopper/block/pwlin_glu_block_1p2c.h:77-85``.
* LayerNorm ``veloxvoice/kernels/csrc/velox_layernorm.cu:52-57``.
"""

from __future__ import annotations

import numpy as np
import torch

from . import formats as F

F32 = np.float32


def matmul_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """a [M,K] @ b[N,K].T in fp32 on the host cores."""
    ta = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    tb = torch.from_numpy(np.ascontiguousarray(b, dtype=np.float32))
    return (ta @ tb.T).numpy()


def gemm_rowscale_ref(xq, wq, sa, sb) -> np.ndarray:
    """``torch_matmul_ref`` of the reference's FP4 GEMM test (unit-scale dot, scales after)."""
    raw = matmul_f32(F.e2m1_decode(F.unpack_codes(xq)), F.e2m1_decode(F.unpack_codes(wq)))
    return raw * F.ue8m0_decode(sa)[:, None] * F.ue8m0_decode(sb)[None, :]


def gemm_ref(fmt: int, aq, asc, bq, bsc, ga=None, gb=None) -> np.ndarray:
    """Dequantize-then-fp32-matmul reference for any format."""
    if fmt == F.FMT_ROWSCALE:
        return gemm_rowscale_ref(aq, bq, asc, bsc)
    fb = F.FMT_BLK16_B if fmt == F.FMT_BLK16_A else fmt
    return matmul_f32(F.dequantize(aq, asc, fmt, ga), F.dequantize(bq, bsc, fb, gb))


def gemm_kernel_order(fmt: int, aq, asc, bq, bsc, ga=None, gb=None) -> np.ndarray:
    """The block-scaled product evaluated the way the tensor-core kernel groups it, with every
    group's dot product taken exactly (fp64) and rounded once -- an idealised tensor core:

    * NV16: ``fp32(sum_k (a_code sfa)(b_code sfb)) * fp32(ga * gb)`` (the hardware applies the E4M3
      block scales inside the MMA; the two per-tensor scales multiply the accumulator);
    * FP8 1x128: per 128-wide K block ``p = fp32(sum_k a8 b8)``, then ``acc = fma(p, fp32(sa sb), acc)``
      block after block (the kernel promotes each block's accumulator in fp32 registers);
    * the power-of-two-scaled formats: identical to :func:`gemm_ref` (every operation is exact).

    :func:`gemm_ref` -- dequantize every element to fp32, then an fp32 matmul in the BLAS
    library's summation order -- stays the acceptance reference; this variant separates what two
    correct implementations differ by (rounding of the dequantized elements, summation order)
    from what the kernel itself adds."""
    if fmt == F.FMT_NV16:
        a = F.e2m1_decode(F.unpack_codes(aq)).astype(np.float64) * np.repeat(F.e4m3_decode(asc), 16, axis=1).astype(np.float64)
        b = F.e2m1_decode(F.unpack_codes(bq)).astype(np.float64) * np.repeat(F.e4m3_decode(bsc), 16, axis=1).astype(np.float64)
        acc = (a @ b.T).astype(np.float32)
        return (acc * (F32(ga) * F32(gb))).astype(np.float32)
    if fmt == F.FMT_FP8_1X128:
        a = F.e4m3_decode(aq).astype(np.float64)
        b = F.e4m3_decode(bq).astype(np.float64)
        M, K = a.shape
        acc = np.zeros((M, b.shape[0]), dtype=np.float32)
        for kb in range(K // 128):
            part = (a[:, 128 * kb: 128 * kb + 128] @ b[:, 128 * kb: 128 * kb + 128].T).astype(np.float32)
            sc = (asc[:, kb].astype(np.float32)[:, None] * bsc[:, kb].astype(np.float32)[None, :]).astype(np.float32)
            acc = fma32(part, sc, acc)
        return acc
    return gemm_ref(fmt, aq, asc, bq, bsc, ga, gb)


def silu(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32)
    return (x / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)


EPI_NONE, EPI_BIAS, EPI_BIAS_SWISH, EPI_BIAS_GLU, EPI_BIAS_RESIDUAL = range(5)


def epilogue_ref(acc: np.ndarray, epi: int, bias=None, residual=None, alpha: float = 1.0) -> np.ndarray:
    """fp32 epilogue on the logical (un-interleaved) accumulator [M, N]."""
    z = acc.astype(np.float32)
    if epi != EPI_NONE and bias is not None:
        z = z + np.asarray(bias, dtype=np.float32)[None, :]
    if epi == EPI_BIAS_SWISH:
        z = silu(z)
    elif epi == EPI_BIAS_GLU:
        h = z.shape[1] // 2
        z = z[:, :h] * sigmoid(z[:, h:])
    elif epi == EPI_BIAS_RESIDUAL:
        z = np.asarray(residual, dtype=np.float32) + F32(alpha) * z
    return z.astype(np.float32)


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round fp32 -> bf16 (RN-even) and return as fp32."""
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).bfloat16().float().numpy()


def glu_interleave_rows(n_out: int, tile: int = 128) -> np.ndarray:
    """Row order of GLU weights inside the GEMM: every `tile` rows hold tile/2 rows of the
    value half followed by the matching tile/2 rows of the gate half."""
    h = n_out // 2
    half = tile // 2
    idx = []
    for t in range(0, h, half):
        idx.extend(range(t, min(t + half, h)))
        idx.extend(range(h + t, min(h + t + half, n_out)))
    return np.asarray(idx, dtype=np.int64)


def fma32(a, b, c) -> np.ndarray:
    """Correctly rounded fp32 fused multiply-add ``a * b + c`` (one rounding), elementwise.

    The product of two fp32 numbers is exact in fp64; the sum with ``c`` is formed in fp64, its
    rounding error recovered exactly (two-sum), and the fp64 result pushed to the neighbour with an
    odd last bit when it was inexact (round to odd).  Rounding that to fp32 then equals a single
    rounding of the exact value (fp64 carries more than two extra bits).
    """
    a = np.asarray(a, dtype=np.float32).astype(np.float64)
    b = np.asarray(b, dtype=np.float32).astype(np.float64)
    c = np.asarray(c, dtype=np.float32).astype(np.float64)
    p = a * b
    s = p + c
    bb = s - p
    err = (p - (s - bb)) + (c - bb)
    s, err = np.broadcast_arrays(s, err)
    bits = s.view(np.int64) if s.flags["C_CONTIGUOUS"] else np.ascontiguousarray(s).view(np.int64)
    inexact = (err != 0) & np.isfinite(s)
    even = (bits & 1) == 0
    toward = np.where(err > 0, np.inf, -np.inf)
    s_odd = np.where(inexact & even, np.nextafter(s, toward), s)
    return s_odd.astype(np.float32)


def rsqrt32(x) -> np.ndarray:
    """Correctly rounded fp32 ``1 / sqrt(x)`` (extended precision, then one rounding to fp32)."""
    x = np.asarray(x, dtype=np.float32).astype(np.longdouble)
    return (np.longdouble(1.0) / np.sqrt(x)).astype(np.float32)


def ln_half_rows(K: int, bf16_input: bool, fmt=None) -> bool:
    """Which of the library's two LayerNorm summation orders a call uses: bf16 rows of exactly 512
    elements that are quantized to an SF-atom FP4 format or FP8 (or not quantized at all) go through
    the half-warp-per-row kernel (``rows2_kernel`` in ``csrc/vx_quant.cu``); everything else through
    the warp-per-row kernels."""
    return bool(bf16_input) and K == 512 and fmt in (None, F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128)


def layernorm_ref(x, gamma, beta, eps: float = 1e-5, half_rows: bool = False) -> np.ndarray:
    """Row LayerNorm with the fused CUDA kernels' exact fp32 operation order.

    Formula of ``velox_layernorm.cu:52-57`` (``var = E[x^2] - mean^2`` clamped at 0), evaluated
    with fused multiply-adds in this library's order.  Warp-per-row kernels (``half_rows=False``):
    lane ``l`` of 32 owns, chunk by chunk of 256 elements, the eight consecutive elements
    ``[256 c + 8 l, +8)`` and keeps separate sums for its even and its odd elements (``S += v``,
    ``Q = fma(v, v, Q)``); the two are added, lanes are combined by a butterfly (xor 16, 8, 4, 2, 1).
    Half-warp-per-row kernel (``half_rows=True``, K = 512, see ``ln_half_rows``): lane ``j`` of 16 owns
    elements ``[32 j, +32)`` as four pieces of eight, accumulated in the rotated order it reads them
    (piece ``(c + (j >> 1)) & 3`` at step ``c``), butterfly xor 8, 4, 2, 1.  Then for both:
    ``mean = s / K``, ``ex2 = q / K``, ``var = max(fma(-mean, mean, ex2), 0)``,
    ``rstd = 1 / sqrt(var + eps)`` correctly rounded in one step,
    ``y = fma(fma(x, rstd, -mean * rstd), gamma, beta)``.
    """
    x = F._f32(x)
    M, K = x.shape
    if half_rows:
        assert K == 512
        xl = x.reshape(M, 16, 4, 4, 2)  # [row, lane, piece, pair, even/odd]
        lanes = np.arange(16)
        s = np.zeros((M, 16, 2), dtype=np.float32)
        sq = np.zeros((M, 16, 2), dtype=np.float32)
        for c in range(4):
            piece = (c + (lanes >> 1)) & 3
            for j in range(4):
                v = xl[:, lanes, piece, j, :]
                s = (s + v).astype(np.float32)
                sq = fma32(v, v, sq)
        rounds = (8, 4, 2, 1)
    else:
        ch = -(-K // 256)
        xp = np.zeros((M, ch * 256), dtype=np.float32)
        xp[:, :K] = x
        xl = xp.reshape(M, ch, 32, 4, 2)  # [row, chunk, lane, pair, even/odd]
        lanes = np.arange(32)
        s = np.zeros((M, 32, 2), dtype=np.float32)
        sq = np.zeros((M, 32, 2), dtype=np.float32)
        for c in range(ch):
            for j in range(4):
                v = xl[:, c, :, j, :]
                s = (s + v).astype(np.float32)
                sq = fma32(v, v, sq)
        rounds = (16, 8, 4, 2, 1)
    s = (s[:, :, 0] + s[:, :, 1]).astype(np.float32)
    sq = (sq[:, :, 0] + sq[:, :, 1]).astype(np.float32)
    for o in rounds:
        s = (s + s[:, lanes ^ o]).astype(np.float32)
        sq = (sq + sq[:, lanes ^ o]).astype(np.float32)
    kf = F32(K)
    mean = (s[:, 0] / kf).astype(np.float32)
    ex2 = (sq[:, 0] / kf).astype(np.float32)
    var = np.maximum(fma32(-mean, mean, ex2), F32(0))
    rstd = rsqrt32((var + F32(eps)).astype(np.float32))
    nmr = ((-mean) * rstd).astype(np.float32)
    g = np.asarray(gamma, dtype=np.float32)[None, :]
    b = np.asarray(beta, dtype=np.float32)[None, :]
    t = fma32(x, rstd[:, None], nmr[:, None])
    return fma32(t, g, b)


def qkv_pack_ref(qkv, p0, pos_u, pos_v, scale: float, heads: int):
    """The attention fold chain behind the fused QKV projection, in bf16 like the model runs it.

    ``veloxvoice/models/wenet/torch_conformer.py:488-510`` (torch ops) and its single-pass
    kernel ``veloxvoice/kernels/csrc/velox_qkv_pack.cu:34-97``:

        q2 = cat([q + pos_u, q + pos_v], -1) * scale     k2 = cat([k, p0], -1)     v2 = cat([v, 0], -1)

    with q | k | v the thirds of ``qkv`` [T, 3d] split into ``heads`` heads; every elementwise
    result is rounded to bf16 (the sum, then the product).  Inputs are arrays of bf16-valued
    numbers; returns three float32 arrays [heads, T, 2 dk] of bf16-valued numbers.
    """
    qkv = np.asarray(qkv, dtype=np.float32)
    T, d3 = qkv.shape
    d = d3 // 3
    dk = d // heads
    u = np.asarray(pos_u, dtype=np.float32).reshape(heads, 1, dk)
    v = np.asarray(pos_v, dtype=np.float32).reshape(heads, 1, dk)
    split = lambda a: a.reshape(T, heads, dk).transpose(1, 0, 2)  # [h, T, dk]
    q, k, vv = split(qkv[:, :d]), split(qkv[:, d:2 * d]), split(qkv[:, 2 * d:])
    s = F32(scale)
    qa = to_bf16((to_bf16(q + u) * s).astype(np.float32))
    qb = to_bf16((to_bf16(q + v) * s).astype(np.float32))
    q2 = np.concatenate([qa, qb], axis=-1)
    k2 = np.concatenate([k, split(np.asarray(p0, dtype=np.float32))], axis=-1)
    v2 = np.concatenate([vv, np.zeros_like(vv)], axis=-1)
    return q2, k2, v2

"""Quantize / pack / dequantize rules of the quantized-linear path, restated in numpy.

TEST INFRASTRUCTURE: the product never imports this file.

Reference rules followed (paths inside the reference project):

* E2M1 encode: six strict ``>`` thresholds 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, so the largest
  magnitude code emitted is 6 (= 4.0) and ties go down; sign bit = ``q < 0`` on the
  normalised value (``veloxvoice/kernels/ops/triton_ops.py:58-67,145-156``;
  ``veloxvoice/models/wenet/nvfp4_linear.py:22-36``).
* pack: low nibble = even k, high nibble = odd k (``triton_ops.py:82-84``;
  ``nvfp4_linear.py:39-40``).
* UE8M0 scale: ``s = max(amax / 6, 1e-6)``, ``e = ceil(log2 s)``, byte = clamp(e + 127, 0, 255),
  values normalised by exactly ``2**e`` (``triton_ops.py:44-50,86-89,228-239,254-258``).
* decode: ``+-LUT[c & 7] * 2**(byte - 127)``, LUT = [0, .5, 1, 1.5, 2, 3, 4, 6]
  (``veloxvoice/kernels/ops/cuda_ops.py:710-723``; ``triton_ops.py:296-309``).

Formats (``FMT_*`` values are shared with ``include/velox_b200.h``):

=========== ===================================================== =========================
name        values / scale                                        natural scale layout
=========== ===================================================== =========================
rowscale    E2M1, one UE8M0 per row (whole K)                     u8 [M]
blk16       E2M1, UE8M0 per 16 columns; "A": shared by a row pair u8 [K/16][M/2] or [K/16][M]
mx32        E2M1, UE8M0 per 32 columns                            u8 [M, K/32]
nv16        E2M1, E4M3 per 16 columns, fp32 per-tensor global     u8 [M, K/16] + f32
fp8_1x128   E4M3 values, fp32 scale per 1x128                     f32 [M, K/128]
=========== ===================================================== =========================

``mx32``, ``nv16`` and ``fp8_1x128`` have no counterpart in the reference (parity unpinned
there); they reuse the E2M1 rule above, and ``mx32`` reuses the UE8M0 rule above.
"""

from __future__ import annotations

import numpy as np

FMT_ROWSCALE = 0
FMT_BLK16_A = 1
FMT_BLK16_B = 2
FMT_MX32 = 3
FMT_NV16 = 4
FMT_FP8_1X128 = 5

FMT_NAMES = {
    "rowscale": FMT_ROWSCALE,
    "blk16_a": FMT_BLK16_A,
    "blk16_b": FMT_BLK16_B,
    "mx32": FMT_MX32,
    "nv16": FMT_NV16,
    "fp8_1x128": FMT_FP8_1X128,
}

E2M1_LUT = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5)

F32 = np.float32


def _f32(x) -> np.ndarray:
    """bf16/fp16/fp32 torch tensor or array -> contiguous float32 ndarray (exact)."""
    if hasattr(x, "detach"):
        x = x.detach().float().cpu().numpy()
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


# --------------------------------------------------------------------------- E2M1


def e2m1_encode(q: np.ndarray) -> np.ndarray:
    """fp32 normalised values -> u8 codes (sign<<3 | mag3). ``triton_ops.py:145-156``."""
    ax = np.abs(q)
    c = np.zeros(q.shape, dtype=np.uint8)
    for t in _THRESHOLDS:
        c += ax > F32(t)
    return c | ((q < 0).astype(np.uint8) << 3)


def e2m1_decode(codes: np.ndarray) -> np.ndarray:
    mag = E2M1_LUT[codes & 7]
    return np.where((codes & 8) > 0, -mag, mag).astype(np.float32)


def pack_codes(codes: np.ndarray) -> np.ndarray:
    """codes u8 [R, K] -> bytes u8 [R, K/2]; low nibble = even k (``nvfp4_linear.py:39-40``)."""
    return ((codes[:, 0::2] & 0xF) | ((codes[:, 1::2] & 0xF) << 4)).astype(np.uint8)


def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """bytes u8 [R, K/2] -> codes u8 [R, K] (``nvfp4_linear.py:103-107``)."""
    lo = packed & 0xF
    hi = packed >> 4
    return np.stack([lo, hi], axis=-1).reshape(packed.shape[0], packed.shape[1] * 2)


# --------------------------------------------------------------------------- UE8M0


def ceil_log2_f32(s: np.ndarray) -> np.ndarray:
    """Exact ceil(log2(s)) for positive normal float32 ``s`` (bit inspection, no libm)."""
    bits = np.ascontiguousarray(s, dtype=np.float32).view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int32) - 127
    man = bits & 0x7FFFFF
    return exp + (man != 0).astype(np.int32)


def ue8m0_from_amax(amax: np.ndarray):
    """amax (fp32) -> (exponent e as int32, scale byte u8). ``triton_ops.py:44-47,86-89``."""
    s = np.maximum(amax.astype(np.float32) / F32(6.0), F32(1e-6)).astype(np.float32)
    e = ceil_log2_f32(s)
    byte = np.clip(e + 127, 0, 255).astype(np.uint8)
    return e, byte


def ue8m0_decode(byte: np.ndarray) -> np.ndarray:
    """u8 -> 2**(byte-127) as float32 (``nvfp4_linear.py:52-53``). byte 0 -> 2**-127 (subnormal)."""
    return np.ldexp(F32(1.0), byte.astype(np.int32) - 127).astype(np.float32)


def _exp2_i(e: np.ndarray) -> np.ndarray:
    return np.ldexp(F32(1.0), e.astype(np.int32)).astype(np.float32)


# --------------------------------------------------------------------------- E4M3 (fn)


def e4m3_encode(v: np.ndarray) -> np.ndarray:
    """float -> E4M3 (fn) byte, round-to-nearest-even, saturating to +-448; NaN -> 0x7F."""
    v = np.asarray(v, dtype=np.float64)
    sign = (np.signbit(v)).astype(np.uint8) << 7
    a = np.abs(v)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, a)
    a = np.minimum(a, 448.0)
    _, ex = np.frexp(np.where(a > 0, a, 1.0))  # a = m * 2**ex, m in [0.5, 1)
    E = np.maximum(ex - 1, -6)  # unbiased exponent, clamped at the subnormal exponent
    quantum = np.ldexp(1.0, E - 3)
    r = np.rint(a / quantum) * quantum  # np.rint = round-half-to-even
    r = np.minimum(r, 448.0)
    _, ex2 = np.frexp(np.where(r > 0, r, 1.0))
    E2 = ex2 - 1
    normal = r >= 2.0**-6
    mant_n = np.rint(r / np.ldexp(1.0, E2 - 3)).astype(np.int64) - 8
    bits_n = ((E2 + 7) << 3) | mant_n
    bits_s = np.rint(r / 2.0**-9).astype(np.int64)
    bits = np.where(normal, bits_n, bits_s).astype(np.uint8)
    out = bits | sign
    return np.where(nan, np.uint8(0x7F), out).astype(np.uint8)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    s = np.where((b & 0x80) > 0, -1.0, 1.0)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 7).astype(np.float64)
    val = np.where(e == 0, m * 2.0**-9, (1.0 + m / 8.0) * np.ldexp(1.0, e - 7))
    val = np.where((b & 0x7F) == 0x7F, np.nan, val)
    return (s * val).astype(np.float32)


# --------------------------------------------------------------------------- quantizers


def quantize_rowscale(x):
    """``per_row_col_quantize`` (``triton_ops.py:8-124``): u8 [M,K/2], u8 [M]."""
    x = _f32(x)
    M, K = x.shape
    assert K % 2 == 0
    amax = np.abs(x).max(axis=1) if K else np.zeros(M, np.float32)
    e, byte = ue8m0_from_amax(amax)
    q = x / _exp2_i(e)[:, None]
    return pack_codes(e2m1_encode(q)), byte


def quantize_blk16(x, mode: str = "A"):
    """``mxfp4_block_quantize`` (``triton_ops.py:169-293``): u8 [R,K/2], u8 [K/16][R/RP] kb-major."""
    x = _f32(x)
    R, K = x.shape
    assert K % 16 == 0
    rp = 2 if mode == "A" else 1
    assert R % rp == 0
    blk = np.abs(x).reshape(R // rp, rp, K // 16, 16).max(axis=(1, 3))  # [R/rp, K/16]
    e, byte = ue8m0_from_amax(blk)
    scale = np.repeat(np.repeat(_exp2_i(e), rp, axis=0), 16, axis=1)  # [R, K]
    q = x / scale
    return pack_codes(e2m1_encode(q)), np.ascontiguousarray(byte.T)


def quantize_mx32(x):
    """E2M1 + UE8M0 per 32 columns (no reference code; rules as above): u8 [M,K/2], u8 [M,K/32]."""
    x = _f32(x)
    M, K = x.shape
    assert K % 32 == 0
    blk = np.abs(x).reshape(M, K // 32, 32).max(axis=2)
    e, byte = ue8m0_from_amax(blk)
    q = x / np.repeat(_exp2_i(e), 32, axis=1)
    return pack_codes(e2m1_encode(q)), byte


def nv16_global_scale(amax_t) -> np.float32:
    """fp32 per-tensor scale g = amax / (6 * 448); 1.0 for an all-zero tensor."""
    amax_t = F32(amax_t)
    if amax_t == 0:
        return F32(1.0)
    return F32(amax_t / F32(2688.0))


def quantize_nv16(x, amax_t=None):
    """E2M1 + E4M3 scale per 16 columns + fp32 global scale (no reference code).

    ``g = amax_t / 2688``; block byte = E4M3-RN-even-sat(blockamax / (6 g));
    ``q = x * fp32(1 / fp32(g * dec(byte)))``, every operation a correctly rounded fp32 one;
    a block whose byte decodes to 0 gets codes 0.
    Returns (u8 [M,K/2], u8 [M,K/16], g).
    """
    x = _f32(x)
    M, K = x.shape
    assert K % 16 == 0
    if amax_t is None:
        amax_t = np.abs(x).max() if x.size else F32(0)
    g = nv16_global_scale(amax_t)
    blk = np.abs(x).reshape(M, K // 16, 16).max(axis=2)
    d6 = F32(F32(6.0) * g)
    t = (blk / d6).astype(np.float32)
    byte = e4m3_encode(t)
    dec = e4m3_decode(byte)
    d = (g * dec).astype(np.float32)
    d_full = np.repeat(d, 16, axis=1)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        rd = np.where(d_full > 0, F32(1.0) / d_full, F32(0)).astype(np.float32)
        q = (x * rd).astype(np.float32)
    return pack_codes(e2m1_encode(q)), byte, g


def quantize_fp8_1x128(x):
    """E4M3 values + fp32 scale per 1x128 (no reference code): u8 [M,K], f32 [M,K/128].

    ``scale = blockamax / 448`` (1.0 for a zero block); ``q = x * fp32(1 / scale)``, each
    operation a correctly rounded fp32 one; value = E4M3 RN-even saturating.
    """
    x = _f32(x)
    M, K = x.shape
    assert K % 128 == 0
    blk = np.abs(x).reshape(M, K // 128, 128).max(axis=2)
    scale = (blk / F32(448.0)).astype(np.float32)
    scale = np.where(blk == 0, F32(1.0), scale).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        rs = (F32(1.0) / scale).astype(np.float32)
        q = (x * np.repeat(rs, 128, axis=1)).astype(np.float32)
    return e4m3_encode(q), scale


# --------------------------------------------------------------------------- dequantizers


def dequant_rowscale(packed, scale_u8):
    """``_dequantize_to_bf16`` without the bf16 cast (``cuda_ops.py:710-723``)."""
    return e2m1_decode(unpack_codes(packed)) * ue8m0_decode(scale_u8)[:, None]


def dequant_blk16(packed, scale_kb, mode: str = "A"):
    """``mxfp4_dequant`` (``triton_ops.py:296-309``)."""
    sv = ue8m0_decode(scale_kb)  # [K/16, R2]
    if mode == "A":
        sv = np.repeat(sv, 2, axis=1)
    return e2m1_decode(unpack_codes(packed)) * np.repeat(sv.T, 16, axis=1)


def dequant_mx32(packed, scale_u8):
    return e2m1_decode(unpack_codes(packed)) * np.repeat(ue8m0_decode(scale_u8), 32, axis=1)


def dequant_nv16(packed, scale_e4m3, g):
    return e2m1_decode(unpack_codes(packed)) * np.repeat(e4m3_decode(scale_e4m3), 16, axis=1) * F32(g)


def dequant_fp8_1x128(vals, scale_f32):
    return e4m3_decode(vals) * np.repeat(scale_f32.astype(np.float32), 128, axis=1)


def quantize(x, fmt: int, **kw):
    """Dispatch by FMT_* -> (values, scales, global_scale or None)."""
    if fmt == FMT_ROWSCALE:
        q, s = quantize_rowscale(x)
        return q, s, None
    if fmt == FMT_BLK16_A:
        q, s = quantize_blk16(x, "A")
        return q, s, None
    if fmt == FMT_BLK16_B:
        q, s = quantize_blk16(x, "B")
        return q, s, None
    if fmt == FMT_MX32:
        q, s = quantize_mx32(x)
        return q, s, None
    if fmt == FMT_NV16:
        return quantize_nv16(x, **kw)
    if fmt == FMT_FP8_1X128:
        q, s = quantize_fp8_1x128(x)
        return q, s, None
    raise ValueError(f"unknown format {fmt}")


def dequantize(q, s, fmt: int, g=None):
    if fmt == FMT_ROWSCALE:
        return dequant_rowscale(q, s)
    if fmt == FMT_BLK16_A:
        return dequant_blk16(q, s, "A")
    if fmt == FMT_BLK16_B:
        return dequant_blk16(q, s, "B")
    if fmt == FMT_MX32:
        return dequant_mx32(q, s)
    if fmt == FMT_NV16:
        return dequant_nv16(q, s, g)
    if fmt == FMT_FP8_1X128:
        return dequant_fp8_1x128(q, s)
    raise ValueError(f"unknown format {fmt}")


# --------------------------------------------------------------------------- scale-factor atoms


def sf_atoms(scales_mk: np.ndarray, pad: int = 0) -> np.ndarray:
    """Natural per-row block scales u8 [R, nk] -> tensor-core scale-factor atoms.

    The block-scaled tcgen05 MMA reads scale factors from tensor memory in chunks of
    128 rows x 4 scale columns; a chunk is a 512-byte atom with byte offset
    ``(r % 32) * 16 + (r // 32) * 4 + (k % 4)``.  Atoms are ordered [R/128][nk/4].
    Rows / columns beyond the tensor are filled with ``pad``.
    """
    R, nk = scales_mk.shape
    Rt, Kt = -(-R // 128), -(-nk // 4)
    full = np.full((Rt * 128, Kt * 4), pad, dtype=np.uint8)
    full[:R, :nk] = scales_mk
    a = full.reshape(Rt, 4, 32, Kt, 4)  # [tile, r//32, r%32, kgroup, k%4]
    a = a.transpose(0, 3, 2, 1, 4)  # [tile, kgroup, r%32, r//32, k%4]
    return np.ascontiguousarray(a).reshape(Rt, Kt, 512)

"""Host-side operators of the quantized-linear path (PyTorch tensors in, C ABI underneath).

Two layers:

* the library's own operators -- :func:`quantize`, :func:`ln_quantize`, :func:`layernorm`,
  :func:`bsgemm` -- which carry every format and fused epilogue;
* the reference's operator names with the reference's signatures
  (``veloxvoice/kernels/ops/triton_ops.py`` and ``veloxvoice/kernels/ops/cuda_ops.py``):
  :func:`per_row_col_quantize`, :func:`triton_quantize_w`, :func:`mxfp4_block_quantize`,
  :func:`mxfp4_dequant`, :func:`dgx_mxfp4_gemm`, :func:`dgx_mxfp4_blkscale_gemm`,
  :func:`mxfp4_gemm`, :func:`nvfp4_linear`, :func:`_dequantize_to_bf16`,
  :func:`fused_layernorm`, so that code written against the reference runs unchanged.

Everything runs on torch's current CUDA stream; nothing synchronises; there is no CPU path.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import (  # noqa: F401  (re-exported)
    DT_BF16,
    DT_F32,
    DT_FP4,
    EPI_BIAS,
    EPI_BIAS_ARGMAX,
    EPI_BIAS_GLU,
    EPI_BIAS_QKVPACK,
    EPI_BIAS_RESIDUAL,
    EPI_BIAS_SWISH,
    EPI_NONE,
    FMT_BLK16_A,
    FMT_BLK16_B,
    FMT_BY_NAME,
    FMT_FP8_1X128,
    FMT_MX32,
    FMT_NV16,
    FMT_ROWSCALE,
    GEMM_DIRECT_STORE,
    GEMM_NARROW_TILES,
    GEMM_OUT_HEADS,
    GEMM_STREAM_B,
    GEMM_WIDE_TILES,
)

_SF_FORMATS = (FMT_BLK16_A, FMT_BLK16_B, FMT_MX32, FMT_NV16)
_BLOCK = {FMT_BLK16_A: 16, FMT_BLK16_B: 16, FMT_NV16: 16, FMT_MX32: 32, FMT_FP8_1X128: 128}


_launches = 0


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def launch_count() -> int:
    """Kernels of this library launched since :func:`reset_launch_count` (host-side count)."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _fmt(fmt) -> int:
    if isinstance(fmt, str):
        try:
            return FMT_BY_NAME[fmt.lower()]
        except KeyError:
            raise ValueError(f"unknown quantization format {fmt!r}") from None
    return int(fmt)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this library has no CPU path")


def _dt(t: torch.Tensor, name: str) -> int:
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise TypeError(f"{name} must be float32 or bfloat16, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _rows2d(x: torch.Tensor, name: str) -> torch.Tensor:
    if x.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(x.shape)}")
    if x.stride(1) != 1:
        x = x.contiguous()
    return x


@dataclass
class Quantized:
    """A quantized [R, K] matrix: packed values plus scales in up to two layouts."""

    fmt: int
    rows: int
    k: int
    codes: torch.Tensor  # u8 [R, K/2] (E2M1) or [R, K] (FP8)
    scales: Optional[torch.Tensor]  # natural layout (see include/velox_b200.h)
    sf: Optional[torch.Tensor]  # SF atoms, u8 [ceil(R/128), kg, 512]
    amax: Optional[torch.Tensor]  # NV16: f32[1] tensor amax

    def gemm_scales(self) -> torch.Tensor:
        if self.fmt in _SF_FORMATS:
            if self.sf is None:
                self.sf = sf_from_natural(self.fmt, self.scales, self.rows, self.k)
            return self.sf
        if self.scales is None:
            raise RuntimeError("natural-layout scales are required for this format")
        return self.scales


def sf_bytes(fmt: int, rows: int, k: int) -> int:
    return int(_lib.load().vx_sf_bytes(fmt, rows, k))


def _alloc_outputs(fmt: int, M: int, K: int, dev, natural: bool, sf: bool):
    fp8 = fmt == FMT_FP8_1X128
    codes = torch.empty((M, K if fp8 else K // 2), dtype=torch.uint8, device=dev)
    scales = None
    if natural:
        if fmt == FMT_ROWSCALE:
            scales = torch.empty((M,), dtype=torch.uint8, device=dev)
        elif fmt == FMT_BLK16_A:
            scales = torch.empty((K // 16, M // 2), dtype=torch.uint8, device=dev)
        elif fmt == FMT_BLK16_B:
            scales = torch.empty((K // 16, M), dtype=torch.uint8, device=dev)
        elif fp8:
            scales = torch.empty((M, K // 128), dtype=torch.float32, device=dev)
        else:
            scales = torch.empty((M, K // _BLOCK[fmt]), dtype=torch.uint8, device=dev)
    sf_t = None
    if sf and fmt in _SF_FORMATS:
        lib = _lib.load()
        kg = int(lib.vx_sf_kgroups(fmt, K))
        sf_t = torch.empty(((M + 127) // 128, kg, 512), dtype=torch.uint8, device=dev)
    return codes, scales, sf_t


def amax(x: torch.Tensor) -> torch.Tensor:
    """max |x| of a 2-D tensor as a device f32[1] (no host sync)."""
    _require_cuda(x, "x")
    x = _rows2d(x, "x")
    out = torch.empty((1,), dtype=torch.float32, device=x.device)
    rc = _lib.load().vx_amax(x.data_ptr(), _dt(x, "x"), x.shape[0], x.shape[1], x.stride(0), out.data_ptr(), _stream())
    _lib.check(rc, "vx_amax")
    _count()
    return out


def quantize(
    x: torch.Tensor,
    fmt,
    *,
    natural: bool = True,
    sf: bool = True,
    amax_t: Optional[torch.Tensor] = None,
) -> Quantized:
    """Quantize + pack the rows of ``x`` [M, K] (f32 or bf16) in format ``fmt``."""
    fmt = _fmt(fmt)
    _require_cuda(x, "x")
    x = _rows2d(x, "x")
    M, K = x.shape
    if fmt == FMT_NV16 and amax_t is None:
        amax_t = amax(x)
    if fmt == FMT_ROWSCALE or fmt == FMT_FP8_1X128:
        natural = True
    codes, scales, sf_t = _alloc_outputs(fmt, M, K, x.device, natural, sf)
    rc = _lib.load().vx_quantize_pack(
        x.data_ptr(), _dt(x, "x"), M, K, x.stride(0), fmt, codes.data_ptr(), codes.stride(0),
        _ptr(scales), _ptr(sf_t), _ptr(amax_t), _stream(),
    )
    _lib.check(rc, "vx_quantize_pack")
    _count()
    return Quantized(fmt, M, K, codes, scales, sf_t, amax_t)


def ln_quantize(
    x: torch.Tensor,
    gamma: torch.Tensor,
    beta: torch.Tensor,
    eps: float,
    fmt,
    *,
    natural: bool = False,
    sf: bool = True,
    amax_t: Optional[torch.Tensor] = None,
    y_dtype: Optional[torch.dtype] = None,
):
    """LayerNorm(x) quantized in one pass.  Returns ``Quantized`` (and ``y`` if ``y_dtype``)."""
    fmt = _fmt(fmt)
    _require_cuda(x, "x")
    x = _rows2d(x, "x")
    M, K = x.shape
    if fmt == FMT_NV16 and amax_t is None:
        raise ValueError("NV16 behind LayerNorm needs a calibrated tensor amax (amax_t)")
    if fmt == FMT_ROWSCALE or fmt == FMT_FP8_1X128:
        natural = True
    gamma = gamma.float().contiguous()
    beta = beta.float().contiguous()
    codes, scales, sf_t = _alloc_outputs(fmt, M, K, x.device, natural, sf)
    y = None
    if y_dtype is not None:
        y = torch.empty((M, K), dtype=y_dtype, device=x.device)
    rc = _lib.load().vx_ln_quantize_pack(
        x.data_ptr(), _dt(x, "x"), M, K, x.stride(0), gamma.data_ptr(), beta.data_ptr(), float(eps), fmt,
        codes.data_ptr(), codes.stride(0), _ptr(scales), _ptr(sf_t), _ptr(amax_t),
        _ptr(y), _dt(y, "y") if y is not None else 0, K, _stream(),
    )
    _lib.check(rc, "vx_ln_quantize_pack")
    _count()
    q = Quantized(fmt, M, K, codes, scales, sf_t, amax_t)
    return (q, y) if y is not None else q


def ln2_quantize(x: torch.Tensor, gamma1, beta1, gamma2, beta2, eps: float, fmt, *, y: Optional[torch.Tensor] = None,
                 natural: bool = False, sf: bool = True, amax_t: Optional[torch.Tensor] = None) -> Quantized:
    """``y = LN1(x)`` stored into ``y`` (may be ``x`` itself) and ``quantize(LN2(y))`` returned, in
    one pass: ``layernorm(x, g1, b1, out=y)`` followed by ``ln_quantize(y, g2, b2)``."""
    fmt = _fmt(fmt)
    _require_cuda(x, "x")
    x = _rows2d(x, "x")
    M, K = x.shape
    if fmt == FMT_NV16 and amax_t is None:
        raise ValueError("NV16 behind LayerNorm needs a calibrated tensor amax (amax_t)")
    if fmt == FMT_ROWSCALE or fmt == FMT_FP8_1X128:
        natural = True
    g1, b1 = gamma1.float().contiguous(), beta1.float().contiguous()
    g2, b2 = gamma2.float().contiguous(), beta2.float().contiguous()
    codes, scales, sf_t = _alloc_outputs(fmt, M, K, x.device, natural, sf)
    if y is not None:
        y = _rows2d(y, "y")
        if y.shape != x.shape:
            raise ValueError("y must have the shape of x")
    rc = _lib.load().vx_ln2_quantize_pack(
        x.data_ptr(), _dt(x, "x"), M, K, x.stride(0), g1.data_ptr(), b1.data_ptr(), g2.data_ptr(), b2.data_ptr(),
        float(eps), fmt, codes.data_ptr(), codes.stride(0), _ptr(scales), _ptr(sf_t), _ptr(amax_t),
        _ptr(y), _dt(y, "y") if y is not None else 0, y.stride(0) if y is not None else K, _stream(),
    )
    _lib.check(rc, "vx_ln2_quantize_pack")
    _count()
    return Quantized(fmt, M, K, codes, scales, sf_t, amax_t)


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5, out=None, out_dtype=None):
    """Row LayerNorm with fp32 statistics; output f32 or bf16."""
    _require_cuda(x, "x")
    shape = x.shape
    x2 = _rows2d(x.reshape(-1, shape[-1]), "x")
    M, K = x2.shape
    if out is None:
        out = torch.empty((M, K), dtype=out_dtype or x.dtype, device=x.device)
    out2 = out.view(M, K)
    gamma = gamma.float().contiguous()
    beta = beta.float().contiguous()
    rc = _lib.load().vx_ln_quantize_pack(
        x2.data_ptr(), _dt(x2, "x"), M, K, x2.stride(0), gamma.data_ptr(), beta.data_ptr(), float(eps), FMT_MX32,
        None, 0, None, None, None, out2.data_ptr(), _dt(out2, "out"), out2.stride(0), _stream(),
    )
    _lib.check(rc, "vx_ln_quantize_pack")
    _count()
    return out.view(shape)


def sf_from_natural(fmt, scales: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Natural-layout block scales -> SF atoms u8 [ceil(rows/128), kg, 512]."""
    fmt = _fmt(fmt)
    _require_cuda(scales, "scales")
    scales = scales.contiguous()
    lib = _lib.load()
    kg = int(lib.vx_sf_kgroups(fmt, k))
    out = torch.empty(((rows + 127) // 128, kg, 512), dtype=torch.uint8, device=scales.device)
    _lib.check(lib.vx_sf_from_natural(fmt, scales.data_ptr(), rows, k, out.data_ptr(), _stream()), "vx_sf_from_natural")
    _count()
    return out


def bsgemm(
    a: Quantized,
    b: Quantized,
    *,
    epilogue: int = EPI_NONE,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    alpha: float = 1.0,
    out_dtype=torch.bfloat16,
    out: Optional[torch.Tensor] = None,
    out_fmt=None,
    out_amax: Optional[torch.Tensor] = None,
    out_natural: bool = False,
    direct_store: bool = False,
    stream_b: bool = False,
    tiles: Optional[str] = None,
    _dbg: int = 0,
):
    """``epilogue(A . B^T)``; A [M,K], B [N,K] quantized in the same format family.

    ``out_fmt`` (MX32 or NV16) re-quantizes the result in the epilogue and returns a
    :class:`Quantized` ready to be the A operand of the next GEMM; otherwise a tensor of
    ``out_dtype`` (float32 / bfloat16) [M, N] ([M, N/2] for the GLU epilogue) is returned.
    ``tiles`` overrides the FP4 tile shape the library would pick ("wide" 128 x 256, one
    accumulator; "narrow" 128 x 128, two accumulators); results do not depend on it.
    """
    fa, fb = a.fmt, b.fmt
    if fa == FMT_BLK16_A:
        if fb != FMT_BLK16_B:
            raise ValueError("BLK16: A must be quantized in mode 'A' and B in mode 'B'")
    elif fa != fb:
        raise ValueError(f"operand formats differ ({fa} vs {fb})")
    if a.k != b.k:
        raise ValueError(f"K mismatch: {a.k} vs {b.k}")
    M, N, K = a.rows, b.rows, a.k
    dev = a.codes.device
    n_out = N // 2 if epilogue == EPI_BIAS_GLU else N
    d = _lib.GemmDesc()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = fa
    d.M, d.N, d.K = M, N, K
    d.a_codes, d.lda = a.codes.data_ptr(), a.codes.stride(0)
    d.b_codes, d.ldb = b.codes.data_ptr(), b.codes.stride(0)
    sa, sb = a.gemm_scales(), b.gemm_scales()
    d.a_scales, d.b_scales = sa.data_ptr(), sb.data_ptr()
    if fa == FMT_NV16:
        d.a_amax, d.b_amax = a.amax.data_ptr(), b.amax.data_ptr()
    d.epilogue = epilogue
    keep = [sa, sb]
    if bias is not None:
        if bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() < N:
            raise ValueError("bias must be a contiguous float32 vector with N entries")
        d.bias = bias.data_ptr()
    if epilogue == EPI_BIAS_RESIDUAL:
        if residual is None:
            raise ValueError("EPI_BIAS_RESIDUAL needs `residual`")
        residual = _rows2d(residual, "residual")
        d.residual, d.residual_dtype, d.ldr = residual.data_ptr(), _dt(residual, "residual"), residual.stride(0)
        d.alpha = float(alpha)
    if tiles not in (None, "wide", "narrow"):
        raise ValueError("tiles must be None, 'wide' or 'narrow'")
    d.flags = ((GEMM_DIRECT_STORE if direct_store else 0) | (GEMM_STREAM_B if stream_b else 0)
               | (GEMM_WIDE_TILES if tiles == "wide" else 0) | (GEMM_NARROW_TILES if tiles == "narrow" else 0) | (_dbg << 8))
    result = None
    if out_fmt is not None:
        ofmt = _fmt(out_fmt)
        codes, scales, sf_t = _alloc_outputs(ofmt, M, n_out, dev, out_natural, True)
        d.out_dtype, d.out, d.ldo = DT_FP4, codes.data_ptr(), codes.stride(0)
        d.out_fmt = ofmt
        d.out_scales_sf = sf_t.data_ptr()
        d.out_scales = _ptr(scales)
        if ofmt == FMT_NV16:
            if out_amax is None:
                raise ValueError("NV16 output needs a calibrated tensor amax (out_amax)")
            d.out_amax = out_amax.data_ptr()
        result = Quantized(ofmt, M, n_out, codes, scales, sf_t, out_amax)
    else:
        if out is None:
            if out_dtype == torch.bfloat16 and n_out % 8 != 0:
                # pad the row pitch to 16 bytes so the TMA store path applies
                ld = (n_out + 7) // 8 * 8
                out = torch.empty((M, ld), dtype=out_dtype, device=dev)[:, :n_out]
            else:
                out = torch.empty((M, n_out), dtype=out_dtype, device=dev)
        if out.dim() != 2 or out.shape[0] != M or out.shape[1] != n_out or out.stride(1) != 1:
            raise ValueError(f"out must be [{M}, {n_out}] with unit column stride")
        d.out_dtype, d.out, d.ldo = _dt(out, "out"), out.data_ptr(), out.stride(0)
        result = out
    _lib.check(_lib.load().vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    del keep
    return result


def bsgemm_argmax(a: Quantized, b: Quantized, bias: Optional[torch.Tensor] = None, *,
                  return_max: bool = False, keys: Optional[torch.Tensor] = None,
                  ids: Optional[torch.Tensor] = None):
    """Per row of ``A . B^T + bias``: the first column holding the maximum of the bf16-rounded
    result -- ``bsgemm(..., out_dtype=bfloat16).argmax(1)`` without writing the [M, N] matrix
    (the greedy CTC head).  Returns int32 ids [M] (and the winning values as float32 [M])."""
    if a.fmt != b.fmt and not (a.fmt == FMT_BLK16_A and b.fmt == FMT_BLK16_B):
        raise ValueError(f"operand formats differ ({a.fmt} vs {b.fmt})")
    if a.k != b.k:
        raise ValueError(f"K mismatch: {a.k} vs {b.k}")
    M, N, K = a.rows, b.rows, a.k
    dev = a.codes.device
    if keys is None:
        keys = torch.empty((M,), dtype=torch.int64, device=dev)
    if ids is None:
        ids = torch.empty((M,), dtype=torch.int32, device=dev)
    if keys.dtype != torch.int64 or keys.numel() < M or ids.dtype != torch.int32 or ids.numel() < M:
        raise ValueError("keys must be int64 [M] and ids int32 [M]")
    d = _lib.GemmDesc()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = a.fmt
    d.M, d.N, d.K = M, N, K
    d.a_codes, d.lda = a.codes.data_ptr(), a.codes.stride(0)
    d.b_codes, d.ldb = b.codes.data_ptr(), b.codes.stride(0)
    sa, sb = a.gemm_scales(), b.gemm_scales()
    d.a_scales, d.b_scales = sa.data_ptr(), sb.data_ptr()
    if a.fmt == FMT_NV16:
        d.a_amax, d.b_amax = a.amax.data_ptr(), b.amax.data_ptr()
    d.epilogue = EPI_BIAS_ARGMAX
    if bias is not None:
        if bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() < N:
            raise ValueError("bias must be a contiguous float32 vector with N entries")
        d.bias = bias.data_ptr()
    d.out_dtype, d.out, d.ldo = DT_F32, keys.data_ptr(), 1
    lib = _lib.load()
    _lib.check(lib.vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    vmax = torch.empty((M,), dtype=torch.float32, device=dev) if return_max else None
    _lib.check(lib.vx_argmax_ids(keys.data_ptr(), M, ids.data_ptr(), _ptr(vmax), _stream()), "vx_argmax_ids")
    _count()
    del sa, sb
    return (ids, vmax) if return_max else ids


def qkv_pack(qkv: torch.Tensor, p0: torch.Tensor, pos_u: torch.Tensor, pos_v: torch.Tensor, scale: float):
    """Single-pass attention fold pack, signature of the reference's ``qkv_pack``
    (``veloxvoice/kernels/ops/cuda_ops.py:554-581``): qkv bf16 [T, 3d], p0 bf16 [T, d],
    pos_u / pos_v [h, dk] -> (q2, k2, v2) bf16 [h, T, 2 dk] each."""
    _require_cuda(qkv, "qkv")
    if qkv.dtype != torch.bfloat16 or p0.dtype != torch.bfloat16:
        raise ValueError("qkv and p0 must be bfloat16")
    T, d3 = qkv.shape
    d = d3 // 3
    h = pos_u.shape[0]
    dk = d // h
    if d * 3 != d3 or h * dk != d or p0.shape != (T, d):
        raise ValueError("shapes: qkv [T, 3 h dk], p0 [T, h dk], pos_u / pos_v [h, dk]")
    qkv, p0 = _rows2d(qkv, "qkv"), _rows2d(p0, "p0")
    u = pos_u.to(torch.bfloat16).contiguous()
    v = pos_v.to(torch.bfloat16).contiguous()
    packed = torch.empty((3, h, T, 2 * dk), dtype=torch.bfloat16, device=qkv.device)
    rc = _lib.load().vx_qkv_pack(qkv.data_ptr(), qkv.stride(0), p0.data_ptr(), p0.stride(0), u.data_ptr(), v.data_ptr(),
                                 float(scale), T, h, dk, packed[0].data_ptr(), packed[1].data_ptr(), packed[2].data_ptr(),
                                 _stream())
    _lib.check(rc, "vx_qkv_pack")
    _count()
    return packed[0], packed[1], packed[2]


def bsgemm_qkv_pack(a: Quantized, w_qkv: Quantized, bias: Optional[torch.Tensor], pos_u: torch.Tensor,
                    pos_v: torch.Tensor, scale: float, *, packed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused QKV projection written straight into the attention fold pack (``qkv_pack`` of the
    bf16 projection, without the [T, 3d] intermediate).  Returns bf16 [3, h, T, 2 dk]:
    ``packed[0]`` = q2, ``packed[1]`` = k2 (second half of every head row NOT written: it belongs
    to ``bsgemm_heads(pos, lp, out=packed[1], col_off=dk)``), ``packed[2]`` = v2."""
    h, dk = pos_u.shape
    M, N, K = a.rows, w_qkv.rows, a.k
    if N != 3 * h * dk or a.k != w_qkv.k or a.fmt != w_qkv.fmt:
        raise ValueError("w_qkv must be [3 h dk, K] in the format of the activations")
    dev = a.codes.device
    if packed is None:
        packed = torch.empty((3, h, M, 2 * dk), dtype=torch.bfloat16, device=dev)
    if packed.shape != (3, h, M, 2 * dk) or packed.dtype != torch.bfloat16 or not packed.is_contiguous():
        raise ValueError("packed must be a contiguous bf16 [3, h, M, 2 dk] tensor")
    u = pos_u.to(torch.bfloat16).contiguous()
    v = pos_v.to(torch.bfloat16).contiguous()
    d = _lib.GemmDesc()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = a.fmt
    d.M, d.N, d.K = M, N, K
    d.a_codes, d.lda = a.codes.data_ptr(), a.codes.stride(0)
    d.b_codes, d.ldb = w_qkv.codes.data_ptr(), w_qkv.codes.stride(0)
    sa, sb = a.gemm_scales(), w_qkv.gemm_scales()
    d.a_scales, d.b_scales = sa.data_ptr(), sb.data_ptr()
    if a.fmt == FMT_NV16:
        d.a_amax, d.b_amax = a.amax.data_ptr(), w_qkv.amax.data_ptr()
    d.epilogue = EPI_BIAS_QKVPACK
    if bias is not None:
        d.bias = bias.data_ptr()
    d.out_dtype, d.out, d.ldo = DT_BF16, packed.data_ptr(), 2 * dk
    d.heads, d.head_dim = h, dk
    d.pos_u, d.pos_v, d.qk_scale = u.data_ptr(), v.data_ptr(), float(scale)
    _lib.check(_lib.load().vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    del sa, sb, u, v
    return packed


def bsgemm_heads(a: Quantized, w: Quantized, bias: Optional[torch.Tensor], out: torch.Tensor, *, col_off: int = 0):
    """``A . W^T (+ bias)`` written head-major: ``out`` bf16 [h, M, width], result column n goes to
    ``out[n // dk, m, col_off + n % dk]`` with dk = N / h.  With ``out = packed[1]`` and
    ``col_off = dk`` this puts lp(pos_emb) where the attention fold pack wants it."""
    h, M, width = out.shape
    N = w.rows
    dk = N // h
    if M != a.rows or h * dk != N or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 [h, M, width] tensor with N = h * dk")
    d = _lib.GemmDesc()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = a.fmt
    d.M, d.N, d.K = M, N, a.k
    d.a_codes, d.lda = a.codes.data_ptr(), a.codes.stride(0)
    d.b_codes, d.ldb = w.codes.data_ptr(), w.codes.stride(0)
    sa, sb = a.gemm_scales(), w.gemm_scales()
    d.a_scales, d.b_scales = sa.data_ptr(), sb.data_ptr()
    if a.fmt == FMT_NV16:
        d.a_amax, d.b_amax = a.amax.data_ptr(), w.amax.data_ptr()
    d.epilogue = EPI_BIAS if bias is not None else EPI_NONE
    if bias is not None:
        d.bias = bias.data_ptr()
    d.out_dtype, d.out, d.ldo = DT_BF16, out.data_ptr(), width
    d.heads, d.head_dim, d.head_col_off = h, dk, col_off
    d.flags = GEMM_OUT_HEADS
    _lib.check(_lib.load().vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    del sa, sb
    return out


def mma_peak_tflops(kind: str = "fp4", n_tile: int = 256, iters: int = 4096) -> float:
    """Measured tensor-core rate of back-to-back MMAs without memory traffic (dense TFLOP/s)."""
    out = C.c_float(0.0)
    rc = _lib.load().vx_mma_peak_probe(0 if kind == "fp4" else 1, n_tile, iters, C.byref(out))
    _lib.check(rc, "vx_mma_peak_probe")
    return float(out.value)


# ======================================================================================
# The reference's operator names (same positional order, defaults and return types).
# ======================================================================================


def per_row_col_quantize(w, block_size=None):
    """[M, K] bf16/fp32 -> (packed u8 [M, K/2], per-row ue8m0 u8 [M]).

    Same contract as ``veloxvoice/kernels/ops/triton_ops.py:92-124``.
    """
    assert w.ndim == 2
    assert w.shape[1] % 2 == 0, "K must be even"
    q = quantize(w, FMT_ROWSCALE, sf=False)
    return q.codes, q.scales


def triton_quantize_w(w, block_size=None):
    """Alias kept for callers of the reference (``triton_ops.py:128-129``)."""
    return per_row_col_quantize(w, block_size)


def quantize_w(w, block_size=16, format="nvfp4"):
    """``veloxvoice/models/wenet/nvfp4_linear.py:66-68``."""
    return per_row_col_quantize(w, block_size)


def mxfp4_block_quantize(w, mode: str = "A"):
    """[R, K] -> (packed u8 [R, K/2], ue8m0 u8 [K/16][R2], kb-major) (``triton_ops.py:261-293``)."""
    assert w.ndim == 2
    assert w.shape[1] % 16 == 0, "K must be divisible by 16"
    assert mode != "A" or w.shape[0] % 2 == 0, "mode A requires even R (row pairs)"
    q = quantize(w, FMT_BLK16_A if mode == "A" else FMT_BLK16_B, sf=False)
    return q.codes, q.scales


_E2M1_LUT = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _decode_e2m1(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    c = torch.stack([lo, hi], -1).reshape(packed.shape[0], packed.shape[1] * 2)
    lut = torch.tensor(_E2M1_LUT, device=packed.device)
    mag = lut[(c & 7).long()]
    return torch.where((c & 8) > 0, -mag, mag)


def mxfp4_dequant(q, s, mode: str = "A"):
    """(packed [R, K/2], kb-major ue8m0 [K/16][R2]) -> f32 [R, K] (``triton_ops.py:296-309``)."""
    sv = 2.0 ** (s.to(torch.int16).to(torch.float32) - 127)
    if mode == "A":
        sv = sv.repeat_interleave(2, dim=1)
    return _decode_e2m1(q) * sv.T.repeat_interleave(16, dim=1)


def _dequantize_to_bf16(packed, scale_u8):
    """packed u8 [N, K/2] + ue8m0 u8 [N] -> bf16 [N, K] (``cuda_ops.py:710-723``)."""
    s = (2.0 ** (scale_u8.to(torch.int16).to(torch.float32) - 127)).unsqueeze(1)
    return (_decode_e2m1(packed) * s).to(torch.bfloat16)


def _as_quantized_rowscale(codes, scales) -> Quantized:
    _require_cuda(codes, "pack")
    codes = _rows2d(codes, "pack")
    return Quantized(FMT_ROWSCALE, codes.shape[0], codes.shape[1] * 2, codes, scales.contiguous().view(-1), None, None)


def dgx_mxfp4_gemm(
    pack_a,
    pack_b,
    scale_a,
    scale_b,
    num_producer_warps=1,
    num_consumer_warps=8,
    group_size_m=16,
    cluster_size_m=1,
):
    """pack_a [M, K/2] u8; pack_b [N, K/2] u8; per-row ue8m0 scales -> out [M, N] f32.

    ``Out = (A . B^T) * 2^(sa[m]-127) * 2^(sb[n]-127)`` (``cuda_ops.py:626-645``).  The four
    tuning arguments of the reference's kernel are accepted and ignored.  Unlike the
    reference, M and N need not be multiples of 128 (K must be a multiple of 32).
    """
    a = _as_quantized_rowscale(pack_a, scale_a)
    b = _as_quantized_rowscale(pack_b, scale_b)
    return bsgemm(a, b, epilogue=EPI_NONE, out_dtype=torch.float32)


def dgx_mxfp4_blkscale_gemm(
    pack_a,
    pack_b,
    scale_a,
    scale_b,
    num_producer_warps=1,
    num_consumer_warps=8,
    group_size_m=16,
    cluster_size_m=1,
):
    """Per-16-column block-scaled product, raw f32 (``cuda_ops.py:679-702``).

    scale_a: ue8m0 u8 [K/16][M/2] (row pairs); scale_b: ue8m0 u8 [K/16][N].
    """
    _require_cuda(pack_a, "pack_a")
    pa, pb = _rows2d(pack_a, "pack_a"), _rows2d(pack_b, "pack_b")
    M, N, K = pa.shape[0], pb.shape[0], pa.shape[1] * 2
    a = Quantized(FMT_BLK16_A, M, K, pa, scale_a.contiguous(), None, None)
    b = Quantized(FMT_BLK16_B, N, K, pb, scale_b.contiguous(), None, None)
    return bsgemm(a, b, epilogue=EPI_NONE, out_dtype=torch.float32)


def mxfp4_gemm(xq, wq, xs, ws, P=1, C=8, group_size_m=16):
    """``cuda_ops.py:705-707``."""
    return dgx_mxfp4_blkscale_gemm(xq, wq, xs, ws, P, C, group_size_m)


def nvfp4_linear(x, wq, ws, P=4, C=8, w_bf16=None):
    """Quantize ``x`` per row and multiply with a pre-quantized weight (``cuda_ops.py:648-676``).

    The reference switches to a bf16 cuBLAS matmul on a pre-dequantized weight for M <= 512;
    here every M runs the FP4 tensor-core kernel (``w_bf16`` is accepted and unused).
    """
    K = x.shape[-1]
    N = wq.shape[0]
    x_2d = x.reshape(-1, K)
    a = quantize(x_2d, FMT_ROWSCALE, sf=False)
    b = _as_quantized_rowscale(wq, ws)
    out = bsgemm(a, b, epilogue=EPI_NONE, out_dtype=torch.float32)
    return out.view(*x.shape[:-1], N)


def fused_layernorm(x, w, b, eps=1e-5, out=None):
    """Row LayerNorm (``cuda_ops.py:204-210``)."""
    return layernorm(x, w, b, eps, out=out)


def _pad16(t: torch.Tensor, multiple: int) -> torch.Tensor:
    """Zero-pad the rows of ``t`` to a multiple of ``multiple``.

    The reference imports this helper from ``veloxvoice.models.wenet.mxfp4_linear``
    (``veloxvoice/models/wenet/torch_conformer.py:222-229``), a module its tree does not
    contain; the call site fixes the behaviour.
    """
    r = t.shape[0]
    rp = (r + multiple - 1) // multiple * multiple
    if rp == r:
        return t
    out = torch.zeros((rp,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    out[:r] = t
    return out

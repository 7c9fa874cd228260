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


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5, out=None, out_dtype=None,
              fmt="mx32"):
    """Row LayerNorm with fp32 statistics; output f32 or bf16.  ``fmt`` names the quantization lane the
    result belongs to: the LayerNorm runs on the kernel (and so with the summation order, which shows in
    the last bit) that ``ln_quantize(..., fmt)`` would use, so that a stored LayerNorm followed by
    ``ln_quantize`` equals ``ln2_quantize`` exactly in every format."""
    fmt = _fmt(fmt)
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
        x2.data_ptr(), _dt(x2, "x"), M, K, x2.stride(0), gamma.data_ptr(), beta.data_ptr(), float(eps), fmt,
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


def _check_vector(t: Optional[torch.Tensor], name: str, n: int, dev, dtype=torch.float32) -> None:
    if t is None:
        return
    _require_cuda(t, name)
    if t.device != dev:
        raise ValueError(f"{name} is on {t.device}, the operands are on {dev}")
    if t.dtype != dtype or not t.is_contiguous() or t.numel() < n:
        raise ValueError(f"{name} must be a contiguous {dtype} tensor with at least {n} entries")


def _gemm_desc(a: Quantized, b: Quantized, bias: Optional[torch.Tensor]):
    """Checks the operands of a GEMM (formats, K, device, bias) and returns a ``vx_gemm_desc``
    with the operand side filled in, plus the tensors that must outlive the launch."""
    if not isinstance(a, Quantized) or not isinstance(b, Quantized):
        raise TypeError("operands must be Quantized (see quantize / ln_quantize)")
    fa, fb = a.fmt, b.fmt
    if fa == FMT_BLK16_A:
        if fb != FMT_BLK16_B:
            raise ValueError("BLK16: A must be quantized in mode 'A' and B in mode 'B'")
    elif fa != fb:
        raise ValueError(f"operand formats differ ({fa} vs {fb})")
    if a.k != b.k:
        raise ValueError(f"K mismatch: {a.k} vs {b.k}")
    _require_cuda(a.codes, "A codes")
    _require_cuda(b.codes, "B codes")
    dev = a.codes.device
    if b.codes.device != dev:
        raise ValueError(f"operands on different devices ({dev} vs {b.codes.device})")
    _check_vector(bias, "bias", b.rows, dev)
    d = _lib.GemmDesc()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = fa
    d.M, d.N, d.K = a.rows, b.rows, a.k
    d.a_codes, d.lda = a.codes.data_ptr(), a.codes.stride(0)
    d.b_codes, d.ldb = b.codes.data_ptr(), b.codes.stride(0)
    sa, sb = a.gemm_scales(), b.gemm_scales()
    d.a_scales, d.b_scales = sa.data_ptr(), sb.data_ptr()
    if fa == FMT_NV16:
        if a.amax is None or b.amax is None:
            raise ValueError("NV16 operands carry their tensor amax")
        d.a_amax, d.b_amax = a.amax.data_ptr(), b.amax.data_ptr()
    if bias is not None:
        d.bias = bias.data_ptr()
    return d, (sa, sb)


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
):
    """``epilogue(A . B^T)``; A [M,K], B [N,K] quantized in the same format family.

    ``out_fmt`` (MX32 or NV16) re-quantizes the result in the epilogue and returns a
    :class:`Quantized` ready to be the A operand of the next GEMM; otherwise a tensor of
    ``out_dtype`` (float32 / bfloat16) [M, N] ([M, N/2] for the GLU epilogue) is returned.
    ``tiles`` overrides the FP4 tile shape the library would pick ("wide" 128 x 256, one
    accumulator; "narrow" 128 x 128, two accumulators); results do not depend on it.
    """
    d, keep = _gemm_desc(a, b, bias)
    M, N, K = a.rows, b.rows, a.k
    dev = a.codes.device
    n_out = N // 2 if epilogue == EPI_BIAS_GLU else N
    d.epilogue = epilogue
    if epilogue == EPI_BIAS_RESIDUAL:
        if residual is None:
            raise ValueError("EPI_BIAS_RESIDUAL needs `residual`")
        _require_cuda(residual, "residual")
        residual = _rows2d(residual, "residual")
        if residual.shape[0] != M or residual.shape[1] != N or residual.device != dev:
            raise ValueError(f"residual must be [{M}, {N}] on {dev}")
        d.residual, d.residual_dtype, d.ldr = residual.data_ptr(), _dt(residual, "residual"), residual.stride(0)
        d.alpha = float(alpha)
    if tiles not in (None, "wide", "narrow"):
        raise ValueError("tiles must be None, 'wide' or 'narrow'")
    d.flags = ((GEMM_DIRECT_STORE if direct_store else 0) | (GEMM_STREAM_B if stream_b else 0)
               | (GEMM_WIDE_TILES if tiles == "wide" else 0) | (GEMM_NARROW_TILES if tiles == "narrow" else 0))
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
            _check_vector(out_amax, "out_amax", 1, dev)
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
        _require_cuda(out, "out")
        if out.dim() != 2 or out.shape[0] != M or out.shape[1] != n_out or out.stride(1) != 1 or out.device != dev:
            raise ValueError(f"out must be [{M}, {n_out}] with unit column stride on {dev}")
        d.out_dtype, d.out, d.ldo = _dt(out, "out"), out.data_ptr(), out.stride(0)
        result = out
    _lib.check(_lib.load().vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    del keep
    return result


def residual_ln_supported(fmt, N: int, K: int) -> bool:
    """Whether :func:`bsgemm_residual_ln` covers a residual GEMM of this format and shape."""
    return bool(_lib.load().vx_bsgemm_residual_ln_supported(_fmt(fmt), int(N), int(K)))


def bsgemm_residual_ln(a: Quantized, b: Quantized, *, bias: Optional[torch.Tensor], residual: torch.Tensor,
                       gamma: torch.Tensor, beta: torch.Tensor, eps: float, alpha: float = 1.0,
                       out: Optional[torch.Tensor] = None, gamma2: Optional[torch.Tensor] = None,
                       beta2: Optional[torch.Tensor] = None):
    """The residual GEMM and the LayerNorm + MX32 quantizer behind it in one launch:
    ``x = bf16(alpha (A . B^T + bias) + residual)`` and ``q = ln_quantize(x, gamma, beta, eps, MX32)``
    -- the same bits as ``bsgemm(..., epilogue=EPI_BIAS_RESIDUAL)`` followed by :func:`ln_quantize`.
    MX32 operands, N = 512, K a multiple of 256; ``residual`` / ``out`` bf16 [M, 512] (``out`` may be
    ``residual``).  Returns ``(x, q)``.

    With ``gamma2`` / ``beta2`` (the end of a Conformer block): ``out`` receives ``y = LN(x; gamma, beta)``
    instead of x and ``q = ln_quantize(y, gamma2, beta2)`` -- the bits of the GEMM followed by
    ``ln2_quantize(x, gamma, beta, gamma2, beta2, eps, MX32, y=x)``.  Returns ``(y, q)``."""
    d, keep = _gemm_desc(a, b, bias)
    M, N = a.rows, b.rows
    dev = a.codes.device
    _require_cuda(residual, "residual")
    residual = _rows2d(residual, "residual")
    if residual.shape[0] != M or residual.shape[1] != N or residual.device != dev:
        raise ValueError(f"residual must be [{M}, {N}] on {dev}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    _require_cuda(out, "out")
    if out.dim() != 2 or out.shape[0] != M or out.shape[1] != N or out.stride(1) != 1 or out.device != dev:
        raise ValueError(f"out must be [{M}, {N}] with unit column stride on {dev}")
    d.epilogue = EPI_BIAS_RESIDUAL
    d.residual, d.residual_dtype, d.ldr = residual.data_ptr(), _dt(residual, "residual"), residual.stride(0)
    d.alpha = float(alpha)
    d.out_dtype, d.out, d.ldo = _dt(out, "out"), out.data_ptr(), out.stride(0)
    gamma = gamma.float().contiguous()
    beta = beta.float().contiguous()
    _check_vector(gamma, "gamma", N, dev)
    _check_vector(beta, "beta", N, dev)
    codes, scales, sf_t = _alloc_outputs(FMT_MX32, M, N, dev, False, True)
    if (gamma2 is None) != (beta2 is None):
        raise ValueError("gamma2 and beta2 go together")
    if gamma2 is None:
        _lib.check(_lib.load().vx_bsgemm_residual_ln(C.byref(d), gamma.data_ptr(), beta.data_ptr(), float(eps),
                                                     codes.data_ptr(), codes.stride(0), sf_t.data_ptr(), _stream()),
                   "vx_bsgemm_residual_ln")
    else:
        gamma2 = gamma2.float().contiguous()
        beta2 = beta2.float().contiguous()
        _check_vector(gamma2, "gamma2", N, dev)
        _check_vector(beta2, "beta2", N, dev)
        _lib.check(_lib.load().vx_bsgemm_residual_ln2(C.byref(d), gamma.data_ptr(), beta.data_ptr(), gamma2.data_ptr(),
                                                      beta2.data_ptr(), float(eps), codes.data_ptr(), codes.stride(0),
                                                      sf_t.data_ptr(), _stream()),
                   "vx_bsgemm_residual_ln2")
    _count()
    del keep
    return out, Quantized(FMT_MX32, M, N, codes, scales, sf_t, None)


def bsgemm_argmax(a: Quantized, b: Quantized, bias: Optional[torch.Tensor] = None, *,
                  return_max: bool = False, keys: Optional[torch.Tensor] = None,
                  ids: Optional[torch.Tensor] = None, return_logp: bool = False):
    """Per row of ``A . B^T + bias``: the first column holding the maximum of the bf16-rounded
    result -- ``bsgemm(..., out_dtype=bfloat16).argmax(1)`` without writing the [M, N] matrix
    (the greedy CTC head).  Returns int32 ids [M] (and the winning values as float32 [M]).

    ``return_logp`` (FP4 formats) also returns ``(lse, logp)`` float32 [M]: the log-sum-exp of the
    row's bf16 logits and ``log_softmax(row)[argmax] = max - lse`` -- what the reference's
    ``ctc_logp`` (``torch_conformer.py:945-949``) holds at the greedy token, still without the
    logits."""
    d, keep = _gemm_desc(a, b, bias)
    M, N, K = a.rows, b.rows, a.k
    dev = a.codes.device
    if keys is None:
        keys = torch.empty((M,), dtype=torch.int64, device=dev)
    if ids is None:
        ids = torch.empty((M,), dtype=torch.int32, device=dev)
    _check_vector(keys, "keys", M, dev, torch.int64)
    _check_vector(ids, "ids", M, dev, torch.int32)
    d.epilogue = EPI_BIAS_ARGMAX
    d.out_dtype, d.out, d.ldo = DT_F32, keys.data_ptr(), 1
    lib = _lib.load()
    parts = None
    if return_logp:
        if a.fmt == FMT_FP8_1X128:
            raise ValueError("return_logp runs on the FP4 formats")
        parts = torch.empty((int(lib.vx_ctc_lse_parts(N)), M, 2), dtype=torch.float32, device=dev)
        d.lse_partials = parts.data_ptr()
    _lib.check(lib.vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    vmax = torch.empty((M,), dtype=torch.float32, device=dev) if return_max else None
    if return_logp:
        lse = torch.empty((M,), dtype=torch.float32, device=dev)
        logp = torch.empty((M,), dtype=torch.float32, device=dev)
        _lib.check(lib.vx_ctc_finish(keys.data_ptr(), parts.data_ptr(), N, M, ids.data_ptr(), _ptr(vmax), lse.data_ptr(),
                                     logp.data_ptr(), _stream()), "vx_ctc_finish")
        _count()
        del keep, parts
        return (ids, vmax, lse, logp) if return_max else (ids, lse, logp)
    _lib.check(lib.vx_argmax_ids(keys.data_ptr(), M, ids.data_ptr(), _ptr(vmax), _stream()), "vx_argmax_ids")
    _count()
    del keep
    return (ids, vmax) if return_max else ids


def bsgemm_topk(a: Quantized, b: Quantized, bias: Optional[torch.Tensor] = None, k: int = 5, *, capacity: int = 64):
    """``torch.topk(log_softmax(A . B^T + bias), k)`` of the bf16-rounded logits without writing the [M, N] matrix:
    the stream the reference's prefix beam search takes (``veloxvoice/stream/rescore.py:252-262``,
    ``cuda_ops.py:836-893``).  Returns ``(logp f32 [M, k], ids int64 [M, k])``, largest first, equal logits by
    ascending column.  Two launches of the GEMM (arg-max + log-sum-exp partials, then the candidate pass against
    the k-th largest 64-column-group maximum of each row) and two small kernels; rows whose candidate list
    overflowed ``capacity`` (many equal bf16 logits) are redone from explicit logits."""
    if a.fmt == FMT_FP8_1X128:
        raise ValueError("bsgemm_topk runs on the FP4 formats")
    if not 1 <= k <= 16:
        raise ValueError("k must be in 1..16")
    d, keep = _gemm_desc(a, b, bias)
    M, N = a.rows, b.rows
    dev = a.codes.device
    lib = _lib.load()
    nparts = int(lib.vx_ctc_lse_parts(N))
    if k > nparts:
        raise ValueError(f"k = {k} exceeds the number of 64-column groups ({nparts})")
    keys = torch.empty((M,), dtype=torch.int64, device=dev)
    parts = torch.empty((nparts, M, 2), dtype=torch.float32, device=dev)
    d.epilogue = EPI_BIAS_ARGMAX
    d.out_dtype, d.out, d.ldo = DT_F32, keys.data_ptr(), 1
    d.lse_partials = parts.data_ptr()
    _lib.check(lib.vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    thr = torch.empty((M,), dtype=torch.float32, device=dev)
    _lib.check(lib.vx_ctc_topk_threshold(parts.data_ptr(), N, M, k, thr.data_ptr(), _stream()), "vx_ctc_topk_threshold")
    cand = torch.empty((M, capacity), dtype=torch.int64, device=dev)
    cnt = torch.zeros((M,), dtype=torch.int32, device=dev)
    over = torch.zeros((1,), dtype=torch.int32, device=dev)
    d.topk_threshold, d.topk_candidates, d.topk_count, d.topk_capacity = thr.data_ptr(), cand.data_ptr(), cnt.data_ptr(), capacity
    _lib.check(lib.vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    ids = torch.empty((M, k), dtype=torch.int32, device=dev)
    logp = torch.empty((M, k), dtype=torch.float32, device=dev)
    _lib.check(lib.vx_ctc_topk_finish(cand.data_ptr(), cnt.data_ptr(), capacity, parts.data_ptr(), N, M, k, ids.data_ptr(),
                                      logp.data_ptr(), over.data_ptr(), _stream()), "vx_ctc_topk_finish")
    _count(4)
    ids = ids.long()
    if int(over.item()):
        # rare: some rows hold more than `capacity` logits at or above their threshold (many equal bf16 values);
        # those rows are redone from explicit logits
        rows = (ids[:, 0] < 0).nonzero()[:, 0]
        z = bsgemm(a, b, epilogue=EPI_BIAS if bias is not None else EPI_NONE, bias=bias, out_dtype=torch.bfloat16)
        v, i = torch.topk(torch.log_softmax(z[rows].float(), dim=-1), k, dim=-1)
        del z
        logp[rows], ids[rows] = v, i
    del keep
    return logp, ids


def qkv_pack(qkv: torch.Tensor, p0: torch.Tensor, pos_u: torch.Tensor, pos_v: torch.Tensor, scale: float):
    """Single-pass attention fold pack, signature of the reference's ``qkv_pack``
    (``veloxvoice/kernels/ops/cuda_ops.py:554-581``): qkv bf16 [T, 3d], p0 bf16 [T, d],
    pos_u / pos_v [h, dk] -> (q2, k2, v2) bf16 [h, T, 2 dk] each."""
    for t, n in ((qkv, "qkv"), (p0, "p0"), (pos_u, "pos_u"), (pos_v, "pos_v")):
        _require_cuda(t, n)
        if t.device != qkv.device:
            raise ValueError(f"{n} is on {t.device}, qkv on {qkv.device}")
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


def relpos_attention(q2: torch.Tensor, k2: torch.Tensor, v2: torch.Tensor, kv_len: Optional[int] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The encoder's relative-position attention on the fold pack: q2, k2, v2 bf16 [h, T, 2 dk] (what
    ``qkv_pack`` / ``bsgemm_qkv_pack`` + ``bsgemm_heads`` produce) -> bf16 [T, h dk], i.e.
    ``scaled_dot_product_attention(q2, k2, v2, scale=1.0)[..., :dk].transpose(0, 1).reshape(T, h * dk)``
    of ``veloxvoice/models/wenet/torch_conformer.py:514-519`` in one launch (``vx_relpos_attention``);
    keys at and beyond ``kv_len`` are masked (a padded span)."""
    for t, n in ((q2, "q2"), (k2, "k2"), (v2, "v2")):
        _require_cuda(t, n)
        if t.dtype != torch.bfloat16 or t.dim() != 3 or t.shape != q2.shape or t.device != q2.device:
            raise ValueError("q2, k2, v2 must be bfloat16 [heads, T, 2 head_dim] tensors of one shape on one device")
    h, T, d2 = q2.shape
    dk = d2 // 2
    if d2 != 128:
        raise ValueError(f"head_dim must be 64 (folded 128), got {dk}")
    q2, k2, v2 = q2.contiguous(), k2.contiguous(), v2.contiguous()
    if out is None:
        out = torch.empty((T, h * dk), dtype=torch.bfloat16, device=q2.device)
    elif out.dtype != torch.bfloat16 or out.dim() != 2 or out.shape[0] != T or out.shape[1] < h * dk or out.stride(1) != 1:
        raise ValueError("out must be bfloat16 [T, >= heads * head_dim] with unit column stride")
    rc = _lib.load().vx_relpos_attention(q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), T, h, dk,
                                         0 if kv_len is None else int(kv_len), out.data_ptr(), out.stride(0), _stream())
    _lib.check(rc, "vx_relpos_attention")
    _count()
    return out


def bsgemm_qkv_pack(a: Quantized, w_qkv: Quantized, bias: Optional[torch.Tensor], pos_u: torch.Tensor,
                    pos_v: torch.Tensor, scale: float, *, packed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused QKV projection written straight into the attention fold pack (``qkv_pack`` of the
    bf16 projection, without the [T, 3d] intermediate).  Returns bf16 [3, h, T, 2 dk]:
    ``packed[0]`` = q2, ``packed[1]`` = k2 (second half of every head row NOT written: it belongs
    to ``bsgemm_heads(pos, lp, out=packed[1], col_off=dk)``), ``packed[2]`` = v2."""
    d, keep = _gemm_desc(a, w_qkv, bias)
    if a.fmt == FMT_ROWSCALE:
        raise ValueError("the fused fold pack runs in the block-scaled formats and FP8, not per-row scales")
    dev = a.codes.device
    for t, n in ((pos_u, "pos_u"), (pos_v, "pos_v")):
        _require_cuda(t, n)
        if t.device != dev or t.dim() != 2 or t.shape != pos_u.shape:
            raise ValueError("pos_u / pos_v must be [h, dk] tensors on the operands' device")
    h, dk = pos_u.shape
    M, N, K = a.rows, w_qkv.rows, a.k
    if N != 3 * h * dk:
        raise ValueError("w_qkv must be [3 h dk, K]")
    if packed is None:
        packed = torch.empty((3, h, M, 2 * dk), dtype=torch.bfloat16, device=dev)
    _require_cuda(packed, "packed")
    if (packed.shape != (3, h, M, 2 * dk) or packed.dtype != torch.bfloat16 or not packed.is_contiguous()
            or packed.device != dev):
        raise ValueError("packed must be a contiguous bf16 [3, h, M, 2 dk] tensor on the operands' device")
    u = pos_u.to(torch.bfloat16).contiguous()
    v = pos_v.to(torch.bfloat16).contiguous()
    d.epilogue = EPI_BIAS_QKVPACK
    d.out_dtype, d.out, d.ldo = DT_BF16, packed.data_ptr(), 2 * dk
    d.heads, d.head_dim = h, dk
    d.pos_u, d.pos_v, d.qk_scale = u.data_ptr(), v.data_ptr(), float(scale)
    _lib.check(_lib.load().vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    del keep, u, v
    return packed


def bsgemm_heads(a: Quantized, w: Quantized, bias: Optional[torch.Tensor], out: torch.Tensor, *, col_off: int = 0):
    """``A . W^T (+ bias)`` written head-major: ``out`` bf16 [h, M, width], result column n goes to
    ``out[n // dk, m, col_off + n % dk]`` with dk = N / h.  With ``out = packed[1]`` and
    ``col_off = dk`` this puts lp(pos_emb) where the attention fold pack wants it."""
    d, keep = _gemm_desc(a, w, bias)
    _require_cuda(out, "out")
    if out.dim() != 3:
        raise ValueError("out must be [h, M, width]")
    h, M, width = out.shape
    N = w.rows
    dk = N // h
    if (M != a.rows or h * dk != N or out.dtype != torch.bfloat16 or not out.is_contiguous()
            or out.device != a.codes.device):
        raise ValueError("out must be a contiguous bf16 [h, M, width] tensor with N = h * dk on the operands' device")
    d.epilogue = EPI_BIAS if bias is not None else EPI_NONE
    d.out_dtype, d.out, d.ldo = DT_BF16, out.data_ptr(), width
    d.heads, d.head_dim, d.head_col_off = h, dk, col_off
    d.flags = GEMM_OUT_HEADS
    _lib.check(_lib.load().vx_bsgemm(C.byref(d), _stream()), "vx_bsgemm")
    _count()
    del keep
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


def rowscale_linear(x2d: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """``x2d [M, K] @ W^T (+ bias)`` on the reference's per-row-scaled FP4 lane, fp32 out, in two
    launches: quantize the activation rows, then one GEMM whose epilogue applies the row and
    column scales and adds the bias.  The reference's ``DenseLinear.forward``
    (``veloxvoice/models/wenet/torch_conformer.py:251-266``) spends a pad copy, a cast, the
    quantizer, the GEMM, a slice and a bias add on the same result."""
    a = quantize(x2d, FMT_ROWSCALE, sf=False)
    b = _as_quantized_rowscale(wq, ws)
    if bias is None:
        return bsgemm(a, b, epilogue=EPI_NONE, out_dtype=torch.float32)
    if bias.dtype != torch.float32 or not bias.is_contiguous():
        bias = bias.float().contiguous()
    return bsgemm(a, b, epilogue=EPI_BIAS, bias=bias, out_dtype=torch.float32)


# ---- bf16 operator names of the reference, served by the quantized path -----------------------
# The reference's fused_qkv_wgmma / pwlin_glu are bf16 Hopper kernels whose sources do not build
# for sm_100a.  Here the same names quantize the activation and run one block-scaled GEMM with
# the bias (+ GLU) in its epilogue.  The weight is quantized once per (tensor, version) and kept
# in a small cache; the format is VELOXVOICE_QFORMAT (mx32 by default).

_WEIGHT_CACHE: "dict" = {}
_WEIGHT_CACHE_MAX = 256


def _qformat() -> int:
    import os

    name = os.environ.get("VELOXVOICE_QFORMAT", "mx32").lower()
    fmt = _fmt(name)
    if fmt not in (FMT_MX32, FMT_NV16, FMT_FP8_1X128):
        raise ValueError("VELOXVOICE_QFORMAT must be mx32, nv16 or fp8_1x128 for the bf16 operator names")
    return fmt


def _packed_weight(w: torch.Tensor, b: Optional[torch.Tensor], fmt: int, glu: bool):
    from .linear import PackedLinear

    key = (w.data_ptr(), tuple(w.shape), w.dtype, w._version, fmt, glu,
           None if b is None else (b.data_ptr(), b._version))
    hit = _WEIGHT_CACHE.get(key)
    if hit is None:
        if len(_WEIGHT_CACHE) >= _WEIGHT_CACHE_MAX:
            _WEIGHT_CACHE.pop(next(iter(_WEIGHT_CACHE)))
        hit = PackedLinear(w.float(), None if b is None else b.float(), fmt, glu=glu)
        _WEIGHT_CACHE[key] = hit
    return hit


def _quantized_activation(x2d: torch.Tensor, fmt: int) -> Quantized:
    return quantize(x2d, fmt, natural=fmt == FMT_FP8_1X128)


def _linear_supported(x, w, glu: bool) -> bool:
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.bfloat16):
        return False
    K = x.shape[-1]
    if w.dim() != 2 or w.shape[1] != K or K % 128 != 0:
        return False
    if glu:
        from .linear import glu_tile

        if w.shape[0] % glu_tile(_qformat()) != 0:
            return False
    return True


def fused_qkv_wgmma(x, w, b, out=None):
    """``out = x @ w^T + b`` in bf16 for the fused q|k|v projection
    (``veloxvoice/kernels/ops/cuda_ops.py:480-539``).  Returns ``None`` when the input is not a
    bf16 CUDA tensor or the shape is not supported, so the caller falls back to ``F.linear``
    exactly as with the reference; never compiles anything at call time."""
    if not _linear_supported(x, w, False):
        return None
    fmt = _qformat()
    x2 = x.reshape(-1, x.shape[-1])
    M, N = x2.shape[0], w.shape[0]
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=x.dtype)
    o2 = out.reshape(M, N)
    if o2.data_ptr() != out.data_ptr() or o2.stride(1) != 1:
        return None
    lin = _packed_weight(w, b, fmt, False)
    am = amax(x2) if fmt == FMT_NV16 else None
    lin(quantize(x2, fmt, natural=fmt == FMT_FP8_1X128, amax_t=am), out=o2)
    return out


def fused_qkv(x, w, bias, out=None):
    """x [M, K]; w [3N, K]; bias [3N] -> out [M, 3N] (``cuda_ops.py:292-304``; the reference's
    kernel is an fp32 GEMV for M <= 32).  bf16 inputs run on the quantized path; anything
    else is computed by ``F.linear`` in the input's dtype, like the reference's result."""
    r = fused_qkv_wgmma(x, w, bias, out)
    if r is not None:
        return r
    y = torch.nn.functional.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
    if out is not None:
        out.copy_(y)
        return out
    return y


def pwlin_glu(x, w, b, out=None):
    """``out = glu(x @ w^T + b)`` in bf16: value = first half of the channels, gate = second half
    (``cuda_ops.py:363-401``).  ``None`` for inputs the path does not take (not bf16 / not CUDA /
    K not a multiple of 128 / channel count not a multiple of the GLU tile)."""
    if not _linear_supported(x, w, True):
        return None
    fmt = _qformat()
    x2 = x.reshape(-1, x.shape[-1])
    M, Nh = x2.shape[0], w.shape[0] // 2
    if out is None:
        out = torch.empty(x.shape[:-1] + (Nh,), device=x.device, dtype=x.dtype)
    o2 = out.reshape(M, Nh)
    if o2.data_ptr() != out.data_ptr() or o2.stride(1) != 1:
        return None
    lin = _packed_weight(w, b, fmt, True)
    am = amax(x2) if fmt == FMT_NV16 else None
    lin(quantize(x2, fmt, natural=fmt == FMT_FP8_1X128, amax_t=am), out=o2)
    return out


# ---- model-side helper names (veloxvoice/models/wenet/nvfp4_linear.py) -------------------------

_E2M1_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5)


def _encode_codes(w: torch.Tensor) -> torch.Tensor:
    """float -> u8 E2M1 codes (sign << 3 | magnitude 0..6), ``nvfp4_linear.py:22-36``: the
    magnitude is the number of thresholds strictly exceeded by |w|, the sign bit is ``w < 0``."""
    edges = torch.tensor(_E2M1_THRESHOLDS, dtype=w.dtype if w.is_floating_point() else torch.float32, device=w.device)
    mag = torch.bucketize(w.abs().contiguous(), edges, right=False).to(torch.uint8)  # edges strictly below |w|
    return mag | ((w < 0).to(torch.uint8) << 3)


def pack_codes(c: torch.Tensor) -> torch.Tensor:
    """codes [R, K] -> packed u8 [R, K/2] on the GPU, even k in the low nibble (``nvfp4_linear.py:39-40``)."""
    lo, hi = c[:, 0::2] & 0xF, c[:, 1::2] & 0xF
    return (lo | (hi << 4)).to(torch.uint8).cuda()


def decode_codes(packed: torch.Tensor) -> torch.Tensor:
    """packed u8 [R, K/2] -> codes u8 [R, K] (``nvfp4_linear.py:103-107``)."""
    both = torch.stack((packed & 0xF, (packed >> 4) & 0xF), dim=-1)
    return both.reshape(packed.shape[0], packed.shape[1] * 2)


def ue8m0_from_scale(s) -> int:
    """Scalar scale -> biased exponent byte with the exponent truncated toward zero
    (``nvfp4_linear.py:43-49``; not the rule the quantize kernels use)."""
    import math

    if s <= 0.0:
        return 0x80
    return max(0, min(255, math.trunc(math.log2(s)) + 127))


def ue8m0_to_float(u) -> float:
    """``nvfp4_linear.py:52-53``."""
    return float(2.0 ** (int(u) - 127))


def quantize_and_gemm(x, wq, ws, P=1, C=8):
    """Quantize ``x`` per row, then the per-row-scaled GEMM (``nvfp4_linear.py:81-100``).  The
    reference quantizes on a side stream and joins with an event; both launches are stream
    ordered here, which gives the same result without the extra stream."""
    xq, xs = quantize_w(x)
    return dgx_mxfp4_gemm(xq, wq, xs, ws, P, C)


def reference_power_mel_log(re, im, mel, cmvn_mean, cmvn_istd):
    """fp32 formula of the filterbank projection (``veloxvoice/kernels/ops/cuda_ops.py:195-202``),
    on whatever device the inputs are; also what ``power_mel_log`` runs for shapes its kernel does
    not take, as the reference does with cuBLAS (``cuda_ops.py:138-148``)."""
    power = re.float() ** 2 + im.float() ** 2
    feat = (power @ mel.T).clamp_min(1.1920929e-7).log()
    if cmvn_mean is not None:
        feat = (feat - cmvn_mean) * cmvn_istd
    return feat


def power_mel_log_tf32(spec, mel, cmvn_mean=None, cmvn_istd=None):
    """Power spectrum -> mel GEMM -> log -> CMVN in one launch of ``vx_power_mel_log`` (tf32 operands on
    the tensor cores, fp32 accumulation), for any number of frames.  spec complex64 [T, F]
    (``torch.fft.rfft`` output), mel f32 [M, F], cmvn_mean / cmvn_istd f32 [M] or None -> f32 [T, M].
    Raises when the filterbank does not fit the kernel (``vx_power_mel_log_supported``)."""
    _require_cuda(spec, "spec")
    _require_cuda(mel, "mel")
    if spec.dim() != 2 or mel.dim() != 2 or spec.shape[1] != mel.shape[1]:
        raise ValueError(f"shapes: spec [T, F], mel [M, F]; got {tuple(spec.shape)} and {tuple(mel.shape)}")
    if not spec.is_complex():
        raise TypeError("spec must be complex (torch.fft.rfft output)")
    if (cmvn_mean is None) != (cmvn_istd is None):
        raise ValueError("cmvn_mean and cmvn_istd go together")
    if mel.device != spec.device:
        raise ValueError(f"mel is on {mel.device}, spec on {spec.device}")
    T, F = spec.shape
    M = mel.shape[0]
    lib = _lib.load()
    if not lib.vx_power_mel_log_supported(F, M):
        raise ValueError(f"a {M} x {F} filterbank does not fit the kernel (M <= 256, filterbank resident in shared memory)")
    ri = torch.view_as_real(spec.to(torch.complex64).contiguous())  # f32 [T, F, 2], interleaved
    melc = _rows2d(mel.float(), "mel")
    mean = istd = None
    if cmvn_mean is not None:
        mean, istd = cmvn_mean.float().contiguous(), cmvn_istd.float().contiguous()
        _check_vector(mean, "cmvn_mean", M, spec.device)
        _check_vector(istd, "cmvn_istd", M, spec.device)
    out = torch.empty((T, M), dtype=torch.float32, device=spec.device)
    rc = lib.vx_power_mel_log(ri.data_ptr(), T, F, F, melc.data_ptr(), M, melc.stride(0), _ptr(mean), _ptr(istd),
                              out.data_ptr(), M, _stream())
    _lib.check(rc, "vx_power_mel_log")
    _count()
    return out


def power_mel_log(spec, mel, cmvn_mean, cmvn_istd):
    """Signature and dispatch of the reference's ``power_mel_log``
    (``veloxvoice/kernels/ops/cuda_ops.py:95-135``): from 64 frames on, the tensor-core kernel
    (``power_mel_log_tf32``; the reference's takes M <= 80, this one M <= 256); below 64 frames, or
    for a filterbank the kernel does not take, the fp32 formula the reference runs through cuBLAS
    (``cuda_ops.py:138-148``), so short inputs stay fp32-grade as its tests expect
    (``tests/kernels/test_power_mel_log.py:80-88,180-203``)."""
    _require_cuda(spec, "spec")
    _require_cuda(mel, "mel")
    if spec.dim() == 2 and mel.dim() == 2 and spec.shape[0] >= 64 and _lib.load().vx_power_mel_log_supported(spec.shape[1], mel.shape[0]):
        return power_mel_log_tf32(spec, mel, cmvn_mean, cmvn_istd)
    return reference_power_mel_log(spec.real, spec.imag, mel.float(), cmvn_mean, cmvn_istd)


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

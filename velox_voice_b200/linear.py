"""Quantized linear layers: pre-packed weights + the model-side names of the reference.

* :class:`PackedLinear` -- a weight [N, K] quantized once (any format), bias kept in fp32;
  ``forward`` takes an already-quantized activation and runs one fused GEMM.
* :class:`DenseLinear` / :class:`Nvfp4Linear` / :func:`nvfp4_gemm` -- same constructor
  arguments, attributes and results as the reference's modules
  (``veloxvoice/models/wenet/torch_conformer.py:200-270``,
  ``veloxvoice/models/wenet/nvfp4_linear.py:128-168``), running on this library's kernels.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
from torch import nn

from . import ops
from .ops import (
    EPI_BIAS,
    EPI_BIAS_GLU,
    EPI_BIAS_RESIDUAL,
    EPI_BIAS_SWISH,
    EPI_NONE,
    FMT_BLK16_A,
    FMT_BLK16_B,
    Quantized,
)


def glu_tile(fmt) -> int:
    """Rows per GLU interleave tile for a format (the GEMM's tile width)."""
    from . import _lib

    return int(_lib.load().vx_glu_tile(ops._fmt(fmt)))


def glu_interleave_index(n_out: int, device=None, tile: int = 256) -> torch.Tensor:
    """Row order the GLU epilogue expects: per `tile` rows, tile/2 value rows then their gate rows."""
    h = n_out // 2
    half = tile // 2
    if h % half != 0:
        raise ValueError(f"GLU output width must be a multiple of {half}")
    a = torch.arange(h, device=device).view(-1, half)
    return torch.cat([a, a + h], dim=1).reshape(-1)


class PackedLinear:
    """Weight of one linear layer, quantized and laid out for the block-scaled GEMM.

    The packed codes and natural-layout scales follow the reference's weight-packing layout
    (u8 [N, K/2], low nibble = even k; ``triton_ops.py:82-89``); the SF-atom copy of the
    scales is a derived, internal layout made here once.
    """

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], fmt, *, glu: bool = False,
                 weight_amax: Optional[torch.Tensor] = None):
        fmt = ops._fmt(fmt)
        if weight.dim() != 2:
            raise ValueError("weight must be [N, K]")
        self.fmt_a = fmt
        self.fmt_b = FMT_BLK16_B if fmt == FMT_BLK16_A else fmt
        self.out_features, self.in_features = weight.shape
        self.glu = glu
        w = weight.detach()
        b = None if bias is None else bias.detach().float()
        if glu:
            idx = glu_interleave_index(self.out_features, w.device, glu_tile(fmt))
            w = w[idx]
            if b is not None:
                b = b[idx]
        self.q: Quantized = ops.quantize(w.contiguous(), self.fmt_b, natural=True, sf=True, amax_t=weight_amax)
        self.bias = None if b is None else b.contiguous()

    def forward(self, a: Quantized, *, act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
                alpha: float = 1.0, out_dtype=torch.bfloat16, out: Optional[torch.Tensor] = None,
                out_fmt=None, out_amax: Optional[torch.Tensor] = None):
        if self.glu:
            epi = EPI_BIAS_GLU
        elif residual is not None:
            epi = EPI_BIAS_RESIDUAL
        elif act == "swish":
            epi = EPI_BIAS_SWISH
        elif self.bias is not None:
            epi = EPI_BIAS
        else:
            epi = EPI_NONE
        return ops.bsgemm(a, self.q, epilogue=epi, bias=self.bias, residual=residual, alpha=alpha,
                          out_dtype=out_dtype, out=out, out_fmt=out_fmt, out_amax=out_amax)

    __call__ = forward

    def residual_ln_supported(self) -> bool:
        """Whether :meth:`residual_ln` covers this layer (MX32, 512 outputs, K a multiple of 256)."""
        return (not self.glu) and ops.residual_ln_supported(self.q.fmt, self.q.rows, self.q.k)

    def residual_ln(self, a: Quantized, *, residual: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
                    eps: float, alpha: float = 1.0, out: Optional[torch.Tensor] = None,
                    gamma2: Optional[torch.Tensor] = None, beta2: Optional[torch.Tensor] = None):
        """``x = alpha (a W^T + bias) + residual`` and ``ln_quantize(x, gamma, beta, eps)`` in one launch:
        ``(x, q)`` with the bits of the two separate calls.  With ``gamma2`` / ``beta2``: ``(LN(x), q)`` with
        ``q = ln_quantize(LN(x), gamma2, beta2)`` -- the end of a block (``ops.ln2_quantize``)."""
        return ops.bsgemm_residual_ln(a, self.q, bias=self.bias, residual=residual, gamma=gamma, beta=beta,
                                      eps=eps, alpha=alpha, out=out, gamma2=gamma2, beta2=beta2)

    def argmax(self, a: Quantized, *, keys: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None,
               return_max: bool = False, return_logp: bool = False):
        """First column of the row maximum of the bf16 result, without writing the result
        (``return_logp``: also the row's log-sum-exp and the winner's log-probability)."""
        if self.glu:
            raise ValueError("argmax head on a GLU layer")
        return ops.bsgemm_argmax(a, self.q, self.bias, keys=keys, ids=ids, return_max=return_max, return_logp=return_logp)


    def topk(self, a: Quantized, k: int = 5):
        """``torch.topk(log_softmax(logits), k)`` of the bf16 logits without writing them (the stream of the
        reference's prefix beam search): ``(logp [M, k], ids [M, k])``."""
        if self.glu:
            raise ValueError("top-k head on a GLU layer")
        return ops.bsgemm_topk(a, self.q, self.bias, k)


# --------------------------------------------------------------------------------------
# Reference-compatible modules


class DenseLinear(nn.Linear):
    """``DenseLinear`` of the reference model with the same ``precision`` switch.

    ``precision`` in ("nvfp4", "mxfp4") quantizes activations per row on the fly and runs the
    FP4 GEMM against the weight pre-quantized per row; anything else is ``F.linear``.  Padding
    of M and N to 128 (``torch_conformer.py:225-229,251-263``) is not needed by this
    library's kernel, so no padded copies are made; results equal the reference's slices.
    """

    def __init__(self, w, b=None):
        super().__init__(w.shape[1], w.shape[0], bias=b is not None)
        with torch.no_grad():
            self.weight.copy_(w)
            if b is not None:
                self.bias.copy_(b)
        self.precision = os.environ.get("VELOXVOICE_ASR_PRECISION", "fp32")
        self._wq = None
        self._ws = None
        self._w_bf16 = None
        self._w_N_actual = w.shape[0]

    def _prequantize_weight(self, precision):
        if precision in ("nvfp4", "mxfp4") and self._wq is None and self.weight.device.type == "cuda":
            w = self.weight.detach().float()
            self._wq, self._ws = ops.per_row_col_quantize(w)
            self._w_bf16 = w.to(torch.bfloat16)
            self._w_N_actual = self.weight.shape[0]

    def forward(self, x):
        precision = getattr(self, "precision", "fp32")
        if precision in ("nvfp4", "mxfp4"):
            orig_shape = x.shape
            x2 = x.reshape(-1, orig_shape[-1])
            if self._wq is None:
                self._prequantize_weight(precision)
            if x2.dtype not in (torch.float32, torch.bfloat16):
                x2 = x2.float()
            # quantize + one GEMM with the scales and the bias in its epilogue (fp32 out)
            out = ops.rowscale_linear(x2, self._wq, self._ws, None if self.bias is None else self.bias.detach())
            return out.view(*orig_shape[:-1], self.out_features)
        return torch.nn.functional.linear(x, self.weight, self.bias)


class Nvfp4Linear(nn.Module):
    """Pre-quantized weight, online activation quantization (``nvfp4_linear.py:128-158``)."""

    def __init__(self, in_features, out_features, bias=True, device=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        w = torch.randn(out_features, in_features, device=device, dtype=torch.bfloat16)
        wq, ws = ops.quantize_w(w)
        self.register_buffer("weight_q", wq)
        self.register_buffer("weight_s", ws)
        self.register_buffer("weight_bf16", ops._dequantize_to_bf16(wq, ws))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, device=device, dtype=torch.float32))
        else:
            self.bias = None

    def forward(self, x):
        orig_shape = x.shape
        x = x.reshape(-1, self.in_features)
        out = ops.rowscale_linear(x, self.weight_q, self.weight_s, self.bias)
        return out.view(*orig_shape[:-1], self.out_features)


def nvfp4_gemm(x, w, b=None):
    """x [M, K] @ w [N, K]^T with both sides quantized online (``nvfp4_linear.py:161-168``)."""
    wq, ws = ops.quantize_w(w)
    return ops.rowscale_linear(x, wq, ws, b)

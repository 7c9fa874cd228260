"""CPU restatement of the encoder's linear stack on the quantized path.  TEST INFRASTRUCTURE.

Same data flow as the reference model's block
(``veloxvoice/models/wenet/torch_conformer.py:705-713``: LN -> FFN with half-step residual,
LN -> q/k/v projections and ``lo``, LN -> pointwise conv + GLU and ``pw2``, LN -> FFN, final
LN; ``after_norm`` ``:745``; CTC head ``:810-814,945-949``) with every linear computed the way
the reference's FP4 lane defines it: quantize the activation, quantize the weight,
dequantize both, fp32 matmul (``tests/kernels/test_dgx_mxfp4_gemm.py:45-61``), add the bias
(``torch_conformer.py:265-266``).  As in the GPU stack, attention and the depthwise
convolution are left out: ``lo`` consumes the value projection, ``pw2`` the GLU output.

Tensors that the GPU path stores in bf16 (residual stream, q/k/v, GLU output, logits) are
rounded to bf16 at the same points; the FFN intermediate is re-quantized from fp32.
"""

from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from . import formats as F
from . import gemm as G


class OracleStack:
    def __init__(self, weights: Dict[str, np.ndarray], fmt: int, blocks: int, d_model: int = 512,
                 eps: float = 1e-5, amax: Optional[Dict[str, float]] = None, fuse_ffn: bool = True,
                 kernel_order: bool = False):
        self.w = {k: np.asarray(v, dtype=np.float32) for k, v in weights.items()}
        self.fmt = fmt
        self.blocks = blocks
        self.d = d_model
        self.eps = eps
        self.amax = amax or {}
        self.fuse_ffn = fuse_ffn
        # kernel_order: every product through gemm.gemm_kernel_order (the kernel's grouping of the
        # sum with exact group sums) instead of dequantize -> fp32 matmul; see that function
        self.kernel_order = kernel_order
        self._wd: Dict[str, np.ndarray] = {}
        self._wq: Dict[str, tuple] = {}

    # weight quantized then dequantized, once
    def _weight(self, key: str) -> np.ndarray:
        if key not in self._wd:
            q, s, g = F.quantize(self.w[key], self.fmt)
            self._wd[key] = F.dequantize(q, s, self.fmt, g)
        return self._wd[key]

    def _act(self, x: np.ndarray, key: str):
        kw = {}
        if self.fmt == F.FMT_NV16:
            kw["amax_t"] = np.float32(self.amax[key]) if key in self.amax else None
        q, s, g = F.quantize(x, self.fmt, **kw)
        if self.kernel_order:
            return (q, s, g)
        return F.dequantize(q, s, self.fmt, g)

    def _lin(self, xq, wkey: str, bkey: Optional[str]) -> np.ndarray:
        if self.kernel_order:
            if wkey not in self._wq:
                self._wq[wkey] = F.quantize(self.w[wkey], self.fmt)
            wq, ws, wg = self._wq[wkey]
            aq, asc, ag = xq
            y = G.gemm_kernel_order(self.fmt, aq, asc, wq, ws, ag, wg)
        else:
            y = G.matmul_f32(xq, self._weight(wkey))
        if bkey is not None:
            y = y + self.w[bkey][None, :]
        return y.astype(np.float32)

    def _ln(self, x: np.ndarray, key: str) -> np.ndarray:
        # the stack's activations are bf16 tensors: rows of 512 go through the half-warp-per-row kernel
        half = G.ln_half_rows(x.shape[1], True, self.fmt)
        return G.layernorm_ref(x, self.w[key + ".g"], self.w[key + ".b"], self.eps, half_rows=half)

    def _ffn(self, x: np.ndarray, b: str, ff: str, ln: str) -> np.ndarray:
        a = self._act(self._ln(x, b + ln), b + ln)
        h = G.silu(self._lin(a, b + ff + ".w1", b + ff + ".b1"))
        if not self.fuse_ffn:
            h = G.to_bf16(h)
        hq = self._act(h, b + ff + ".h")
        y = self._lin(hq, b + ff + ".w2", b + ff + ".b2")
        return G.to_bf16(x + np.float32(0.5) * y)

    def forward(self, x: np.ndarray, return_hidden: bool = False):
        """x: fp32 array of bf16-representable values [T, d]; returns logits (bf16 values as fp32)."""
        x = G.to_bf16(np.asarray(x, dtype=np.float32))
        d = self.d
        for i in range(self.blocks):
            b = f"b{i}."
            x = self._ffn(x, b, "ffm", "ln_ffm")
            a = self._act(self._ln(x, b + "ln_mha"), b + "ln_mha")
            qkv = G.to_bf16(self._lin(a, b + "qkv.w", b + "qkv.b"))
            ctx = self._act(qkv[:, 2 * d:], b + "ctx")
            x = G.to_bf16(x + self._lin(ctx, b + "lo.w", b + "lo.b"))
            a = self._act(self._ln(x, b + "ln_conv"), b + "ln_conv")
            z = self._lin(a, b + "pw1.w", b + "pw1.b")
            h = z.shape[1] // 2
            gl = G.to_bf16(z[:, :h] * G.sigmoid(z[:, h:]))
            x = G.to_bf16(x + self._lin(self._act(gl, b + "glu"), b + "pw2.w", b + "pw2.b"))
            x = self._ffn(x, b, "ff", "ln_ff")
            x = G.to_bf16(self._ln(x, b + "ln_final"))
        a = self._act(self._ln(x, "after"), "after")
        logits = G.to_bf16(self._lin(a, "ctc.w", "ctc.b"))
        return (logits, x) if return_hidden else logits


def cpu_linear_stack_fp32(weights: Dict[str, np.ndarray], x: np.ndarray, blocks: int, d_model: int = 512,
                          eps: float = 1e-5):
    """The reference's actual CPU lane: unquantized fp32 ``F.linear`` for every layer
    (``torch_conformer.py:270``; platform "cpu", ``veloxvoice/runtime/device.py:54``)."""
    import torch
    import torch.nn.functional as Fn

    w = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in weights.items()}
    x = torch.from_numpy(np.asarray(x, dtype=np.float32))
    d = d_model

    def ln(t, key):
        return Fn.layer_norm(t, (d,), w[key + ".g"], w[key + ".b"], eps)

    for i in range(blocks):
        b = f"b{i}."
        x = x + 0.5 * Fn.linear(Fn.silu(Fn.linear(ln(x, b + "ln_ffm"), w[b + "ffm.w1"], w[b + "ffm.b1"])), w[b + "ffm.w2"], w[b + "ffm.b2"])
        qkv = Fn.linear(ln(x, b + "ln_mha"), w[b + "qkv.w"], w[b + "qkv.b"])
        x = x + Fn.linear(qkv[:, 2 * d:], w[b + "lo.w"], w[b + "lo.b"])
        z = Fn.linear(ln(x, b + "ln_conv"), w[b + "pw1.w"], w[b + "pw1.b"])
        x = x + Fn.linear(Fn.glu(z, dim=1), w[b + "pw2.w"], w[b + "pw2.b"])
        x = x + 0.5 * Fn.linear(Fn.silu(Fn.linear(ln(x, b + "ln_ff"), w[b + "ff.w1"], w[b + "ff.b1"])), w[b + "ff.w2"], w[b + "ff.b2"])
        x = ln(x, b + "ln_final")
    return Fn.linear(ln(x, "after"), w["ctc.w"], w["ctc.b"]).numpy()

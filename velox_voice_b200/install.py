"""Drop this library's operators into an importable ``veloxvoice`` package.

``install()`` makes the reference's own import statements resolve to this library:

* ``veloxvoice.kernels.ops.triton_ops`` -> a module exposing ``per_row_col_quantize``,
  ``triton_quantize_w``, ``mxfp4_block_quantize``, ``mxfp4_dequant``, ``MXFP4_CODE_LUT``
  (the reference's module needs Triton and creates a CUDA tensor at import,
  ``veloxvoice/kernels/ops/triton_ops.py:132``);
* ``veloxvoice.kernels.ops.cuda_ops`` / ``veloxvoice.kernels.ops``: ``dgx_mxfp4_gemm``,
  ``dgx_mxfp4_blkscale_gemm``, ``mxfp4_gemm``, ``nvfp4_linear``, ``_dequantize_to_bf16`` are
  replaced (the reference's build of them raises off sm_121a, ``cuda_ops.py:591-597``), and
  ``qkv_pack`` (``cuda_ops.py:554-581``) runs on this library's kernel;
* ``veloxvoice.models.wenet.mxfp4_linear`` -> provides ``_pad16``, which
  ``DenseLinear._prequantize_weight`` imports (``torch_conformer.py:222-226``) from a module
  the reference tree does not contain;
* ``veloxvoice.models.wenet.nvfp4_linear``: ``quantize_w``, ``Nvfp4Linear``, ``nvfp4_gemm``,
  ``quantize_and_gemm`` and the pure-torch helpers ``_encode_codes``, ``pack_codes``,
  ``decode_codes``, ``ue8m0_from_scale``, ``ue8m0_to_float``, ``CODE_LUT``;
* ``power_mel_log`` / ``reference_power_mel_log`` (``cuda_ops.py:95-135,195-202``): the front-end's
  filterbank projection on the tcgen05 tf32 kernel (the reference's is an ``mma.sync`` build for
  sm_121a);
* the bf16 operator names ``fused_qkv``, ``fused_qkv_wgmma``, ``pwlin_glu`` (the reference's
  builds of the last two are sm_90a sources, ``cuda_ops.py:363-401,480-539``) run quantize + one
  GEMM with the bias (+ GLU) in its epilogue and keep the ``Tensor | None`` convention.

After that ``Velox.load(..., kernel_precision="mxfp4")`` / ``transcribe_pcm`` run their FP4
lane on a B200 without any change to the reference's files.
"""

from __future__ import annotations

import importlib
import sys
import types

from . import linear, ops

_TRITON_OPS = "veloxvoice.kernels.ops.triton_ops"
_CUDA_OPS = "veloxvoice.kernels.ops.cuda_ops"
_OPS_PKG = "veloxvoice.kernels.ops"
_MXFP4_LINEAR = "veloxvoice.models.wenet.mxfp4_linear"
_NVFP4_LINEAR = "veloxvoice.models.wenet.nvfp4_linear"

GEMM_NAMES = ("dgx_mxfp4_gemm", "dgx_mxfp4_blkscale_gemm", "mxfp4_gemm", "nvfp4_linear", "_dequantize_to_bf16",
              "qkv_pack", "fused_qkv", "fused_qkv_wgmma", "pwlin_glu", "power_mel_log", "reference_power_mel_log")
# names of veloxvoice.kernels.ops (the package re-exports these; the reference's own tests import them from there)
OPS_PKG_NAMES = tuple(n for n in GEMM_NAMES if n != "_dequantize_to_bf16")
QUANT_NAMES = ("per_row_col_quantize", "triton_quantize_w", "mxfp4_block_quantize", "mxfp4_dequant")


def _lazy_lut():
    import torch

    return torch.tensor(ops._E2M1_LUT, device="cuda" if torch.cuda.is_available() else "cpu")


def make_triton_ops_module() -> types.ModuleType:
    m = types.ModuleType(_TRITON_OPS)
    m.__doc__ = "velox_voice_b200 replacement of the reference's Triton quantizers"
    for n in QUANT_NAMES:
        setattr(m, n, getattr(ops, n))
    m.MXFP4_CODE_LUT = _lazy_lut()
    return m


def make_mxfp4_linear_module() -> types.ModuleType:
    m = types.ModuleType(_MXFP4_LINEAR)
    m._pad16 = ops._pad16
    return m


def make_nvfp4_linear_module() -> types.ModuleType:
    m = types.ModuleType(_NVFP4_LINEAR)
    m.BLOCK = 16
    m.CODE_LUT = _lazy_lut()
    m.quantize_w = ops.quantize_w
    m._encode_codes = ops._encode_codes
    m.pack_codes = ops.pack_codes
    m.decode_codes = ops.decode_codes
    m.ue8m0_from_scale = ops.ue8m0_from_scale
    m.ue8m0_to_float = ops.ue8m0_to_float
    m.quantize_and_gemm = ops.quantize_and_gemm
    m.Nvfp4Linear = linear.Nvfp4Linear
    m.nvfp4_gemm = linear.nvfp4_gemm
    m.dgx_mxfp4_gemm = ops.dgx_mxfp4_gemm
    m.per_row_col_quantize = ops.per_row_col_quantize
    m._dequantize_impl = ops._dequantize_to_bf16
    m.dequantize_w = ops._dequantize_to_bf16
    m.unquantize_w = ops._dequantize_to_bf16
    return m


def install(patch_modules: bool = True) -> dict:
    """Install the replacements; returns {module name: module}.  Idempotent.

    Call before the first ``import veloxvoice.kernels.ops`` (or at any later time: already
    imported modules get their attributes replaced too).
    """
    done = {}
    sys.modules[_TRITON_OPS] = done[_TRITON_OPS] = make_triton_ops_module()
    sys.modules[_MXFP4_LINEAR] = done[_MXFP4_LINEAR] = make_mxfp4_linear_module()
    sys.modules[_NVFP4_LINEAR] = done[_NVFP4_LINEAR] = make_nvfp4_linear_module()
    if patch_modules:
        for name in (_CUDA_OPS, _OPS_PKG):
            try:
                mod = importlib.import_module(name)
            except ImportError:
                continue  # no veloxvoice on this machine: the replacement modules still stand
            for n in (GEMM_NAMES if name == _CUDA_OPS else OPS_PKG_NAMES):
                setattr(mod, n, getattr(ops, n))
            if name == _OPS_PKG:
                for n in QUANT_NAMES:
                    setattr(mod, n, getattr(ops, n))
            done[name] = mod
        for parent, child in ((_OPS_PKG, "triton_ops"), ("veloxvoice.models.wenet", "mxfp4_linear"),
                              ("veloxvoice.models.wenet", "nvfp4_linear")):
            pm = sys.modules.get(parent)
            if pm is not None:
                setattr(pm, child, sys.modules[f"{parent}.{child}"])
    return done

"""velox_voice_b200 -- B200 (sm_100a) quantized-linear path for the Velox Voice encoder.

A thin PyTorch host layer over ``libvelox_b200.so`` (C ABI, ``include/velox_b200.h``):
activation quantize/pack fused behind LayerNorm, tcgen05 block-scaled FP4 / FP8 GEMMs with
fused bias / Swish / GLU / residual epilogues, and frame-sharded multi-GPU execution.
"""

import importlib

__all__ = ["ops", "linear", "stack", "install", "build"]


def __getattr__(name):
    if name in __all__:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)

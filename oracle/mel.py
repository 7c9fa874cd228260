"""TEST INFRASTRUCTURE: CPU restatement of the front-end's filterbank projection.

``out[t, m] = (log(max(sum_f (re^2 + im^2)[t, f] * mel[m, f], 2^-23)) - mean[m]) * istd[m]``

* ``power_mel_log_fp32``: the reference's fp32 formula (``veloxvoice/kernels/ops/cuda_ops.py:195-202``,
  ``reference_power_mel_log``; the cuBLAS lane ``cuda_ops.py:138-148`` is the same arithmetic).
* ``power_mel_log_tf32``: what its tensor-core kernel computes
  (``veloxvoice/kernels/csrc/dgx/block/nv_block_power_mel_log.h:35-190``), as the reference's own test
  restates it (``tests/kernels/test_power_mel_log.py:41-72``): power in fp32 (two rounded squares, one
  rounded add), both operands truncated to tf32 (low 13 mantissa bits dropped), products summed --
  here in float64 and rounded once, so the result carries no summation-order noise of its own.

Pinned by ``tests/golden/mel.npz``: outputs of the reference's ``reference_power_mel_log`` and of its
test's ``emulated_power_mel_log`` on seeded inputs (``tests/golden/make_golden.py``).  Only tests,
the smoke check and the CPU-baseline leg of the benchmark may import this module.
"""

from __future__ import annotations

import numpy as np

LOG_FLOOR = np.float32(1.1920929e-7)


def tf32_rz(x: np.ndarray) -> np.ndarray:
    """fp32 -> tf32 by truncation (``tests/kernels/test_power_mel_log.py:41-44``)."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def power(spec: np.ndarray) -> np.ndarray:
    """|spec|^2 as ``spec.real**2 + spec.imag**2`` in fp32 (``cuda_ops.py:142``)."""
    re = np.ascontiguousarray(spec.real, dtype=np.float32)
    im = np.ascontiguousarray(spec.imag, dtype=np.float32)
    return (re * re + im * im).astype(np.float32)


def _finish(acc: np.ndarray, mean, istd) -> np.ndarray:
    out = np.log(np.maximum(acc.astype(np.float32), LOG_FLOOR)).astype(np.float32)
    if mean is not None:
        out = ((out - np.asarray(mean, np.float32)[None, :]) * np.asarray(istd, np.float32)[None, :]).astype(np.float32)
    return out


def power_mel_log_fp32(spec, mel, mean=None, istd=None) -> np.ndarray:
    acc = power(spec).astype(np.float64) @ np.asarray(mel, np.float32).astype(np.float64).T
    return _finish(acc, mean, istd)


def power_mel_log_tf32(spec, mel, mean=None, istd=None) -> np.ndarray:
    acc = tf32_rz(power(spec)).astype(np.float64) @ tf32_rz(np.asarray(mel, np.float32)).astype(np.float64).T
    return _finish(acc, mean, istd)


def mel_filterbank(F: int, M: int, seed: int = 0) -> np.ndarray:
    """A non-negative triangular filterbank [M, F] with seeded, uneven centre spacing (the production
    regime of ``tests/kernels/test_power_mel_log.py:75-80``: no cancellation in the sum)."""
    rng = np.random.default_rng(seed)
    edges = np.sort(rng.uniform(0, F - 1, M + 2)).astype(np.float64)
    edges[0], edges[-1] = 0.0, F - 1.0
    f = np.arange(F, dtype=np.float64)[None, :]
    lo, ce, hi = edges[:-2, None], edges[1:-1, None], edges[2:, None]
    up = (f - lo) / np.maximum(ce - lo, 1e-3)
    dn = (hi - f) / np.maximum(hi - ce, 1e-3)
    return np.maximum(0.0, np.minimum(up, dn)).astype(np.float32)

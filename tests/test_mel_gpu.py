"""The filterbank projection (``vx_power_mel_log``, tcgen05 ``kind::tf32``) against the CPU oracle
and the reference-generated golden outputs."""

import os

import numpy as np
import pytest
import torch

from oracle import mel as ML

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from velox_voice_b200 import ops as o

    return o


def _run(ops, spec, bank, mean=None, istd=None):
    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return ops.power_mel_log_tf32(t(spec), t(bank), t(mean), t(istd)).cpu().numpy()


def _spec(T, F, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return ((rng.standard_normal((T, F)) + 1j * rng.standard_normal((T, F))) * scale).astype(np.complex64)


def test_golden_cases(ops, golden_dir):
    """Reference outputs (fp32 formula and the reference test's tf32 emulation) on seeded inputs."""
    g = np.load(os.path.join(golden_dir, "mel.npz"))
    for name in sorted({k[:-5] for k in g.files if k.endswith("_spec")}):
        sp = g[f"{name}_spec"]
        spec = (sp[..., 0] + 1j * sp[..., 1]).astype(np.complex64)
        bank = g[f"{name}_mel"]
        mean = g[f"{name}_mean"] if f"{name}_mean" in g.files else None
        istd = g[f"{name}_istd"] if mean is not None else None
        out = _run(ops, spec, bank, mean, istd)
        ref = g[f"{name}_tf32"]
        assert out.shape == ref.shape and out.dtype == np.float32 and np.isfinite(out).all()
        if (bank >= 0).all():
            d = np.abs(out - ref).max()
            print(f"[{name}] max |log diff| vs the reference's tf32 emulation {d:.3g}, vs its fp32 formula {np.abs(out - g[f'{name}_fp32']).max():.3g}")
            assert d < 1e-5
            assert np.abs(out - g[f"{name}_fp32"]).max() < 5e-3  # the reference's bound for this regime
        else:
            lin = np.abs(np.exp(out.astype(np.float64)) - np.exp(ref.astype(np.float64))).max()
            ok = ref > -9.0
            q = np.quantile(np.abs(out - ref)[ok], 0.999)
            print(f"[{name}] pre-log max abs diff {lin:.3g}, 99.9th pct |log diff| {q:.3g}")
            assert q < 5e-3


@pytest.mark.parametrize("T,F,M", [(1, 64, 1), (64, 257, 80), (98, 129, 64), (127, 257, 80), (129, 201, 80), (2048, 257, 80),
                                   (300, 513, 80), (515, 257, 128), (260, 100, 256), (40000, 257, 80)])
def test_non_negative_filterbank_matches_the_oracle(ops, T, F, M):
    """No cancellation in the sum, so the tensor core's summation order is invisible: the kernel must
    sit on the oracle's tf32-truncated product (exact accumulation) to fp32 rounding of the log."""
    spec = _spec(T, F, seed=T + F, scale=3.0)
    bank = ML.mel_filterbank(F, M, seed=M)
    rng = np.random.default_rng(1)
    mean, istd = (rng.standard_normal(M).astype(np.float32), (rng.random(M) + 0.5).astype(np.float32)) if T % 2 else (None, None)
    out = _run(ops, spec, bank, mean, istd)
    ref = ML.power_mel_log_tf32(spec, bank, mean, istd)
    assert out.shape == (T, M)
    d = np.abs(out - ref).max()
    assert d < 2e-5, d
    assert np.abs(out - ML.power_mel_log_fp32(spec, bank, mean, istd)).max() < 5e-3


def test_random_sign_filterbank_by_the_reference_criterion(ops):
    """tests/kernels/test_power_mel_log.py:90-116: pre-log absolute error everywhere, 99.9th percentile of the
    log error where the value is meaningful."""
    for seed, T, F, M in [(42, 128, 257, 80), (1, 256, 513, 80), (7, 2048, 257, 80), (3, 98, 129, 64)]:
        rng = np.random.default_rng(seed)
        spec = _spec(T, F, seed)
        bank = rng.standard_normal((M, F)).astype(np.float32)
        out = _run(ops, spec, bank)
        ref = ML.power_mel_log_tf32(spec, bank)
        lin = np.abs(np.exp(out.astype(np.float64)) - np.exp(ref.astype(np.float64))).max()
        assert lin < 0.35
        ok = ref > -9.0
        assert np.quantile(np.abs(out - ref)[ok], 0.999) < 5e-3


def test_floor_large_values_and_unsupported_shapes(ops):
    # silence: every bin zero -> log of the 2^-23 floor; loud input stays finite
    bank = ML.mel_filterbank(257, 80, 0)
    out = _run(ops, np.zeros((70, 257), np.complex64), bank)
    assert np.abs(out - np.log(np.float32(1.1920929e-7))).max() < 2e-6
    assert np.isfinite(_run(ops, _spec(128, 257, 3, scale=100.0), np.random.default_rng(3).standard_normal((80, 257)).astype(np.float32))).all()
    # the reference's dispatch: a filterbank the kernel does not take, or fewer than 64 frames, goes through the
    # fp32 formula (its cuBLAS lane); the kernel entry itself refuses the filterbank
    spec, wide = _spec(80, 64, 9), np.abs(np.random.default_rng(9).standard_normal((300, 64))).astype(np.float32)
    tc = lambda a: torch.from_numpy(a).cuda()
    assert np.abs(ops.power_mel_log(tc(spec), tc(wide), None, None).cpu().numpy() - ML.power_mel_log_fp32(spec, wide)).max() < 1e-4
    with pytest.raises(ValueError, match="does not fit"):
        ops.power_mel_log_tf32(tc(spec), tc(wide))
    short = _spec(20, 257, 2)
    assert np.abs(ops.power_mel_log(tc(short), tc(bank), None, None).cpu().numpy() - ML.power_mel_log_fp32(short, bank)).max() < 1e-5
    # empty input
    assert tuple(ops.power_mel_log_tf32(torch.zeros(0, 257, dtype=torch.cfloat, device="cuda"), tc(bank)).shape) == (0, 80)
    # a strided view of a longer spectrum (rfft output sliced in time)
    full = tc(_spec(200, 257, 4))
    assert torch.equal(ops.power_mel_log(full[::2], tc(bank), None, None), ops.power_mel_log(full[::2].contiguous(), tc(bank), None, None))

"""The CPU oracle against the bytes the reference's own code produced.

``tests/golden/*.npz`` were written by ``tests/golden/make_golden.py``, which runs the
reference's Triton quantizers (CPU interpreter), ``mxfp4_dequant``, ``_dequantize_to_bf16``,
``_encode_codes`` / ``decode_codes`` and the GEMM definition of its kernel test.
"""

import os

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import gemm as G
from oracle import mel as ML


def _cases(npz, suffix):
    return sorted({k[: -len(suffix)] for k in npz.files if k.endswith(suffix)})


@pytest.fixture(scope="module")
def rowscale(golden_dir):
    return np.load(os.path.join(golden_dir, "rowscale.npz"))


@pytest.fixture(scope="module")
def blk16(golden_dir):
    return np.load(os.path.join(golden_dir, "blk16.npz"))


@pytest.fixture(scope="module")
def gemm(golden_dir):
    return np.load(os.path.join(golden_dir, "gemm_rowscale.npz"))


def test_rowscale_bytes_match_reference(rowscale):
    names = _cases(rowscale, "_x")
    assert len(names) >= 7
    for n in names:
        q, s = F.quantize_rowscale(rowscale[n + "_x"])
        assert np.array_equal(q, rowscale[n + "_q"]), n
        assert np.array_equal(s, rowscale[n + "_s"]), n


def test_rowscale_zero_row_scale_byte(rowscale):
    # all-zero row: s = 1e-6 -> ceil(log2) = -19 -> byte 108
    x = rowscale["edge_x"]
    zero_rows = np.nonzero(np.abs(x).max(axis=1) == 0)[0]
    assert len(zero_rows) >= 1
    assert (rowscale["edge_s"][zero_rows] == 108).all()
    _, s = F.quantize_rowscale(np.zeros((2, 64), np.float32))
    assert (s == 108).all()


def test_rowscale_dequant_matches_reference(rowscale):
    for n in _cases(rowscale, "_x"):
        d = F.dequant_rowscale(rowscale[n + "_q"], rowscale[n + "_s"])
        got = torch.from_numpy(d).bfloat16().float().numpy()
        assert np.array_equal(got, rowscale[n + "_deq_bf16_as_f32"]), n


def test_blk16_bytes_match_reference(blk16):
    names = _cases(blk16, "_x")
    assert len(names) >= 5
    for n in names:
        for mode in "AB":
            q, s = F.quantize_blk16(blk16[n + "_x"], mode)
            assert np.array_equal(q, blk16[f"{n}_{mode}_q"]), (n, mode)
            assert np.array_equal(s, blk16[f"{n}_{mode}_s"]), (n, mode)
            d = F.dequant_blk16(blk16[f"{n}_{mode}_q"], blk16[f"{n}_{mode}_s"], mode)
            assert np.array_equal(d, blk16[f"{n}_{mode}_deq"]), (n, mode)


def test_e2m1_helpers_match_reference(gemm):
    assert np.array_equal(F.e2m1_encode(gemm["enc_in"]), gemm["enc_out"])
    assert np.array_equal(F.unpack_codes(gemm["dec_in"]), gemm["dec_out"])
    assert np.array_equal(F.e2m1_decode(F.unpack_codes(gemm["dec_in"])), gemm["unpack_out"])
    # largest magnitude code emitted is 6, ties go down
    assert F.e2m1_encode(np.array([6.0, 100.0], np.float32)).tolist() == [6, 6]
    assert F.e2m1_encode(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5], np.float32)).tolist() == [0, 1, 2, 3, 4, 5]
    assert F.e2m1_encode(np.array([-0.0, -1e-30], np.float32)).tolist() == [0, 8]


def test_gemm_definition_matches_reference(gemm):
    for seed in (0, 1, 2):
        xq, xs = F.quantize_rowscale(gemm[f"gemm{seed}_x"])
        wq, ws = F.quantize_rowscale(gemm[f"gemm{seed}_w"])
        assert np.array_equal(xq, gemm[f"gemm{seed}_xq"]) and np.array_equal(xs, gemm[f"gemm{seed}_xs"])
        assert np.array_equal(wq, gemm[f"gemm{seed}_wq"]) and np.array_equal(ws, gemm[f"gemm{seed}_ws"])
        ref = G.gemm_rowscale_ref(xq, wq, xs, ws)
        # exact: E2M1 products are multiples of 0.25 and the partial sums fit 24 bits
        assert np.array_equal(ref, gemm[f"gemm{seed}_ref"]), seed


@pytest.fixture(scope="module")
def mel(golden_dir):
    return np.load(os.path.join(golden_dir, "mel.npz"))


def _mel_case(npz, name):
    sp = npz[f"{name}_spec"]
    spec = (sp[..., 0] + 1j * sp[..., 1]).astype(np.complex64)
    mean = npz[f"{name}_mean"] if f"{name}_mean" in npz.files else None
    istd = npz[f"{name}_istd"] if mean is not None else None
    return spec, npz[f"{name}_mel"], mean, istd


def test_filterbank_projection_matches_reference(mel):
    """oracle/mel.py against outputs of the reference's fp32 formula (``reference_power_mel_log``) and
    of its test's tf32 emulation (``emulated_power_mel_log``).  A non-negative filterbank has no
    cancellation: fp32-grade agreement.  A random-sign filterbank is compared the way the reference's
    own test compares (pre-log absolute error, 99.9th percentile of the log error on meaningful values,
    tests/kernels/test_power_mel_log.py:90-116), with bounds 100x tighter than its kernel's."""
    for name in _cases(mel, "_spec"):
        spec, bank, mean, istd = _mel_case(mel, name)
        assert np.array_equal(ML.tf32_rz(bank), mel[f"{name}_rz_bits"])
        for kind, fn in (("fp32", ML.power_mel_log_fp32), ("tf32", ML.power_mel_log_tf32)):
            ref, out = mel[f"{name}_{kind}"], fn(spec, bank, mean, istd)
            assert out.shape == ref.shape and out.dtype == np.float32
            if (bank >= 0).all():
                assert np.abs(out - ref).max() < 2e-6, (name, kind)
            else:
                scale = 1.0 if istd is None else float(np.max(istd))
                lin = np.abs(np.exp(out.astype(np.float64)) - np.exp(ref.astype(np.float64)))
                ok = ref > -9.0
                assert lin.max() < 3.5e-3 * max(1.0, float(np.exp(ref).max()) * 1e-3), (name, kind)
                assert np.quantile(np.abs(out - ref)[ok], 0.999) < 5e-4 * scale, (name, kind)

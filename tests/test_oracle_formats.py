"""Properties of the formats the reference has no code for (mx32, nv16, fp8_1x128) and of the
oracle's building blocks."""

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import gemm as G


def test_ceil_log2_exact():
    v = np.array([1.0, 1.0000001, 0.5, 0.75, 2.0, 3.0, 1e-6, 2.0**-19, 2.0**100], np.float32)
    assert F.ceil_log2_f32(v).tolist() == [0, 1, -1, 0, 1, 2, -19, -19, 100]


def test_e4m3_against_torch_cast():
    rng = np.random.default_rng(0)
    v = (rng.standard_normal(100000) * 10.0 ** rng.uniform(-4, 3, 100000)).astype(np.float32)
    v = np.concatenate([v, np.array([0, 448, 449, 1e9, -1e9, 2**-9, 2**-10, 1.5 * 2**-10, 17.0, 18.0, 19.0], np.float32)])
    want = torch.from_numpy(np.clip(v, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(F.e4m3_encode(v), want)
    allb = np.arange(256, dtype=np.uint8)
    d = F.e4m3_decode(allb)
    t = torch.from_numpy(allb).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(d, nan=1e9), np.nan_to_num(t, nan=1e9))
    ok = ~np.isnan(d)
    assert np.array_equal(F.e4m3_encode(d[ok]) & 0x7F, allb[ok] & 0x7F)  # round trip (+-0 aside)


@pytest.mark.parametrize("fmt", [F.FMT_ROWSCALE, F.FMT_BLK16_A, F.FMT_BLK16_B, F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128])
def test_quantize_dequantize_error_bound(fmt):
    rng = np.random.default_rng(fmt)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    q, s, g = F.quantize(x, fmt)
    d = F.dequantize(q, s, fmt, g)
    assert d.shape == x.shape
    if fmt == F.FMT_FP8_1X128:
        assert np.abs(d - x).max() <= np.abs(x).max() * 2.0**-4
    else:
        # E2M1 with the scale chosen so that |q| <= 6 (6.5 after E4M3 scale rounding): the
        # magnitude cap at code 6 (= 4.0) bounds the error by a third of the block maximum
        assert np.abs(d - x).max() <= np.abs(x).max() * 0.36


def test_largest_code_is_six_so_requantizing_is_not_idempotent():
    # The reference's encoder never emits code 7 (6.0): a row whose maximum lands on code 5
    # (3.0) is rescaled by half on the next pass and its maximum saturates at 4.0.
    x = np.array([[3.4, 1.0] + [0.0] * 30], np.float32)
    q, s = F.quantize_rowscale(x)
    d = F.dequant_rowscale(q, s)
    assert d[0, 0] == 3.0 and s[0] == 127
    q2, s2 = F.quantize_rowscale(d)
    assert s2[0] == 126 and F.dequant_rowscale(q2, s2)[0, 0] == 2.0


def test_mx32_is_rowscale_rule_per_block():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((16, 128)).astype(np.float32)
    q, s = F.quantize_mx32(x)
    for kb in range(4):
        qb, sb = F.quantize_rowscale(x[:, 32 * kb : 32 * kb + 32])
        assert np.array_equal(q[:, 16 * kb : 16 * kb + 16], qb)
        assert np.array_equal(s[:, kb], sb)


def test_nv16_zero_and_scale_rules():
    x = np.zeros((4, 64), np.float32)
    q, s, g = F.quantize_nv16(x)
    assert g == np.float32(1.0) and not q.any() and not s.any()
    x[1, 3] = 2688.0
    q, s, g = F.quantize_nv16(x)
    assert g == np.float32(1.0)
    assert s[1, 0] == F.e4m3_encode(np.array([448.0]))[0]  # block amax / (6 g) = 448
    assert (q[1, 1] >> 4) == 6  # element 3 -> |q| = 6 -> code 6
    assert not s[0].any() and not q[0].any()


def test_fp8_zero_block_scale_is_one():
    x = np.zeros((2, 256), np.float32)
    x[0, 130] = -3.0
    q, s = F.quantize_fp8_1x128(x)
    assert s[0, 0] == 1.0 and s[1, 0] == 1.0 and s[1, 1] == 1.0
    assert s[0, 1] == np.float32(3.0) / np.float32(448.0)
    d = F.dequant_fp8_1x128(q, s)
    assert abs(d[0, 130] + 3.0) < 1e-6


def test_sf_atoms_layout():
    R, nk = 300, 10
    s = (np.arange(R * nk) % 251).astype(np.uint8).reshape(R, nk)
    a = F.sf_atoms(s)
    assert a.shape == (3, 3, 512)
    for r, kb in [(0, 0), (31, 3), (32, 0), (127, 7), (128, 9), (299, 5)]:
        off = (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4
        assert a[r // 128, kb // 4, off] == s[r, kb]
    assert a[2, 2, (299 % 32) * 16 + ((299 // 32) % 4) * 4 + 2] == 0  # kb 10: padding
    assert a[2, 0, (45 % 32) * 16 + (1) * 4] == 0  # row 301: padding


def test_layernorm_ref_close_to_torch():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((33, 512)).astype(np.float32) * 3 + 1
    g = rng.standard_normal(512).astype(np.float32)
    b = rng.standard_normal(512).astype(np.float32)
    y = G.layernorm_ref(x, g, b, 1e-5)
    t = torch.nn.functional.layer_norm(torch.from_numpy(x), (512,), torch.from_numpy(g), torch.from_numpy(b), 1e-5).numpy()
    assert np.abs(y - t).max() < 1e-4  # the reference's own LayerNorm tolerance
    # the half-warp-per-row order of the 512-element bf16 lanes: same formula, other summation tree
    yh = G.layernorm_ref(x, g, b, 1e-5, half_rows=True)
    assert np.abs(yh - t).max() < 1e-4 and np.abs(yh - y).max() < 1e-5
    assert G.ln_half_rows(512, True, F.FMT_MX32) and G.ln_half_rows(512, True) and not G.ln_half_rows(512, False, F.FMT_MX32)
    assert not G.ln_half_rows(1024, True, F.FMT_MX32) and not G.ln_half_rows(512, True, F.FMT_ROWSCALE)


def test_layernorm_ref_half_rows_is_the_cluster_exchange_order():
    """The fused residual GEMM + LayerNorm kernel (two CTAs of 256 columns, csrc/vx_gemm_ln.cu) sums a row like this:
    block j of 32 columns accumulates its four 8-column pieces in the order (c + (j >> 1)) & 3 into an even and an odd
    sum (squares by fused multiply-add), adds the two, and every thread then combines the 16 block sums as entries
    (j, j + 8) first, then strides 4, 2, 1.  Restated here independently: the statistics, and so the output, are those
    of ``layernorm_ref(half_rows=True)`` bit for bit."""
    rng = np.random.default_rng(5)
    M = 64
    x = G.to_bf16(rng.standard_normal((M, 512)).astype(np.float32) * 3.0 + 0.7)
    g = (1.0 + 0.2 * rng.standard_normal(512)).astype(np.float32)
    b = (0.1 * rng.standard_normal(512)).astype(np.float32)
    f32 = np.float32
    S = np.zeros((M, 16), f32)
    Q = np.zeros((M, 16), f32)
    for j in range(16):
        se, so, qe, qo = (np.zeros(M, f32) for _ in range(4))
        for c in range(4):
            p0 = 32 * j + 8 * ((c + (j >> 1)) & 3)
            for e in range(4):
                ve, vo = x[:, p0 + 2 * e], x[:, p0 + 2 * e + 1]
                se, so = (se + ve).astype(f32), (so + vo).astype(f32)
                qe, qo = G.fma32(ve, ve, qe), G.fma32(vo, vo, qo)
        S[:, j], Q[:, j] = (se + so).astype(f32), (qe + qo).astype(f32)
    for o in (8, 4, 2, 1):
        S = (S[:, :o] + S[:, o:2 * o]).astype(f32)
        Q = (Q[:, :o] + Q[:, o:2 * o]).astype(f32)
    mean = (S[:, 0] * f32(1.0 / 512.0)).astype(f32)
    ex2 = (Q[:, 0] * f32(1.0 / 512.0)).astype(f32)
    var = np.maximum(G.fma32(-mean, mean, ex2), f32(0))
    rstd = G.rsqrt32((var + f32(1e-5)).astype(f32))
    nmr = ((-mean) * rstd).astype(f32)
    y = G.fma32(G.fma32(x, rstd[:, None], nmr[:, None]), g[None, :], b[None, :])
    assert np.array_equal(y.view(np.uint32), G.layernorm_ref(x, g, b, 1e-5, half_rows=True).view(np.uint32))


def test_glu_interleave_is_a_permutation():
    idx = G.glu_interleave_rows(1024)
    assert sorted(idx.tolist()) == list(range(1024))
    assert idx[:64].tolist() == list(range(64)) and idx[64:128].tolist() == list(range(512, 576))


def test_epilogue_ref_shapes():
    acc = np.ones((4, 8), np.float32)
    assert G.epilogue_ref(acc, G.EPI_BIAS_GLU, np.zeros(8, np.float32)).shape == (4, 4)
    r = G.epilogue_ref(acc, G.EPI_BIAS_RESIDUAL, np.ones(8, np.float32), np.full((4, 8), 3.0, np.float32), 0.5)
    assert np.allclose(r, 4.0)

"""CUDA quantize / pack kernels (through the C ABI) against the CPU oracle and the reference's
golden bytes.  Everything here is bit-exact: packed codes, scale bytes, fp32 scales."""

import os

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import gemm as G

pytestmark = pytest.mark.gpu

ALL_FMTS = [F.FMT_ROWSCALE, F.FMT_BLK16_A, F.FMT_BLK16_B, F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128]


@pytest.fixture(scope="module")
def ops():
    from velox_voice_b200 import ops as o

    return o


def _natural_as_rows(fmt, s):
    """Natural-layout scales -> [R, nblocks] (what sf_atoms expects)."""
    if fmt == F.FMT_BLK16_A:
        return np.repeat(np.ascontiguousarray(s.T), 2, axis=0)
    if fmt == F.FMT_BLK16_B:
        return np.ascontiguousarray(s.T)
    return s


def _check(ops, x, fmt, **kw):
    q = ops.quantize(x, fmt, **kw)
    torch.cuda.synchronize()
    xo = x.float().cpu().numpy()
    okw = {}
    if fmt == F.FMT_NV16 and kw.get("amax_t") is not None:
        okw["amax_t"] = float(kw["amax_t"].item())
    oq, os_, og = F.quantize(xo, fmt, **okw)
    assert np.array_equal(q.codes.cpu().numpy(), oq), f"codes differ (fmt {fmt}, shape {tuple(x.shape)})"
    assert np.array_equal(q.scales.cpu().numpy(), os_), f"scales differ (fmt {fmt})"
    if fmt == F.FMT_NV16:
        assert np.float32(q.amax.item()) == np.abs(xo).max() or okw
    if q.sf is not None:
        want = F.sf_atoms(_natural_as_rows(fmt, os_))
        got = q.sf.cpu().numpy()
        assert got.shape[0] == want.shape[0] and got.shape[1] >= want.shape[1]
        assert np.array_equal(got[:, : want.shape[1]], want), f"SF atoms differ (fmt {fmt})"
        assert not got[:, want.shape[1] :].any(), "SF padding must be zero"
    return q


def test_reference_golden_rowscale(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "rowscale.npz"))
    for n in sorted({k[:-2] for k in g.files if k.endswith("_x")}):
        x = torch.from_numpy(g[n + "_x"]).cuda()
        if bool(g[n + "_isbf16"]):
            x = x.bfloat16()
        q, s = ops.per_row_col_quantize(x)
        assert np.array_equal(q.cpu().numpy(), g[n + "_q"]), n
        assert np.array_equal(s.cpu().numpy(), g[n + "_s"]), n
        d = ops._dequantize_to_bf16(q, s).float().cpu().numpy()
        assert np.array_equal(d, g[n + "_deq_bf16_as_f32"]), n


def test_reference_golden_blk16(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "blk16.npz"))
    for n in sorted({k[:-2] for k in g.files if k.endswith("_x")}):
        x = torch.from_numpy(g[n + "_x"]).cuda()
        for mode in "AB":
            q, s = ops.mxfp4_block_quantize(x, mode=mode)
            assert np.array_equal(q.cpu().numpy(), g[f"{n}_{mode}_q"]), (n, mode)
            assert np.array_equal(s.cpu().numpy(), g[f"{n}_{mode}_s"]), (n, mode)
            d = ops.mxfp4_dequant(q, s, mode).cpu().numpy()
            assert np.array_equal(d, g[f"{n}_{mode}_deq"]), (n, mode)


@pytest.mark.parametrize("fmt", ALL_FMTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 128), (130, 512), (256, 2048), (64, 256), (1000, 1024)])
def test_all_formats_bit_exact(ops, fmt, dtype, shape):
    torch.manual_seed(hash((fmt, shape)) % 1000)
    M, K = shape
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-3, 3, M, device="cuda")[:, None]).to(dtype)
    if M > 4:
        x[3] = 0  # all-zero row: scale byte 108 / fp32 scale 1.0
        x[4, : K // 2] = 0
    _check(ops, x, fmt)


@pytest.mark.parametrize("fmt,K", [(F.FMT_ROWSCALE, 96), (F.FMT_ROWSCALE, 8), (F.FMT_BLK16_A, 48), (F.FMT_BLK16_B, 16),
                                   (F.FMT_MX32, 96), (F.FMT_NV16, 80), (F.FMT_FP8_1X128, 384), (F.FMT_MX32, 9728)])
def test_odd_widths(ops, fmt, K):
    torch.manual_seed(K)
    x = torch.randn(34, K, device="cuda").bfloat16()
    _check(ops, x, fmt)


@pytest.mark.parametrize("fmt", ALL_FMTS)
def test_ties_and_power_of_two_scales(ops, fmt):
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 0.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -0.0, 6.0, 4.0])
    rows = [(ties * 2.0**sh).repeat(8) for sh in (-9, -3, 0, 5, 20)]
    rows += [torch.full((128,), 1.5), torch.full((128,), -1e-9), torch.zeros(128)]
    x = torch.stack(rows).cuda()
    _check(ops, x, fmt)
    _check(ops, x.bfloat16(), fmt)


def test_empty_inputs(ops):
    q = ops.quantize(torch.empty(0, 128, device="cuda", dtype=torch.bfloat16), F.FMT_MX32)
    assert q.codes.shape == (0, 64)


def test_ten_million_values_with_ties(ops):
    # byte-level agreement over >= 1e7 seeded bf16 values, exact ties mixed in
    torch.manual_seed(123)
    x = torch.randn(20480, 512, device="cuda")
    tie = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5], device="cuda")
    idx = torch.randint(0, 6, (20480, 512), device="cuda")
    x = torch.where(torch.rand_like(x) < 0.05, tie[idx] * torch.sign(x), x).bfloat16()
    x[::97] = 0
    for fmt in (F.FMT_ROWSCALE, F.FMT_MX32, F.FMT_BLK16_A):
        _check(ops, x, fmt, sf=False)


def test_strided_rows(ops):
    torch.manual_seed(1)
    big = torch.randn(64, 1536, device="cuda").bfloat16()
    v = big[:, 1024:]  # a column slice: row stride 1536
    q = ops.quantize(v, F.FMT_MX32)
    oq, os_, _ = F.quantize(v.float().cpu().numpy(), F.FMT_MX32)
    assert np.array_equal(q.codes.cpu().numpy(), oq) and np.array_equal(q.scales.cpu().numpy(), os_)


def test_nv16_given_amax(ops):
    torch.manual_seed(2)
    x = torch.randn(100, 256, device="cuda").bfloat16()
    am = torch.tensor([7.5], device="cuda")
    _check(ops, x, F.FMT_NV16, amax_t=am)


def test_amax_kernel(ops):
    torch.manual_seed(3)
    for dt in (torch.bfloat16, torch.float32):
        x = torch.randn(333, 1024, device="cuda").to(dt)
        assert ops.amax(x).item() == x.float().abs().max().item()
    assert ops.amax(torch.zeros(8, 64, device="cuda")).item() == 0.0


def test_sf_from_natural(ops):
    rng = np.random.default_rng(0)
    for fmt, R, K in [(F.FMT_MX32, 300, 512), (F.FMT_NV16, 129, 256), (F.FMT_BLK16_B, 128, 64), (F.FMT_BLK16_A, 260, 96)]:
        blk = 32 if fmt == F.FMT_MX32 else 16
        if fmt == F.FMT_BLK16_A:
            s = rng.integers(0, 255, (K // blk, R // 2), dtype=np.uint8)
        elif fmt == F.FMT_BLK16_B:
            s = rng.integers(0, 255, (K // blk, R), dtype=np.uint8)
        else:
            s = rng.integers(0, 255, (R, K // blk), dtype=np.uint8)
        got = ops.sf_from_natural(fmt, torch.from_numpy(s).cuda(), R, K).cpu().numpy()
        want = F.sf_atoms(_natural_as_rows(fmt, s))
        assert np.array_equal(got[:, : want.shape[1]], want)
        assert not got[:, want.shape[1] :].any()


@pytest.mark.parametrize("fmt", [F.FMT_ROWSCALE, F.FMT_BLK16_A, F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("K", [512, 256, 1024, 2048])
def test_layernorm_fused_quantize_bit_exact(ops, fmt, dtype, K):
    torch.manual_seed(K + fmt)
    M = 258
    x = (torch.randn(M, K, device="cuda") * 3 + 0.5).to(dtype)
    x[7] = 0.25  # constant row: variance 0
    g = torch.randn(K, device="cuda")
    b = torch.randn(K, device="cuda")
    am = torch.tensor([9.0], device="cuda") if fmt == F.FMT_NV16 else None
    q, y = ops.ln_quantize(x, g, b, 1e-5, fmt, natural=True, amax_t=am, y_dtype=torch.float32)
    torch.cuda.synchronize()
    half = G.ln_half_rows(K, dtype == torch.bfloat16, fmt)
    yo = G.layernorm_ref(x.float().cpu().numpy(), g.cpu().numpy(), b.cpu().numpy(), 1e-5, half_rows=half)
    assert np.array_equal(y.cpu().numpy(), yo), "fused LayerNorm differs from its CPU restatement"
    oq, os_, _ = F.quantize(yo, fmt, **({"amax_t": 9.0} if fmt == F.FMT_NV16 else {}))
    assert np.array_equal(q.codes.cpu().numpy(), oq)
    assert np.array_equal(q.scales.cpu().numpy(), os_)
    # the reference's own tolerance for its LayerNorm kernel (tests/kernels/test_cuda_ops.py:24-45)
    t = torch.nn.functional.layer_norm(x.float(), (K,), g, b, 1e-5)
    assert (y - t).abs().max().item() < 2e-4 * max(1.0, t.abs().max().item())


def test_layernorm_only_and_bf16_output(ops):
    torch.manual_seed(9)
    x = torch.randn(300, 512, device="cuda").bfloat16()
    g = torch.rand(512, device="cuda") + 0.5
    b = torch.randn(512, device="cuda")
    y = ops.layernorm(x, g, b, 1e-5)
    yo = G.layernorm_ref(x.float().cpu().numpy(), g.cpu().numpy(), b.cpu().numpy(), 1e-5, half_rows=G.ln_half_rows(512, True))
    assert y.dtype == torch.bfloat16
    assert np.array_equal(y.float().cpu().numpy(), G.to_bf16(yo))
    y32 = ops.fused_layernorm(x.float(), g, b)  # fp32 rows: the warp-per-row order
    assert np.array_equal(y32.cpu().numpy(), G.layernorm_ref(x.float().cpu().numpy(), g.cpu().numpy(), b.cpu().numpy(), 1e-5))
    # in place
    x2 = x.clone()
    ops.layernorm(x2, g, b, 1e-5, out=x2)
    assert torch.equal(x2, y)


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128])
@pytest.mark.parametrize("M", [1, 2, 129, 4097])
def test_half_warp_per_row_lanes(ops, fmt, M):
    """bf16 rows of 512 elements (the activation shape of the encoder): two rows per warp.  Odd row
    counts leave the second half of the last warp without a row; every combination of outputs -- SF
    atoms, natural scales, y in bf16 / fp32 / in place, one or two LayerNorms -- gives the oracle's bytes."""
    torch.manual_seed(M + fmt)
    K = 512
    x = (torch.randn(M, K, device="cuda") * 2 - 0.3).bfloat16()
    x[0, :32] = 0  # an all-zero block
    g1, b1 = torch.rand(K, device="cuda") + 0.5, torch.randn(K, device="cuda") * 0.2
    g2, b2 = torch.rand(K, device="cuda") + 0.5, torch.randn(K, device="cuda") * 0.2
    am = torch.tensor([9.0], device="cuda") if fmt == F.FMT_NV16 else None
    kw = {"amax_t": 9.0} if fmt == F.FMT_NV16 else {}
    xn = x.float().cpu().numpy()
    # plain quantize: natural scales, and the SF atoms agree with the relayout of the natural ones
    q = ops.quantize(x, fmt, natural=True, amax_t=am)
    oq, os_, _ = F.quantize(xn, fmt, **kw)
    assert np.array_equal(q.codes.cpu().numpy(), oq) and np.array_equal(q.scales.cpu().numpy(), os_)
    if fmt != F.FMT_FP8_1X128:
        q_sf = ops.quantize(x, fmt, natural=False, amax_t=am)
        assert torch.equal(q_sf.codes, q.codes)
        assert torch.equal(q_sf.sf, ops.sf_from_natural(fmt, q.scales, M, K))
    # LayerNorm + quantize, y in fp32 and in bf16
    y1 = G.layernorm_ref(xn, g1.cpu().numpy(), b1.cpu().numpy(), 1e-5, half_rows=True)
    ql, y = ops.ln_quantize(x, g1, b1, 1e-5, fmt, natural=True, amax_t=am, y_dtype=torch.float32)
    assert np.array_equal(y.cpu().numpy(), y1)
    oq, os_, _ = F.quantize(y1, fmt, **kw)
    assert np.array_equal(ql.codes.cpu().numpy(), oq) and np.array_equal(ql.scales.cpu().numpy(), os_)
    yb = ops.layernorm(x, g1, b1, 1e-5)
    assert np.array_equal(yb.float().cpu().numpy(), G.to_bf16(y1))
    # two LayerNorms, the first stored in place
    xin = x.clone()
    q2 = ops.ln2_quantize(xin, g1, b1, g2, b2, 1e-5, fmt, y=xin, natural=True, amax_t=am)
    assert np.array_equal(xin.float().cpu().numpy(), G.to_bf16(y1))
    y2 = G.layernorm_ref(G.to_bf16(y1), g2.cpu().numpy(), b2.cpu().numpy(), 1e-5, half_rows=True)
    oq, os_, _ = F.quantize(y2, fmt, **kw)
    assert np.array_equal(q2.codes.cpu().numpy(), oq) and np.array_equal(q2.scales.cpu().numpy(), os_)


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_FP8_1X128, F.FMT_NV16])
def test_full_size_activation_shape(ops, fmt):
    # benchmark shapes: T = 90000 frames x d_model 512; oracle compared on every row
    torch.manual_seed(0)
    x = torch.randn(90000, 512, device="cuda").bfloat16()
    _check(ops, x, fmt)


def test_argument_errors_raise(ops):
    from velox_voice_b200._lib import VeloxError

    with pytest.raises(VeloxError):
        ops.quantize(torch.zeros(4, 40, device="cuda"), F.FMT_MX32)  # K not a multiple of 32
    with pytest.raises(VeloxError):
        ops.quantize(torch.zeros(3, 64, device="cuda"), F.FMT_BLK16_A)  # odd row count
    with pytest.raises(TypeError):
        ops.quantize(torch.zeros(4, 64, device="cuda", dtype=torch.float16), F.FMT_MX32)


@pytest.mark.parametrize("fmt", ["mx32", "nv16", "fp8_1x128", "rowscale"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_two_layernorms_fused_equal_the_two_launches(fmt, dtype):
    """vx_ln2_quantize_pack == LayerNorm launch (stored y) followed by LayerNorm + quantize."""
    from velox_voice_b200 import ops

    torch.manual_seed(5)
    M, K = 333, 512
    x = (torch.randn(M, K, device="cuda") * 3 + 0.5).to(dtype)
    g1, b1 = torch.rand(K, device="cuda") + 0.5, torch.randn(K, device="cuda") * 0.1
    g2, b2 = torch.rand(K, device="cuda") + 0.5, torch.randn(K, device="cuda") * 0.1
    am = torch.tensor([8.0], device="cuda") if fmt == "nv16" else None
    y_ref = ops.layernorm(x.clone(), g1, b1, 1e-5, fmt=fmt)
    q_ref = ops.ln_quantize(y_ref, g2, b2, 1e-5, fmt, natural=True, amax_t=am)
    xin = x.clone()
    q = ops.ln2_quantize(xin, g1, b1, g2, b2, 1e-5, fmt, y=xin, natural=True, amax_t=am)  # in place
    torch.cuda.synchronize()
    assert torch.equal(xin, y_ref)
    assert torch.equal(q.codes, q_ref.codes)
    assert torch.equal(q.scales, q_ref.scales)
    if q.sf is not None:
        assert torch.equal(q.sf, q_ref.sf)


@pytest.mark.parametrize("fmt", ["mx32", "nv16"])
def test_sf_rows_beyond_m_read_as_zero_on_recycled_memory(fmt):
    """The SF atoms cover rows in tiles of 128; the rows between M and the next multiple of 128
    must be zero whatever the buffer held before (the kernels clear them, no memset launch)."""
    from velox_voice_b200 import ops

    def poison(nbytes):
        t = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        del t  # the caching allocator hands these bytes to the next torch.empty of that size

    torch.manual_seed(3)
    M, K, N = 300, 512, 256
    x = torch.randn(M, K, device="cuda").bfloat16()
    g, b = torch.ones(K, device="cuda"), torch.zeros(K, device="cuda")
    am = torch.tensor([8.0], device="cuda") if fmt == "nv16" else None
    lib_sf = lambda rows, k: ((rows + 127) // 128) * int(ops._lib.load().vx_sf_kgroups(ops._fmt(fmt), k)) * 512

    def check(q, rows):
        sf = q.sf.view((rows + 127) // 128, -1, 32, 4, 4)  # [tile, kg, r % 32, (r / 32) % 4, kb % 4]
        r = torch.arange(128, device="cuda")
        pad = (r + 128 * ((rows - 1) // 128)) >= rows
        last = sf[-1]  # [kg, 32, 4, 4]
        by_row = last.permute(2, 1, 0, 3).reshape(128, -1)  # row = (r/32 % 4) * 32 + r % 32
        assert int(by_row[pad].max()) == 0, "scale factors of rows beyond M are not zero"
        assert int(by_row[~pad].max()) > 0

    poison(lib_sf(M, K))
    check(ops.quantize(x, fmt, natural=False, amax_t=am), M)
    poison(lib_sf(M, K))
    check(ops.ln_quantize(x, g, b, 1e-5, fmt, amax_t=am), M)
    w = ops.quantize(0.05 * torch.randn(N, K, device="cuda"), fmt)
    a = ops.quantize(x, fmt, amax_t=am)
    poison(lib_sf(M, N))
    check(ops.bsgemm(a, w, epilogue=ops.EPI_BIAS_SWISH, bias=torch.zeros(N, device="cuda"), out_fmt=fmt, out_amax=am), M)

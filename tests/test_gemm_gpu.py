"""tcgen05 block-scaled GEMMs (through the C ABI) against the CPU oracle.

Per-row-scaled FP4 follows the reference's own test methodology
(tests/kernels/test_dgx_mxfp4_gemm.py in the reference project): quantize seeded bf16 data,
run the GEMM, compare with ``unpack(xq) @ unpack(wq).T * row_scale * col_scale`` and require
``diff == 0``.  Formats without a reference kernel are held to the path's acceptance bound:
max relative error 1e-2 against dequantize-then-fp32-matmul.
"""

import os

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import gemm as G

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2  # acceptance bound of the path (bf16 output)


@pytest.fixture(scope="module")
def ops():
    from velox_voice_b200 import ops as o

    return o


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from velox_voice_b200 import _lib

    assert _lib.device_status() == 0, "a bounded device-side wait expired"


def rel_err(got, ref):
    return float(np.abs(got - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def ref_from_q(fmt, a, b):
    ga = F.nv16_global_scale(a.amax.item()) if a.amax is not None else None
    gb = F.nv16_global_scale(b.amax.item()) if b.amax is not None else None
    return G.gemm_ref(fmt, a.codes.cpu().numpy(), a.scales.cpu().numpy(), b.codes.cpu().numpy(), b.scales.cpu().numpy(), ga, gb)


# ------------------------------------------------------------------ reference methodology


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 64), (256, 128, 128), (512, 512, 2048),
                                   (1024, 512, 1024), (2048, 2048, 2048)])
def test_bit_exact_methodology(ops, M, N, K):
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    xq, xs = ops.quantize_w(x)
    wq, ws = ops.quantize_w(w)
    out = ops.dgx_mxfp4_gemm(xq, wq, xs, ws)
    ref = G.gemm_rowscale_ref(xq.cpu().numpy(), wq.cpu().numpy(), xs.cpu().numpy(), ws.cpu().numpy())
    assert out.shape == (M, N) and out.dtype == torch.float32
    assert np.abs(out.cpu().numpy() - ref).max() == 0.0


def test_same_shape_new_tensors(ops):
    """Same shapes, different tensors: no stale tensor-map state may survive between calls."""
    torch.manual_seed(1)
    M, N, K = 512, 512, 2048
    outs = []
    for _ in range(2):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        xq, xs = ops.quantize_w(x)
        wq, ws = ops.quantize_w(w)
        out = ops.dgx_mxfp4_gemm(xq, wq, xs, ws)
        ref = G.gemm_rowscale_ref(xq.cpu().numpy(), wq.cpu().numpy(), xs.cpu().numpy(), ws.cpu().numpy())
        assert np.abs(out.cpu().numpy() - ref).max() == 0.0
        outs.append(out)
    assert (outs[0] - outs[1]).abs().max().item() > 0.0


def test_unit_scale_parity(ops):
    torch.manual_seed(2)
    M, N, K = 256, 256, 128
    pa = torch.randint(0, 8, (M, K), dtype=torch.uint8)
    pb = torch.randint(0, 8, (N, K), dtype=torch.uint8)
    qa = torch.from_numpy(F.pack_codes(pa.numpy())).cuda()
    qb = torch.from_numpy(F.pack_codes(pb.numpy())).cuda()
    sa = torch.full((M,), 0x7F, dtype=torch.uint8, device="cuda")
    sb = torch.full((N,), 0x7F, dtype=torch.uint8, device="cuda")
    out = ops.dgx_mxfp4_gemm(qa, qb, sa, sb)
    ref = G.matmul_f32(F.e2m1_decode(pa.numpy()), F.e2m1_decode(pb.numpy()))
    assert np.abs(out.cpu().numpy() - ref).max() == 0.0


def test_all_code_pairs(ops):
    """Every E2M1 code (incl. 7 = 6.0 and -0) against every other: 16 x 16 products, one per k."""
    codes = np.arange(16, dtype=np.uint8)
    a = np.zeros((128, 64), np.uint8)
    b = np.zeros((128, 64), np.uint8)
    for i in range(16):
        a[i, :16] = codes[i]          # row i: code i in the first 16 k
        b[i, :16] = codes             # col j: all codes
    for j in range(16):
        b[16 + j, j] = codes[j]       # isolate single products
    qa = torch.from_numpy(F.pack_codes(a)).cuda()
    qb = torch.from_numpy(F.pack_codes(b)).cuda()
    s = torch.full((128,), 0x7F, dtype=torch.uint8, device="cuda")
    out = ops.dgx_mxfp4_gemm(qa, qb, s, s).cpu().numpy()
    ref = G.matmul_f32(F.e2m1_decode(a), F.e2m1_decode(b))
    assert np.array_equal(out, ref)


def test_reference_golden_gemm(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "gemm_rowscale.npz"))
    for seed in (0, 1, 2):
        t = lambda k: torch.from_numpy(g[f"gemm{seed}_{k}"]).cuda()
        out = ops.dgx_mxfp4_gemm(t("xq"), t("wq"), t("xs"), t("ws"))
        assert np.array_equal(out.cpu().numpy(), g[f"gemm{seed}_ref"]), seed


def test_extreme_row_scales(ops):
    torch.manual_seed(3)
    x = torch.randn(128, 128, device="cuda") * torch.logspace(-12, 12, 128, device="cuda")[:, None]
    w = torch.randn(128, 128, device="cuda") * torch.logspace(-6, 6, 128, device="cuda")[:, None]
    xq, xs = ops.quantize_w(x)
    wq, ws = ops.quantize_w(w)
    out = ops.dgx_mxfp4_gemm(xq, wq, xs, ws)
    ref = G.gemm_rowscale_ref(xq.cpu().numpy(), wq.cpu().numpy(), xs.cpu().numpy(), ws.cpu().numpy())
    assert np.array_equal(out.cpu().numpy(), ref)


def test_nvfp4_linear_and_3d_input(ops):
    torch.manual_seed(4)
    x = torch.randn(4, 50, 128, device="cuda")
    w = torch.randn(64, 128, device="cuda")
    wq, ws = ops.quantize_w(w)
    out = ops.nvfp4_linear(x, wq, ws)
    assert out.shape == (4, 50, 64) and out.dtype == torch.float32 and torch.isfinite(out).all()
    xq, xs = ops.quantize_w(x.reshape(-1, 128))
    ref = G.gemm_rowscale_ref(xq.cpu().numpy(), wq.cpu().numpy(), xs.cpu().numpy(), ws.cpu().numpy())
    assert np.array_equal(out.reshape(-1, 64).cpu().numpy(), ref)


# ------------------------------------------------------------------ block-scaled formats


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 512), (300, 200, 512), (130, 136, 1024)])
def test_blk16_through_reference_signature(ops, M, N, K):
    torch.manual_seed(5)
    if M % 2:
        M += 1
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    aq, asc = ops.mxfp4_block_quantize(x, mode="A")
    bq, bsc = ops.mxfp4_block_quantize(w, mode="B")
    out = ops.mxfp4_gemm(aq, bq, asc, bsc)
    ref = G.matmul_f32(F.dequant_blk16(aq.cpu().numpy(), asc.cpu().numpy(), "A"),
                       F.dequant_blk16(bq.cpu().numpy(), bsc.cpu().numpy(), "B"))
    assert out.dtype == torch.float32
    assert rel_err(out.cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 128, 512), (256, 384, 1024), (300, 200, 512),
                                   (1, 8, 256), (129, 5538, 512), (1024, 512, 2048)])
@pytest.mark.parametrize("direct", [False, True])
def test_block_formats_f32_out(ops, fmt, M, N, K, direct):
    torch.manual_seed(6)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.02 * torch.randn(N, K, device="cuda")).bfloat16()
    a, b = ops.quantize(x, fmt), ops.quantize(w, fmt)
    out = ops.bsgemm(a, b, out_dtype=torch.float32, direct_store=direct)
    assert rel_err(out.cpu().numpy(), ref_from_q(fmt, a, b)) < 1e-5


def test_cfg1_single_mxfp4_linear(ops):
    """benchmark configs[0]: x bf16 [1024, 512] ~ N(0,1), W [2048, 512] ~ N(0, 0.02), seed 0, bf16 out."""
    torch.manual_seed(0)
    x = torch.randn(1024, 512).bfloat16().cuda()
    w = (0.02 * torch.randn(2048, 512)).cuda()
    a, b = ops.quantize(x, "mx32"), ops.quantize(w, "mx32")
    out = ops.bsgemm(a, b, out_dtype=torch.bfloat16)
    assert out.shape == (1024, 2048) and out.dtype == torch.bfloat16
    assert rel_err(out.float().cpu().numpy(), ref_from_q(F.FMT_MX32, a, b)) < REL_TOL


# ------------------------------------------------------------------ epilogues


@pytest.fixture(scope="module")
def epi_case(ops):
    torch.manual_seed(7)
    M, N, K = 384, 512, 512
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    return M, N, K, x, w, bias, res


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_NV16, F.FMT_FP8_1X128, F.FMT_ROWSCALE])
@pytest.mark.parametrize("epi", [G.EPI_BIAS, G.EPI_BIAS_SWISH, G.EPI_BIAS_RESIDUAL])
@pytest.mark.parametrize("direct", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_fused_epilogues(ops, epi_case, fmt, epi, direct, out_dtype):
    M, N, K, x, w, bias, res = epi_case
    a, b = ops.quantize(x, fmt), ops.quantize(w, fmt)
    out = ops.bsgemm(a, b, epilogue=epi, bias=bias, residual=res, alpha=0.5, out_dtype=out_dtype, direct_store=direct)
    ref = G.epilogue_ref(ref_from_q(fmt, a, b), epi, bias.cpu().numpy(), res.float().cpu().numpy(), 0.5)
    assert out.dtype == out_dtype
    assert rel_err(out.float().cpu().numpy(), ref) < REL_TOL


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_FP8_1X128])
@pytest.mark.parametrize("direct", [False, True])
def test_glu_epilogue(ops, epi_case, fmt, direct):
    from velox_voice_b200.linear import glu_interleave_index, glu_tile

    M, N, K, x, w, bias, res = epi_case
    tile = glu_tile(fmt)
    idx = glu_interleave_index(N, "cuda", tile)
    assert np.array_equal(idx.cpu().numpy(), G.glu_interleave_rows(N, tile))
    a = ops.quantize(x, fmt)
    b_plain = ops.quantize(w, fmt)
    b = ops.quantize(w[idx].contiguous(), fmt)
    out = ops.bsgemm(a, b, epilogue=G.EPI_BIAS_GLU, bias=bias[idx].contiguous(), out_dtype=torch.bfloat16, direct_store=direct)
    ref = G.epilogue_ref(ref_from_q(fmt, a, b_plain), G.EPI_BIAS_GLU, bias.cpu().numpy())
    assert out.shape == (M, N // 2)
    assert rel_err(out.float().cpu().numpy(), ref) < REL_TOL


def test_residual_in_place(ops, epi_case):
    M, N, K, x, w, bias, res = epi_case
    a, b = ops.quantize(x, "mx32"), ops.quantize(w, "mx32")
    want = ops.bsgemm(a, b, epilogue=G.EPI_BIAS_RESIDUAL, bias=bias, residual=res, alpha=0.5)
    buf = res.clone()
    got = ops.bsgemm(a, b, epilogue=G.EPI_BIAS_RESIDUAL, bias=bias, residual=buf, alpha=0.5, out=buf)
    assert got.data_ptr() == buf.data_ptr() and torch.equal(got, want)


def test_tma_and_direct_stores_agree_and_respect_bounds(ops):
    torch.manual_seed(8)
    M, N, K = 200, 264, 512
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    a, b = ops.quantize(x, "mx32"), ops.quantize(w, "mx32")
    outs = []
    for direct in (False, True):
        canvas = torch.full((M + 8, N + 24), -7.0, device="cuda", dtype=torch.bfloat16)
        view = canvas[:M, :N]
        ops.bsgemm(a, b, out=view, direct_store=direct)
        assert (canvas[M:] == -7.0).all() and (canvas[:, N:] == -7.0).all(), "store went past the logical output"
        outs.append(view.clone())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("out_fmt", [F.FMT_MX32, F.FMT_NV16])
def test_requantized_output_is_the_quantizer_of_the_f32_output(ops, epi_case, out_fmt):
    M, N, K, x, w, bias, res = epi_case
    a, b = ops.quantize(x, "mx32"), ops.quantize(w, "mx32")
    am = torch.tensor([3.0], device="cuda") if out_fmt == F.FMT_NV16 else None
    for epi in (G.EPI_NONE, G.EPI_BIAS_SWISH):
        h = ops.bsgemm(a, b, epilogue=epi, bias=bias, out_dtype=torch.float32)
        hq = ops.bsgemm(a, b, epilogue=epi, bias=bias, out_fmt=out_fmt, out_amax=am, out_natural=True)
        oq, os_, _ = F.quantize(h.cpu().numpy(), out_fmt, **({"amax_t": 3.0} if am is not None else {}))
        assert np.array_equal(hq.codes.cpu().numpy(), oq)
        assert np.array_equal(hq.scales.cpu().numpy(), os_)
        want_sf = F.sf_atoms(os_)
        assert np.array_equal(hq.sf.cpu().numpy()[:, : want_sf.shape[1]], want_sf)
        # and it chains: the re-quantized tensor is a valid A operand
        w2 = (0.05 * torch.randn(256, N, device="cuda")).bfloat16()
        b2 = ops.quantize(w2, out_fmt)
        y = ops.bsgemm(hq, b2, out_dtype=torch.float32)
        ref = G.gemm_ref(out_fmt, oq, os_, b2.codes.cpu().numpy(), b2.scales.cpu().numpy(),
                         F.nv16_global_scale(3.0) if am is not None else None,
                         F.nv16_global_scale(b2.amax.item()) if am is not None else None)
        assert rel_err(y.cpu().numpy(), ref) < 1e-5


# ------------------------------------------------------------------ benchmark sizes


@pytest.mark.parametrize("fmt,N,K,epi", [(F.FMT_FP8_1X128, 1536, 512, G.EPI_BIAS), (F.FMT_NV16, 2048, 512, G.EPI_BIAS_SWISH),
                                         (F.FMT_NV16, 512, 2048, G.EPI_BIAS_RESIDUAL), (F.FMT_MX32, 5538, 512, G.EPI_BIAS)])
def test_full_size_T90000_sampled_rows(ops, fmt, N, K, epi):
    """configs[1] (fused QKV, FP8 1x128) and configs[2] (NVFP4 FFN) at T = 90000: the whole
    GEMM runs on the GPU; 640 sampled rows (first / last tile included) are checked on the CPU."""
    torch.manual_seed(0)
    T = 90000
    x = torch.randn(T, K, device="cuda").bfloat16()
    bound = (6.0 / (K + N)) ** 0.5
    w = ((torch.rand(N, K, device="cuda") * 2 - 1) * bound) if fmt == F.FMT_FP8_1X128 else 0.02 * torch.randn(N, K, device="cuda")
    bias = 0.1 * torch.randn(N, device="cuda")
    res = torch.randn(T, N, device="cuda").bfloat16() if epi == G.EPI_BIAS_RESIDUAL else None
    a, b = ops.quantize(x, fmt), ops.quantize(w, fmt)
    out = ops.bsgemm(a, b, epilogue=epi, bias=bias, residual=res, alpha=0.5, out_dtype=torch.bfloat16)
    rows = torch.cat([torch.arange(0, 128), torch.arange(T - 128, T), torch.randint(0, T, (384,))]).cuda()
    ga = F.nv16_global_scale(a.amax.item()) if a.amax is not None else None
    gb = F.nv16_global_scale(b.amax.item()) if b.amax is not None else None
    acc = G.gemm_ref(fmt, a.codes[rows].cpu().numpy(), a.scales[rows].cpu().numpy(), b.codes.cpu().numpy(),
                     b.scales.cpu().numpy(), ga, gb)
    ref = G.epilogue_ref(acc, epi, bias.cpu().numpy(), res[rows].float().cpu().numpy() if res is not None else None, 0.5)
    assert rel_err(out[rows].float().cpu().numpy(), ref) < REL_TOL
    # rows are independent: any 2-way split of the frames gives the same bytes (what sharding relies on)
    half = 45056
    a2 = ops.quantize(x[half:], fmt, amax_t=a.amax)
    out2 = ops.bsgemm(a2, b, epilogue=epi, bias=bias, residual=None if res is None else res[half:], alpha=0.5,
                      out_dtype=torch.bfloat16)
    assert torch.equal(out2, out[half:])


def test_argument_errors_raise(ops):
    from velox_voice_b200._lib import VeloxError

    x = torch.randn(128, 64, device="cuda").bfloat16()
    a = ops.quantize(x, "mx32")
    b = ops.quantize(torch.randn(128, 128, device="cuda").bfloat16(), "mx32")
    with pytest.raises(ValueError):
        ops.bsgemm(a, b)  # K mismatch
    with pytest.raises(ValueError):
        ops.bsgemm(a, ops.quantize(x, "nv16"))  # format mismatch
    with pytest.raises(VeloxError):
        ops.dgx_mxfp4_gemm(torch.zeros(128, 24, dtype=torch.uint8, device="cuda"), torch.zeros(128, 24, dtype=torch.uint8, device="cuda"),
                           torch.zeros(128, dtype=torch.uint8, device="cuda"), torch.zeros(128, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("fmt", ["mx32", "nv16", "fp8_1x128", "rowscale"])
@pytest.mark.parametrize("M,N,K", [(1000, 5538, 512), (130, 96, 256), (257, 700, 1024)])
def test_argmax_epilogue_equals_argmax_of_the_bf16_logits(fmt, M, N, K):
    """VX_EPI_BIAS_ARGMAX == bsgemm(bias, bf16).argmax(1), ties to the lowest column."""
    from velox_voice_b200 import ops

    torch.manual_seed(11)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda") * 0.05
    w[N // 2] = w[3]           # duplicated vocabulary rows: exact ties in the logits
    w[N - 1] = w[3]
    bias = torch.randn(N, device="cuda") * 0.01
    bias[N // 2] = bias[3]
    bias[N - 1] = bias[3]
    am = {}
    if fmt == "nv16":
        am = {"amax_t": ops.amax(x)}
    a = ops.quantize(x, fmt, **am)
    b = ops.quantize(w, fmt)
    logits = ops.bsgemm(a, b, epilogue=ops.EPI_BIAS, bias=bias, out_dtype=torch.bfloat16)
    want = logits.float().argmax(dim=1).to(torch.int32)
    ids, vmax = ops.bsgemm_argmax(a, b, bias, return_max=True)
    torch.cuda.synchronize()
    assert torch.equal(ids, want)
    assert torch.equal(vmax, logits.float().max(dim=1).values)
    # rows whose maximum sits on the duplicated column must report the first copy
    assert not bool(((ids == N // 2) | (ids == N - 1)).any())
    if fmt != "fp8_1x128":
        # the CTC tail: log-sum-exp of the row and the winner's log-probability, without the logits
        ids2, vmax2, lse, logp = ops.bsgemm_argmax(a, b, bias, return_max=True, return_logp=True)
        torch.cuda.synchronize()
        assert torch.equal(ids2, want) and torch.equal(vmax2, vmax)
        ls = torch.log_softmax(logits.float(), dim=1)
        want_lse = torch.logsumexp(logits.float(), dim=1)
        assert (lse - want_lse).abs().max().item() < 1e-3
        assert (logp - ls.gather(1, want.long()[:, None])[:, 0]).abs().max().item() < 1e-3


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_NV16, F.FMT_ROWSCALE])
@pytest.mark.parametrize("M,N,K", [(300, 200, 512), (129, 5538, 512), (1024, 512, 2048), (257, 384, 256)])
@pytest.mark.parametrize("epi", [G.EPI_NONE, G.EPI_BIAS, G.EPI_BIAS_SWISH, G.EPI_BIAS_RESIDUAL])
def test_wide_and_narrow_tiles_give_the_same_bytes(ops, fmt, M, N, K, epi):
    """The 128 x 256 single-accumulator and 128 x 128 double-accumulator FP4 kernels are two
    schedules of the same arithmetic: outputs must be identical, and equal to the oracle."""
    torch.manual_seed(21)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    bias = torch.randn(N, device="cuda") if epi != G.EPI_NONE else None
    res = torch.randn(M, N, device="cuda").bfloat16() if epi == G.EPI_BIAS_RESIDUAL else None
    a, b = ops.quantize(x, fmt), ops.quantize(w, fmt)
    outs = [ops.bsgemm(a, b, epilogue=epi, bias=bias, residual=res, alpha=0.5, out_dtype=torch.float32, tiles=t)
            for t in ("wide", "narrow", None)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref = G.epilogue_ref(ref_from_q(fmt, a, b), epi, None if bias is None else bias.cpu().numpy(),
                         None if res is None else res.float().cpu().numpy(), 0.5)
    assert rel_err(outs[1].cpu().numpy(), ref) < REL_TOL
    if fmt != F.FMT_ROWSCALE and N % 128 == 0 and epi in (G.EPI_NONE, G.EPI_BIAS, G.EPI_BIAS_SWISH):
        am = torch.tensor([8.0], device="cuda") if fmt == F.FMT_NV16 else None
        qs = [ops.bsgemm(a, b, epilogue=epi, bias=bias, out_fmt=fmt, out_amax=am, out_natural=True, tiles=t)
              for t in ("wide", "narrow")]
        assert torch.equal(qs[0].codes, qs[1].codes) and torch.equal(qs[0].sf, qs[1].sf)
        assert torch.equal(qs[0].scales, qs[1].scales)


@pytest.mark.parametrize("fmt", [F.FMT_MX32, F.FMT_NV16])
@pytest.mark.parametrize("M,k", [(300, 5), (1, 1), (129, 8), (2000, 16)])
def test_ctc_topk_without_logits(ops, fmt, M, k):
    """torch.topk(log_softmax(bf16 logits), k) from two launches of the head and two small kernels, no [M, N]
    matrix: values within 1e-3 (the log-sum-exp is summed in another order), ids equal wherever the k-th and
    (k+1)-th logits differ (equal bf16 logits may come in either order from torch.topk; here: lowest column first)."""
    torch.manual_seed(M + k)
    N, K = 5538, 512
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    bias = torch.randn(N, device="cuda")
    am = torch.tensor([8.0], device="cuda") if fmt == F.FMT_NV16 else None
    a, b = ops.quantize(x, fmt, natural=False, amax_t=am), ops.quantize(w, fmt)
    logp, ids = ops.bsgemm_topk(a, b, bias, k)
    assert logp.shape == (M, k) and ids.shape == (M, k) and ids.dtype == torch.int64
    z = ops.bsgemm(a, b, epilogue=G.EPI_BIAS, bias=bias, out_dtype=torch.bfloat16)
    ref = torch.log_softmax(z.float(), dim=-1)
    rv, ri = torch.topk(ref, k, dim=-1)
    assert (logp - rv).abs().max().item() < 1e-3
    # the gathered reference log-probabilities of the returned ids are the top-k values: ids are right up to ties
    assert (ref.gather(1, ids) - rv).abs().max().item() == 0.0
    assert (logp[:, :-1] >= logp[:, 1:]).all() if k > 1 else True
    # rows sorted by ascending column among equal values
    eq = (logp[:, :-1] == logp[:, 1:]) if k > 1 else torch.zeros(M, 0, dtype=torch.bool, device="cuda")
    assert (ids[:, :-1][eq] < ids[:, 1:][eq]).all()


def test_ctc_topk_overflowing_rows_fall_back_to_logits(ops):
    """All-equal logits: every column reaches the threshold, the candidate lists overflow, and the rows are redone
    from explicit logits."""
    M, N, K = 40, 512, 256
    x = torch.zeros(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    a, b = ops.quantize(x, F.FMT_MX32, natural=False), ops.quantize(w, F.FMT_MX32)
    logp, ids = ops.bsgemm_topk(a, b, None, 5, capacity=16)
    assert (ids >= 0).all() and torch.allclose(logp, torch.full_like(logp, -float(np.log(N))), atol=1e-4)

"""The drop-in boundary on the GPU: cached tensor maps, the bounded-wait self-test, several
devices in one process, and the reference's operator / module names running on this library."""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import gemm as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from velox_voice_b200 import ops as o

    return o


def _cache_stats():
    from velox_voice_b200 import _lib

    h, m = C.c_int64(0), C.c_int64(0)
    assert _lib.load().vx_tmap_cache_stats(C.byref(h), C.byref(m)) == 0
    return h.value, m.value


def test_tensor_maps_are_encoded_once_per_buffer(ops):
    torch.manual_seed(0)
    a = ops.quantize(torch.randn(256, 512, device="cuda").bfloat16(), "mx32")
    b = ops.quantize(torch.randn(384, 512, device="cuda").bfloat16(), "mx32")
    out = torch.empty(256, 384, device="cuda", dtype=torch.bfloat16)
    first = ops.bsgemm(a, b, out=out).clone()
    h0, m0 = _cache_stats()
    for _ in range(5):
        ops.bsgemm(a, b, out=out)
    h1, m1 = _cache_stats()
    assert m1 == m0, "steady-state calls on the same buffers must not encode new tensor maps"
    assert h1 - h0 == 5 * 3  # A, B and the output map, every call
    assert torch.equal(out, first)
    # same shapes, other buffers: new maps, correct results (the reference's stale-descriptor case,
    # tests/kernels/test_dgx_mxfp4_gemm.py:93-112)
    a2 = ops.quantize(torch.randn(256, 512, device="cuda").bfloat16(), "mx32")
    out2 = ops.bsgemm(a2, b, out_dtype=torch.float32)
    ref = G.gemm_ref(F.FMT_MX32, a2.codes.cpu().numpy(), a2.scales.cpu().numpy(), b.codes.cpu().numpy(), b.scales.cpu().numpy())
    assert np.array_equal(out2.cpu().numpy(), ref)


def test_a_bounded_wait_that_runs_out_is_reported_once_and_the_gpu_stays_usable(ops):
    """An mbarrier nobody arrives at, a limit of 2 ms: the waiting thread gives up, the status word
    names the site and the CTA, a second read is clean, and the next GEMM is correct."""
    from velox_voice_b200 import _lib

    lib = _lib.load()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    site = 0x5A
    assert lib.vx_wait_selftest(2_000_000, site, torch.cuda.current_stream().cuda_stream) == 0
    status = _lib.device_status()  # synchronises
    assert status == (1 << 24) | (site << 16) | 0, hex(status)
    assert _lib.device_status() == 0, "the status word is reported once, then cleared"
    a = ops.quantize(torch.randn(128, 256, device="cuda").bfloat16(), "rowscale", sf=False)
    b = ops.quantize(torch.randn(128, 256, device="cuda").bfloat16(), "rowscale", sf=False)
    out = ops.bsgemm(a, b, out_dtype=torch.float32)
    ref = G.gemm_rowscale_ref(a.codes.cpu().numpy(), b.codes.cpu().numpy(), a.scales.cpu().numpy(), b.scales.cpu().numpy())
    assert np.array_equal(out.cpu().numpy(), ref)
    assert _lib.device_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_in_one_process(ops):
    """One GEMM per device from the same process (no peer access): kernel attributes, the status
    word and the SM count are kept per device."""
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            torch.manual_seed(5)
            x = torch.randn(300, 512).bfloat16().cuda()
            w = torch.randn(640, 512).bfloat16().cuda()
            a, b = ops.quantize(x, "mx32"), ops.quantize(w, "mx32")
            outs.append(ops.bsgemm(a, b, out_dtype=torch.float32).cpu())
            torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


def test_bf16_operator_names_run_on_the_quantized_path(ops, monkeypatch):
    """fused_qkv_wgmma / fused_qkv / pwlin_glu with the reference's signatures: the result is the
    oracle's quantize -> dequantize -> fp32 matmul (+ bias, GLU) of the same inputs."""
    monkeypatch.delenv("VELOXVOICE_QFORMAT", raising=False)
    torch.manual_seed(11)
    T = 200
    x = torch.randn(T, 512, device="cuda").bfloat16()
    w = (0.05 * torch.randn(1536, 512, device="cuda")).bfloat16()
    b = torch.randn(1536, device="cuda").bfloat16()
    y = ops.fused_qkv_wgmma(x, w, b)
    assert y is not None and y.shape == (T, 1536) and y.dtype == torch.bfloat16

    def deq(t):
        q, s, g = F.quantize(t.float().cpu().numpy(), F.FMT_MX32)
        return F.dequantize(q, s, F.FMT_MX32, g)

    ref = G.matmul_f32(deq(x), deq(w)) + b.float().cpu().numpy()[None, :]
    err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err < 1e-2
    out = torch.empty(T, 1536, device="cuda", dtype=torch.bfloat16)
    assert ops.fused_qkv(x, w, b, out) is out and torch.equal(out, y)
    # [n, T, d] input and GLU: value = first half of the channels, gate = second half
    wg = (0.05 * torch.randn(1024, 512, device="cuda")).bfloat16()
    bg = torch.randn(1024, device="cuda").bfloat16()
    x3 = x.view(2, T // 2, 512)
    g = ops.pwlin_glu(x3, wg, bg)
    assert g is not None and g.shape == (2, T // 2, 512)
    z = G.matmul_f32(deq(x), deq(wg)) + bg.float().cpu().numpy()[None, :]
    ref = z[:, :512] * G.sigmoid(z[:, 512:])
    err = np.abs(g.float().cpu().numpy().reshape(T, 512) - ref).max() / np.abs(ref).max()
    assert err < 1e-2
    # inputs the path does not take: None, like the reference's wrappers
    assert ops.pwlin_glu(x.float(), wg, bg) is None
    assert ops.fused_qkv_wgmma(x[:, :500], w[:, :500], b) is None


def test_reference_modules_on_this_library(ops):
    """DenseLinear / Nvfp4Linear / nvfp4_gemm / quantize_and_gemm: exactly the oracle's per-row
    FP4 product plus bias (the reference checks shape, dtype and finiteness only,
    tests/kernels/test_power_mel_log.py:217-266; fp32 mode must be exactly F.linear)."""
    from velox_voice_b200.linear import DenseLinear, Nvfp4Linear, nvfp4_gemm

    torch.manual_seed(3)
    w = torch.randn(64, 128)
    b = torch.randn(64)
    x = torch.randn(32, 128).cuda()
    lin = DenseLinear(w, b).cuda()
    lin.precision = "fp32"
    assert torch.equal(lin(x), torch.nn.functional.linear(x, lin.weight, lin.bias))

    def oracle_linear(xt, wt, bt):
        xq, xs, _ = F.quantize(xt.float().cpu().numpy(), F.FMT_ROWSCALE)
        wq, ws, _ = F.quantize(wt.float().cpu().numpy(), F.FMT_ROWSCALE)
        y = G.gemm_rowscale_ref(xq, wq, xs, ws)
        return y if bt is None else (y + bt.float().cpu().numpy()[None, :]).astype(np.float32)

    for mode in ("mxfp4", "nvfp4"):
        lin.precision = mode
        y = lin(x)
        assert y.shape == (32, 64) and y.dtype == torch.float32 and torch.isfinite(y).all()
        assert np.array_equal(y.cpu().numpy(), oracle_linear(x, lin.weight.detach(), lin.bias.detach()))
        y3 = lin(x.view(2, 16, 128))
        assert y3.shape == (2, 16, 64) and torch.equal(y3.view(32, 64), y)
    # the embedding's drain linear: K = 9728 (torch_conformer.py:290-292)
    wd = 0.02 * torch.randn(512, 9728)
    xd = torch.randn(70, 9728).cuda()
    drain = DenseLinear(wd, None).cuda()
    drain.precision = "mxfp4"
    assert np.array_equal(drain(xd).cpu().numpy(), oracle_linear(xd, drain.weight.detach(), None))

    m = Nvfp4Linear(128, 64, bias=True, device="cuda")
    xb = torch.randn(40, 128, device="cuda").bfloat16()
    ym = m(xb)
    xq, xs, _ = F.quantize(xb.float().cpu().numpy(), F.FMT_ROWSCALE)
    ref = G.gemm_rowscale_ref(xq, m.weight_q.cpu().numpy(), xs, m.weight_s.cpu().numpy()) + m.bias.cpu().numpy()[None, :]
    assert np.array_equal(ym.cpu().numpy(), ref.astype(np.float32))
    wq, ws = ops.quantize_w(w.cuda())
    assert np.array_equal(ops.quantize_and_gemm(x, wq, ws).cpu().numpy(), oracle_linear(x, w, None))
    assert np.array_equal(nvfp4_gemm(x, w.cuda(), b.cuda()).cpu().numpy(), oracle_linear(x, w, b))


@pytest.mark.parametrize("fmt", ["rowscale", "mx32"])
def test_drain_shape_gemm(ops, fmt):
    """embed.drain: 9728 -> 512, K is 38 stages of 256 (rowscale: the reference's lane; mx32)."""
    torch.manual_seed(12)
    x = torch.randn(300, 9728, device="cuda").bfloat16()
    w = (0.02 * torch.randn(512, 9728, device="cuda")).bfloat16()
    sf = fmt != "rowscale"
    a, b = ops.quantize(x, fmt, sf=sf), ops.quantize(w, fmt, sf=sf)
    out = ops.bsgemm(a, b, out_dtype=torch.float32)
    fid = F.FMT_NAMES[fmt]
    ref = G.gemm_ref(fid, a.codes.cpu().numpy(), a.scales.cpu().numpy(), b.codes.cpu().numpy(), b.scales.cpu().numpy())
    err = np.abs(out.cpu().numpy() - ref).max() / np.abs(ref).max()
    # K = 9728: partial sums no longer fit 24 bits, so the two summation orders differ in the last bits
    assert err < 1e-5

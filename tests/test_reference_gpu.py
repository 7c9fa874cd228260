"""The reference project's own code on the B200, next to this library.

Needs the copy of the reference package that ``oracle/make_ref.py`` puts into the git-ignored
``oracle/_ref`` (it travels with the built library); every test here is skipped when it is
absent.  Nothing of the reference is part of this repository.

* its real Triton quantizers (``veloxvoice/kernels/ops/triton_ops.py:92-124,261-293``), compiled
  for sm_100 by Triton, against ``vx_quantize_pack`` byte for byte on more than 1e7 seeded values
  with exact ties, zero rows and tiny values mixed in (the goldens under tests/golden come from
  the Triton interpreter on a CPU; this is the same comparison with Triton's GPU code);
* its own kernel test bodies (``tests/kernels/test_dgx_mxfp4_gemm.py:66-124``) executed against
  the operators ``install()`` puts in place;
* its own ``DenseLinear`` class with ``precision = "mxfp4"`` running on the installed operators.
"""

import importlib
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

from oracle import make_ref

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not make_ref.available(), reason="oracle/_ref is absent (python oracle/make_ref.py)")]

REF = make_ref.DEST


def _load_file(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref_triton():
    """The reference's Triton quantizer module, loaded from its file (independent of what
    ``install()`` may have put into ``sys.modules``)."""
    pytest.importorskip("triton")
    return _load_file("_velox_ref_triton_ops", os.path.join(REF, "veloxvoice", "kernels", "ops", "triton_ops.py"))


@pytest.fixture()
def installed():
    """``import veloxvoice`` resolves to the copy, with this library's operators installed; the
    replaced modules are dropped again afterwards."""
    from velox_voice_b200 import install

    make_ref.add_to_path()
    before = set(sys.modules)
    install.install()
    yield
    for n in list(sys.modules):
        if n not in before and (n == "veloxvoice" or n.startswith("veloxvoice.") or n.startswith("_velox_ref")):
            del sys.modules[n]


def _mixed_values(rows, K, seed):
    torch.manual_seed(seed)
    x = torch.randn(rows, K, device="cuda") * torch.logspace(-2, 2, rows, device="cuda")[:, None]
    tie = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], device="cuda")
    idx = torch.randint(0, 8, (rows, K), device="cuda")
    x = torch.where(torch.rand_like(x) < 0.05, tie[idx] * torch.sign(x), x)
    x = torch.where(torch.rand_like(x) < 0.01, x * 1e-12, x)
    x[::97] = 0
    x[5::193, : K // 2] = 0
    return x


def test_reference_triton_per_row_quantizer_bytes(ref_triton):
    from velox_voice_b200 import ops

    total = 0
    for rows, K, dtype, seed in ((20480, 512, torch.bfloat16, 1), (3000, 2048, torch.bfloat16, 2), (2048, 512, torch.float32, 3),
                                 (128, 9728, torch.bfloat16, 4), (130, 96, torch.bfloat16, 5)):
        x = _mixed_values(rows, K, seed).to(dtype)
        rq, rs = ref_triton.per_row_col_quantize(x)
        q, s = ops.per_row_col_quantize(x)
        torch.cuda.synchronize()
        assert torch.equal(q, rq), f"codes differ from the reference's Triton kernel ({rows}x{K} {dtype})"
        assert torch.equal(s, rs.view(-1)), f"scale bytes differ ({rows}x{K} {dtype})"
        total += rows * K
    assert total >= 10_000_000


def test_reference_triton_block_quantizer_bytes(ref_triton):
    from velox_voice_b200 import ops

    total = 0
    for rows, K, dtype, seed in ((20480, 512, torch.bfloat16, 6), (1024, 1024, torch.float32, 7), (34, 48, torch.bfloat16, 8)):
        x = _mixed_values(rows, K, seed).to(dtype)
        for mode in "AB":
            rq, rs = ref_triton.mxfp4_block_quantize(x, mode=mode)
            q, s = ops.mxfp4_block_quantize(x, mode=mode)
            torch.cuda.synchronize()
            assert torch.equal(q, rq), f"codes differ (mode {mode}, {rows}x{K} {dtype})"
            assert torch.equal(s, rs), f"scale bytes differ (mode {mode}, {rows}x{K} {dtype})"
            # and the reference's own inverse agrees with this library's
            assert torch.equal(ops.mxfp4_dequant(q, s, mode), ref_triton.mxfp4_dequant(rq, rs, mode))
        total += rows * K
    assert total >= 10_000_000


def test_reference_kernel_test_bodies_through_install(installed):
    """tests/kernels/test_dgx_mxfp4_gemm.py of the reference, imported with the replacement
    operators in place (its module-level skip mark asks for sm_121a; the bodies are called
    directly): bit-exact GEMM on its six shapes, fresh tensors of the same shape, unit scales."""
    mod = _load_file("_velox_ref_test_dgx_mxfp4_gemm", os.path.join(REF, "ref_tests", "test_dgx_mxfp4_gemm.py"))
    from velox_voice_b200 import ops

    assert mod.dgx_mxfp4_gemm is ops.dgx_mxfp4_gemm and mod.quantize_w is ops.quantize_w
    t = mod.TestDgxMxfp4Gemm()
    shapes = None
    for mark in getattr(mod.TestDgxMxfp4Gemm.test_bit_exact_methodology, "pytestmark", []):
        if mark.name == "parametrize":
            shapes = mark.args[1]
    assert shapes and len(shapes) >= 6
    for M, N, K in shapes:
        t.test_bit_exact_methodology(M, N, K)
    t.test_same_shape_new_tensors()
    t.test_unit_scale_parity()


def test_reference_dense_linear_class_on_installed_ops(installed):
    """The reference's own DenseLinear (torch_conformer.py:200-270) in its mxfp4 / nvfp4 lanes:
    pads, quantizes and multiplies through the installed operators; the result is the
    reference's GEMM definition of the same quantized operands plus the bias."""
    from veloxvoice.models.wenet.torch_conformer import DenseLinear  # the reference's class

    from oracle import formats as F
    from oracle import gemm as G

    torch.manual_seed(21)
    w, b = torch.randn(192, 256), torch.randn(192)
    lin = DenseLinear(w, b).cuda()
    x = torch.randn(2, 75, 256, device="cuda")
    xq, xs, _ = F.quantize(x.view(-1, 256).cpu().numpy(), F.FMT_ROWSCALE)
    wq, ws, _ = F.quantize(w.numpy(), F.FMT_ROWSCALE)
    ref = (G.gemm_rowscale_ref(xq, wq, xs, ws) + b.numpy()[None, :]).astype(np.float32)
    for mode in ("mxfp4", "nvfp4"):
        lin.precision = mode
        lin._wq = None
        with torch.no_grad():
            y = lin(x)
        assert y.shape == (2, 75, 192) and y.dtype == torch.float32
        assert np.array_equal(y.view(-1, 192).cpu().numpy(), ref), mode


def test_reference_model_fp4_lane_end_to_end(installed, ref_triton, monkeypatch):
    """The reference's own ``WenetConformerASR`` (random init, full size: d = 512, 12 blocks,
    vocab 5538; no checkpoint exists here) in its mxfp4 lane through ``set_precision`` and
    ``encode_ctc_utterance``, twice on the same features:

      A  every DenseLinear on the operators ``install()`` provides (this library's kernels);
      B  the same model object with the reference's REAL Triton quantizer and the reference's GEMM
         definition (unit-scale dot in exact arithmetic, scales afterwards) in plain torch.

    Gate of the reference's tools for two lanes of one model (``tools/bench_wenet.py:187-236``):
    greedy tokens may diverge in at most max(3, 0.1 %) frames; here they must not diverge at all,
    because quantizer bytes and GEMM results are bit-identical."""
    import veloxvoice.kernels.ops as kops
    from veloxvoice.models.wenet.torch_conformer import DenseLinear

    from oracle import ref_model
    from velox_voice_b200 import ops, synth

    monkeypatch.setenv("VELOXVOICE_ASR_PRECISION", "mxfp4")  # read by DenseLinear / the attention at construction
    state = ref_model.random_state(seed=3)
    model = ref_model.build_reference_asr(state, "cuda:0")
    model.set_jit(False)
    model.set_precision("mxfp4")  # pre-quantizes every DenseLinear weight through the installed quantizer
    n_dense = sum(isinstance(m, DenseLinear) for m in model.encoder.modules()) + 1
    assert n_dense == 12 * 9 + 2
    _, mel = synth.encoder_features(1000, 1500, device="cuda")  # 20 s of the synthetic hour: [2000, 80]
    launches0 = ops.launch_count()
    with torch.inference_mode():
        lp_a = model.encode_ctc_utterance(mel[None]).clone()
    torch.cuda.synchronize()
    assert ops.launch_count() - launches0 >= 2 * n_dense, "the FP4 lane did not run on this library's kernels"
    assert lp_a.shape[0] == 1 and lp_a.shape[2] == 5538 and torch.isfinite(lp_a).all()

    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device="cuda", dtype=torch.float64)

    def unpack(p):
        c = torch.stack([p & 0xF, p >> 4], -1).reshape(p.shape[0], p.shape[1] * 2)
        mag = lut[(c & 7).long()]
        return torch.where((c & 8) > 0, -mag, mag)

    def reference_gemm(pack_a, pack_b, scale_a, scale_b, *args, **kw):
        raw = unpack(pack_a) @ unpack(pack_b).T  # fp64: exact for these operands
        sa = 2.0 ** (scale_a.double() - 127)
        sb = 2.0 ** (scale_b.double() - 127)
        return (raw * sa[:, None] * sb[None, :]).float()

    monkeypatch.setitem(sys.modules, "veloxvoice.kernels.ops.triton_ops", ref_triton)
    monkeypatch.setattr(kops, "dgx_mxfp4_gemm", reference_gemm)
    for m in list(model.encoder.modules()) + [model.ctc_lo]:
        if isinstance(m, DenseLinear):
            m._wq = None  # weights are quantized again, by the reference's Triton kernel
    launches1 = ops.launch_count()
    with torch.inference_mode():
        lp_b = model.encode_ctc_utterance(mel[None])
    torch.cuda.synchronize()
    assert ops.launch_count() == launches1, "lane B must not touch this library"
    tok_a, tok_b = lp_a.argmax(-1), lp_b.argmax(-1)
    n = tok_a.numel()
    diverged = int((tok_a != tok_b).sum())
    print(f"[reference model, {n} frames] token divergence {diverged}, max |dlogp| {(lp_a - lp_b).abs().max().item():.3g}")
    assert diverged <= max(3, n // 1000)
    assert diverged == 0 and (lp_a - lp_b).abs().max().item() < 1e-4


def test_reference_fp4_filterbank_lane_through_install(installed):
    """The front-end's FP4 mel projection, ``power_mel_log_mxfp4`` of the reference
    (``veloxvoice/kernels/ops/cuda_ops.py:149-192``: power spectrum -> ``mxfp4_block_quantize`` ->
    ``dgx_mxfp4_blkscale_gemm`` -> log -> CMVN), executed unchanged on the installed operators and
    compared with the same chain on the CPU oracle (bit-exact product) and with the reference's own
    fp32 formula (``reference_power_mel_log``, FP4 tolerance)."""
    import veloxvoice.kernels.ops.cuda_ops as cu

    from oracle import formats as F
    from oracle import gemm as G
    from velox_voice_b200 import ops

    torch.manual_seed(31)
    T, Fbins, M = 300, 257, 80
    spec = torch.randn(T, Fbins, dtype=torch.complex64, device="cuda") * 100.0
    mel = torch.rand(M, Fbins, device="cuda") * (torch.rand(M, Fbins, device="cuda") < 0.1)
    F_padded, M_padded = 320, 128
    mel_p = torch.zeros(M_padded, F_padded, device="cuda")
    mel_p[:M, :Fbins] = mel
    mel_codes, mel_scales = ops.mxfp4_block_quantize(mel_p, mode="B")
    mean, istd = torch.randn(M, device="cuda"), torch.rand(M, device="cuda") + 0.5
    out = cu.power_mel_log_mxfp4(spec, mel_codes, mel_scales, mean, istd, F_padded, M_padded)
    assert out.shape == (T, M) and out.dtype == torch.float32 and torch.isfinite(out).all()
    # oracle: same quantizers, block-scaled product of the dequantized operands, log, CMVN
    power = (spec.real ** 2 + spec.imag ** 2).cpu().numpy()
    pp = np.zeros((384, F_padded), dtype=np.float32)
    pp[:T, :Fbins] = power
    aq, asc, _ = F.quantize(pp, F.FMT_BLK16_A)
    bq, bsc, _ = F.quantize(mel_p.cpu().numpy(), F.FMT_BLK16_B)
    assert np.array_equal(bq, mel_codes.cpu().numpy()) and np.array_equal(bsc, mel_scales.cpu().numpy())
    acc = G.gemm_ref(F.FMT_BLK16_A, aq, asc, bq, bsc)[:T, :M]
    ref = (np.log(np.maximum(acc, np.float32(1.1920929e-7))) - mean.cpu().numpy()[None, :]) * istd.cpu().numpy()[None, :]
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-4
    # against the unquantized formula of the reference: FP4 noise only
    full = cu.reference_power_mel_log(spec.real, spec.imag, mel, mean, istd)
    nz = (mel.sum(1) > 0).cpu().numpy()
    assert np.median(np.abs(out.cpu().numpy() - full.cpu().numpy())[:, nz]) < 0.2


def test_reference_filterbank_test_bodies_through_install(installed):
    """tests/kernels/test_power_mel_log.py of the reference (class TestPowerMelLogBf16), imported with
    ``power_mel_log`` / ``reference_power_mel_log`` replaced by this library's: its tf32-emulation
    comparisons, CMVN, real filterbank vs fp32, tiny and odd frame counts, shape and finiteness."""
    mod = _load_file("_velox_ref_test_power_mel_log", os.path.join(REF, "ref_tests", "test_power_mel_log.py"))
    from velox_voice_b200 import ops

    assert mod.power_mel_log is ops.power_mel_log and mod.reference_power_mel_log is ops.reference_power_mel_log
    t = mod.TestPowerMelLogBf16()
    before = ops.launch_count()
    t.test_matches_tf32_truncation_emulation()
    t.test_matches_emulation_various_sizes()
    t.test_with_cmvn()
    if mod._real_mel_fbank_available():
        t.test_real_mel_fbank_matches_fp32()
    t.test_tiny_input()
    # test_various_T_values (:180-192) bounds the single worst element of a random-sign filterbank by 3e-2
    # against its cuBLAS-chunked emulation: at cancellation points that bound depends on the summation
    # order of the hardware (one element of T = 256 measures 0.038 here, closer to the exactly summed tf32
    # product than the emulation is).  Same inputs, the file's own noise-aware criterion (:90-116) instead;
    # the fp32 lane below 64 frames keeps the 3e-2 bound.
    torch.manual_seed(2)
    for T in [1, 8, 16, 32, 64, 98, 127, 128, 256]:
        spec = torch.randn(T, 257, device="cuda", dtype=torch.cfloat)
        mel = torch.randn(80, 257, device="cuda", dtype=torch.float32)
        ref = mod.reference_for_dispatch(spec, mel)
        out = mod.power_mel_log(spec, mel, None, None)
        assert out.shape == (T, 80)
        if T >= 64:
            mod._assert_close(out, ref)
        else:
            assert (out - ref).abs().max().item() < 3e-2
    t.test_output_shape()
    t.test_numerical_stability()
    assert ops.launch_count() > before  # the kernel ran, not only the fp32 lane

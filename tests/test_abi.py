"""The C-ABI shared library: it loads without a GPU, exports every symbol the public header
declares, and rejects bad arguments before touching a device."""

import ctypes as C
import os
import re

import pytest

from velox_voice_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def _declared_symbols():
    with open(os.path.join(ROOT, "include", "velox_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vx_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_in_tree():
    assert os.path.exists(build.LIB_PATH)
    assert os.path.dirname(build.LIB_PATH).startswith(ROOT)


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/velox_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_abi_version_and_struct_size(lib):
    assert lib.vx_abi_version() == 6
    assert C.sizeof(_lib.GemmDesc) == 256


def test_sf_geometry(lib):
    # mx32: 2 atoms per 256-wide K stage; 16-blocks: 4 atoms per stage
    assert lib.vx_sf_kgroups(_lib.FMT_MX32, 512) == 4
    assert lib.vx_sf_kgroups(_lib.FMT_NV16, 512) == 8
    assert lib.vx_sf_kgroups(_lib.FMT_BLK16_A, 64) == 4
    assert lib.vx_sf_kgroups(_lib.FMT_ROWSCALE, 512) == 0
    assert lib.vx_sf_bytes(_lib.FMT_MX32, 1024, 512) == 8 * 4 * 512
    assert lib.vx_sf_bytes(_lib.FMT_MX32, 1025, 512) == 9 * 4 * 512


def test_argument_errors_do_not_need_a_device(lib):
    assert lib.vx_bsgemm(None, None) == -1
    assert b"desc" in lib.vx_last_error()
    d = _lib.GemmDesc()
    d.struct_size = 8
    assert lib.vx_bsgemm(C.byref(d), None) == -1
    assert b"struct_size" in lib.vx_last_error()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = 99
    assert lib.vx_bsgemm(C.byref(d), None) == -1
    # quantizer: unknown format, bad dtype, K not a multiple of the block
    assert lib.vx_quantize_pack(C.c_void_p(256), 1, 4, 64, 64, 42, C.c_void_p(256), 32, None, None, None, None) == -1
    assert lib.vx_quantize_pack(C.c_void_p(256), 7, 4, 64, 64, 0, C.c_void_p(256), 32, None, None, None, None) == -1
    assert lib.vx_quantize_pack(C.c_void_p(256), 1, 4, 48, 48, _lib.FMT_MX32, C.c_void_p(256), 24, None, None, None, None) == -1
    assert b"multiple" in lib.vx_last_error()
    # misaligned rows
    assert lib.vx_quantize_pack(C.c_void_p(258), 1, 4, 64, 64, 0, C.c_void_p(256), 32, None, None, None, None) == -1
    # NV16 without the tensor amax
    assert lib.vx_quantize_pack(C.c_void_p(256), 1, 4, 64, 64, _lib.FMT_NV16, C.c_void_p(256), 32, None, None, None, None) == -1
    # empty problems are a no-op
    assert lib.vx_quantize_pack(None, 1, 0, 64, 64, 0, None, 32, None, None, None, None) == 0
    # filterbank projection: shape limits, NULL operands, misaligned spectrum, one-sided CMVN
    assert lib.vx_power_mel_log_supported(257, 80) == 1 and lib.vx_power_mel_log_supported(513, 80) == 1
    assert lib.vx_power_mel_log_supported(257, 257) == 0 and lib.vx_power_mel_log_supported(4096, 256) == 0
    mel_args = lambda **k: [k.get("spec", C.c_void_p(256)), k.get("T", 8), k.get("F", 64), k.get("ld", 64), k.get("mel", C.c_void_p(512)),
                            k.get("M", 16), 64, k.get("mean", None), None, C.c_void_p(1024), k.get("ldo", 16), None]
    assert lib.vx_power_mel_log(*mel_args(T=0)) == 0
    assert lib.vx_power_mel_log(*mel_args(M=300, ldo=300)) == -1 and b"256" in lib.vx_last_error()
    assert lib.vx_power_mel_log(*mel_args(spec=None)) == -1
    assert lib.vx_power_mel_log(*mel_args(spec=C.c_void_p(260))) == -1 and b"aligned" in lib.vx_last_error()
    assert lib.vx_power_mel_log(*mel_args(mean=C.c_void_p(2048))) == -1 and b"together" in lib.vx_last_error()
    assert lib.vx_power_mel_log(*mel_args(ld=32)) == -1
    assert lib.vx_power_mel_log(*mel_args(ldo=8)) == -1
    # CTC top-k helpers: k range, NULL arguments
    assert lib.vx_ctc_topk_threshold(C.c_void_p(256), 5538, 0, 5, C.c_void_p(512), None) == 0
    assert lib.vx_ctc_topk_threshold(C.c_void_p(256), 5538, 8, 17, C.c_void_p(512), None) == -1
    assert lib.vx_ctc_topk_threshold(None, 5538, 8, 5, C.c_void_p(512), None) == -1
    assert lib.vx_ctc_topk_threshold(C.c_void_p(256), 100, 8, 9, C.c_void_p(512), None) == -1  # 8 groups of 64 columns only
    assert lib.vx_ctc_topk_finish(C.c_void_p(256), C.c_void_p(512), 4, C.c_void_p(768), 5538, 8, 5, C.c_void_p(1024),
                                  C.c_void_p(1280), C.c_void_p(1536), None) == -1  # capacity < k
    # attention: head dimension, NULL operands, alignment
    assert lib.vx_relpos_attention(C.c_void_p(256), C.c_void_p(512), C.c_void_p(768), 0, 8, 64, 0, C.c_void_p(1024), 512, None) == 0
    assert lib.vx_relpos_attention(C.c_void_p(256), C.c_void_p(512), C.c_void_p(768), 16, 8, 32, 0, C.c_void_p(1024), 512, None) == -1
    assert b"head_dim" in lib.vx_last_error()
    assert lib.vx_relpos_attention(None, C.c_void_p(512), C.c_void_p(768), 16, 8, 64, 0, C.c_void_p(1024), 512, None) == -1
    assert lib.vx_relpos_attention(C.c_void_p(258), C.c_void_p(512), C.c_void_p(768), 16, 8, 64, 0, C.c_void_p(1024), 512, None) == -1
    assert lib.vx_relpos_attention(C.c_void_p(256), C.c_void_p(512), C.c_void_p(768), 16, 8, 64, 0, C.c_void_p(1024), 100, None) == -1


def _gemm_desc(lib, fmt=_lib.FMT_MX32, epi=_lib.EPI_NONE, flags=0):
    """A descriptor whose pointers are never dereferenced: argument checks come before any launch."""
    d = _lib.GemmDesc()
    d.struct_size = C.sizeof(_lib.GemmDesc)
    d.fmt = fmt
    d.M, d.N, d.K = 128, 1536, 512
    d.a_codes, d.b_codes, d.lda, d.ldb = 4096, 8192, 256, 256
    d.a_scales, d.b_scales = 12288, 16384
    d.out, d.ldo, d.out_dtype = 20480, 1536, _lib.DT_BF16
    d.epilogue, d.flags = epi, flags
    return d


def test_gemm_rejects_what_it_cannot_run_before_any_launch(lib):
    # the fold-pack epilogue has no per-row-scaled route: an argument error, not a launch
    d = _gemm_desc(lib, fmt=_lib.FMT_ROWSCALE, epi=_lib.EPI_BIAS_QKVPACK)
    d.heads, d.head_dim, d.ldo = 8, 64, 128
    d.pos_u, d.pos_v = 24576, 28672
    assert lib.vx_bsgemm(C.byref(d), None) == -1
    assert b"QKVPACK" in lib.vx_last_error()
    # unknown flag bits (anything above the documented VX_GEMM_* values)
    for bad in (1 << 8, 1 << 9, 1 << 20, 32):
        d = _gemm_desc(lib, flags=bad)
        assert lib.vx_bsgemm(C.byref(d), None) == -1
        assert b"flags" in lib.vx_last_error()
    # the top-k candidate pass goes with the log-sum-exp partials and a sane capacity
    d = _gemm_desc(lib, epi=_lib.EPI_BIAS_ARGMAX)
    d.out_dtype, d.ldo = _lib.DT_F32, 1
    d.topk_threshold, d.topk_candidates, d.topk_count, d.topk_capacity = 32768, 36864, 40960, 64
    assert lib.vx_bsgemm(C.byref(d), None) == -1 and b"top-k" in lib.vx_last_error()  # no lse_partials
    d.lse_partials, d.topk_capacity = 45056, 1000
    assert lib.vx_bsgemm(C.byref(d), None) == -1 and b"top-k" in lib.vx_last_error()
    # the residual GEMM with the LayerNorm + quantizer behind it: MX32, N = 512, K % 256 == 0, bf16 in and out
    assert lib.vx_bsgemm_residual_ln_supported(_lib.FMT_MX32, 512, 512) == 1
    assert lib.vx_bsgemm_residual_ln_supported(_lib.FMT_MX32, 512, 2048) == 1
    assert lib.vx_bsgemm_residual_ln_supported(_lib.FMT_NV16, 512, 512) == 0
    assert lib.vx_bsgemm_residual_ln_supported(_lib.FMT_MX32, 1536, 512) == 0
    assert lib.vx_bsgemm_residual_ln_supported(_lib.FMT_MX32, 512, 384) == 0
    vp = C.c_void_p
    d = _gemm_desc(lib, epi=_lib.EPI_BIAS_RESIDUAL)  # N = 1536
    assert lib.vx_bsgemm_residual_ln(C.byref(d), vp(256), vp(512), 1e-5, vp(1024), 256, vp(2048), None) == -1
    d.N, d.ldo, d.residual, d.ldr, d.residual_dtype = 512, 512, 24576, 512, _lib.DT_F32
    assert lib.vx_bsgemm_residual_ln(C.byref(d), vp(256), vp(512), 1e-5, vp(1024), 256, vp(2048), None) == -1  # f32 residual
    assert b"bf16" in lib.vx_last_error()
    d.residual_dtype = _lib.DT_BF16
    assert lib.vx_bsgemm_residual_ln(C.byref(d), None, vp(512), 1e-5, vp(1024), 256, vp(2048), None) == -1  # no gamma
    assert lib.vx_bsgemm_residual_ln(C.byref(d), vp(256), vp(512), 1e-5, vp(1024), 100, vp(2048), None) == -1  # ldc
    assert lib.vx_bsgemm_residual_ln(C.byref(d), vp(256), vp(512), 1e-5, vp(1024), 256, None, None) == -1  # no scale factors
    assert lib.vx_bsgemm_residual_ln2(C.byref(d), vp(256), vp(512), None, vp(768), 1e-5, vp(1024), 256, vp(2048), None) == -1
    assert lib.vx_bsgemm_residual_ln2(C.byref(d), vp(256), vp(512), vp(768), vp(1024), 1e-5, vp(1024), 100, vp(2048), None) == -1
    d.M = 0
    assert lib.vx_bsgemm_residual_ln(C.byref(d), vp(256), vp(512), 1e-5, vp(1024), 256, vp(2048), None) == 0  # nothing to do
    assert lib.vx_bsgemm_residual_ln2(C.byref(d), vp(256), vp(512), vp(768), vp(1024), 1e-5, vp(1024), 256, vp(2048), None) == 0
    # the bounded-wait self-test takes a limit of at most 100 ms and a site below 255
    assert lib.vx_wait_selftest(0, 1, None) == -1
    assert lib.vx_wait_selftest(10**9, 1, None) == -1
    assert lib.vx_wait_selftest(1000, 255, None) == -1


def test_host_wrappers_validate_operands_without_a_device():
    import torch

    from velox_voice_b200 import ops

    cpu_q = ops.Quantized(_lib.FMT_MX32, 4, 64, torch.zeros(4, 32, dtype=torch.uint8), None,
                          torch.zeros(1, 2, 512, dtype=torch.uint8), None)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.bsgemm(cpu_q, cpu_q)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.bsgemm_argmax(cpu_q, cpu_q)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.bsgemm_heads(cpu_q, cpu_q, None, torch.zeros(1, 4, 64, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.bsgemm_qkv_pack(cpu_q, cpu_q, None, torch.zeros(1, 64), torch.zeros(1, 64), 1.0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.qkv_pack(torch.zeros(4, 192, dtype=torch.bfloat16), torch.zeros(4, 64, dtype=torch.bfloat16),
                     torch.zeros(1, 64), torch.zeros(1, 64), 1.0)
    other = ops.Quantized(_lib.FMT_NV16, 4, 64, cpu_q.codes, None, cpu_q.sf, None)
    with pytest.raises(ValueError, match="formats differ"):
        ops.bsgemm_heads(cpu_q, other, None, torch.zeros(1, 4, 64, dtype=torch.bfloat16))
    wider = ops.Quantized(_lib.FMT_MX32, 4, 128, torch.zeros(4, 64, dtype=torch.uint8), None, cpu_q.sf, None)
    with pytest.raises(ValueError, match="K mismatch"):
        ops.bsgemm_heads(cpu_q, wider, None, torch.zeros(1, 4, 64, dtype=torch.bfloat16))
    # the bf16 operator names keep the reference's convention: None means "not taken, fall back"
    assert ops.fused_qkv_wgmma(torch.zeros(64, 512), torch.zeros(1536, 512), torch.zeros(1536)) is None
    assert ops.pwlin_glu(torch.zeros(64, 512, dtype=torch.bfloat16), torch.zeros(1024, 512), torch.zeros(1024)) is None
    x = torch.randn(3, 8)
    w, b = torch.randn(6, 8), torch.randn(6)
    assert torch.allclose(ops.fused_qkv(x, w, b), torch.nn.functional.linear(x, w, b))


def test_model_side_helpers_follow_the_reference_rules():
    import numpy as np
    import torch

    from oracle import formats as F
    from velox_voice_b200 import ops

    torch.manual_seed(0)
    w = torch.randn(16, 64) * 2
    w[0, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, -0.25, -1e-9])
    codes = ops._encode_codes(w)
    assert np.array_equal(codes.numpy(), F.e2m1_encode(w.numpy()))
    assert np.array_equal(ops.decode_codes(torch.from_numpy(F.pack_codes(codes.numpy()))).numpy(), codes.numpy())
    assert ops.ue8m0_to_float(127) == 1.0 and ops.ue8m0_to_float(130) == 8.0
    assert ops.ue8m0_from_scale(1.0) == 127 and ops.ue8m0_from_scale(0.3) == 126 and ops.ue8m0_from_scale(0.0) == 0x80
    assert ops.ue8m0_from_scale(3.9) == 128 and ops.ue8m0_from_scale(1e-60) == 0


def test_ops_refuse_cpu_tensors():
    import torch

    from velox_voice_b200 import ops

    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.quantize(torch.zeros(4, 64), "mx32")
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.per_row_col_quantize(torch.zeros(4, 64))


def test_install_wires_reference_import_names():
    import sys

    from velox_voice_b200 import install, ops

    mods = install.install(patch_modules=False)
    tri = sys.modules["veloxvoice.kernels.ops.triton_ops"]
    assert tri.per_row_col_quantize is ops.per_row_col_quantize
    assert tri.triton_quantize_w is ops.triton_quantize_w
    assert tri.mxfp4_block_quantize is ops.mxfp4_block_quantize
    assert sys.modules["veloxvoice.models.wenet.mxfp4_linear"]._pad16 is ops._pad16
    assert "veloxvoice.models.wenet.nvfp4_linear" in mods
    nv = sys.modules["veloxvoice.models.wenet.nvfp4_linear"]
    for name in ("CODE_LUT", "_encode_codes", "dequantize_w", "pack_codes", "quantize_w", "ue8m0_from_scale",
                 "ue8m0_to_float", "decode_codes", "quantize_and_gemm", "Nvfp4Linear", "nvfp4_gemm"):
        assert hasattr(nv, name), name  # what the reference's kernel test imports (tests/kernels/test_dgx_mxfp4_gemm.py:24-32)
    for name in ("fused_qkv", "fused_qkv_wgmma", "pwlin_glu", "qkv_pack", "dgx_mxfp4_gemm", "power_mel_log", "reference_power_mel_log"):
        assert name in install.OPS_PKG_NAMES
    for n in ("veloxvoice.kernels.ops.triton_ops", "veloxvoice.models.wenet.mxfp4_linear", "veloxvoice.models.wenet.nvfp4_linear"):
        del sys.modules[n]


def test_pad16_matches_call_site_contract():
    import torch

    from velox_voice_b200 import ops

    t = torch.arange(10.0).reshape(5, 2)
    p = ops._pad16(t, 4)
    assert p.shape == (8, 2) and torch.equal(p[:5], t) and not p[5:].any()
    assert ops._pad16(t[:4], 4) is not None and ops._pad16(t[:4], 4).shape == (4, 2)

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
    assert lib.vx_abi_version() == 2
    assert C.sizeof(_lib.GemmDesc) == 216


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
    for n in ("veloxvoice.kernels.ops.triton_ops", "veloxvoice.models.wenet.mxfp4_linear", "veloxvoice.models.wenet.nvfp4_linear"):
        del sys.modules[n]


def test_pad16_matches_call_site_contract():
    import torch

    from velox_voice_b200 import ops

    t = torch.arange(10.0).reshape(5, 2)
    p = ops._pad16(t, 4)
    assert p.shape == (8, 2) and torch.equal(p[:5], t) and not p[5:].any()
    assert ops._pad16(t[:4], 4) is not None and ops._pad16(t[:4], 4).shape == (4, 2)

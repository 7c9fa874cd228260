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
        y = lin(x)
        assert y.shape == (2, 75, 192) and y.dtype == torch.float32
        assert np.array_equal(y.view(-1, 192).cpu().numpy(), ref), mode

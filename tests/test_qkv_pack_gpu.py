"""Attention fold pack on the GPU against the oracle (bit-exact: bf16 elementwise work)."""

import numpy as np
import pytest
import torch

from oracle import gemm as G

pytestmark = pytest.mark.gpu


def _case(T, h, dk, seed=0):
    torch.manual_seed(seed)
    d = h * dk
    qkv = (torch.randn(T, 3 * d) * 2).bfloat16()
    p0 = torch.randn(T, d).bfloat16()
    u, v = torch.randn(h, dk).bfloat16(), torch.randn(h, dk).bfloat16()
    return qkv, p0, u, v, dk ** -0.5


@pytest.mark.parametrize("T,h,dk", [(1, 8, 64), (77, 8, 64), (1000, 4, 32), (300, 8, 64)])
def test_qkv_pack_kernel_equals_the_oracle(T, h, dk):
    from velox_voice_b200 import ops

    qkv, p0, u, v, scale = _case(T, h, dk)
    got = ops.qkv_pack(qkv.cuda(), p0.cuda(), u.cuda(), v.cuda(), scale)
    want = G.qkv_pack_ref(qkv.float().numpy(), p0.float().numpy(), u.float().numpy(), v.float().numpy(), scale, h)
    for g, w in zip(got, want):
        assert g.shape == w.shape and g.dtype == torch.bfloat16 and g.is_contiguous()
        assert np.array_equal(g.float().cpu().numpy(), w)


def test_qkv_pack_takes_a_strided_qkv():
    from velox_voice_b200 import ops

    qkv, p0, u, v, scale = _case(130, 8, 64, seed=1)
    wide = torch.zeros(130, 3 * 512 + 64, dtype=torch.bfloat16, device="cuda")
    wide[:, : 3 * 512] = qkv.cuda()
    a = ops.qkv_pack(wide[:, : 3 * 512], p0.cuda(), u.cuda(), v.cuda(), scale)
    b = ops.qkv_pack(qkv.cuda(), p0.cuda(), u.cuda(), v.cuda(), scale)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("fmt", ["mx32", "nv16", "fp8_1x128"])
@pytest.mark.parametrize("T", [300, 1000])
def test_fused_qkv_projection_writes_the_fold_pack(fmt, T):
    """QKV GEMM with the pack epilogue + the positional projection written head-major ==
    qkv_pack of the same two GEMMs' ordinary bf16 outputs, bit for bit."""
    from velox_voice_b200 import ops

    torch.manual_seed(4)
    h, dk, K = 8, 64, 512
    d = h * dk
    x = torch.randn(T, K, device="cuda").bfloat16()
    pos = torch.randn(T, K, device="cuda").bfloat16()
    wqkv = 0.05 * torch.randn(3 * d, K, device="cuda")
    wlp = 0.05 * torch.randn(d, K, device="cuda")
    bias = 0.1 * torch.randn(3 * d, device="cuda")
    u, v = torch.randn(h, dk, device="cuda").bfloat16(), torch.randn(h, dk, device="cuda").bfloat16()
    am = {"amax_t": torch.tensor([6.0], device="cuda")} if fmt == "nv16" else {}
    a, ap = ops.quantize(x, fmt, **am), ops.quantize(pos, fmt, **am)
    wq, wl = ops.quantize(wqkv, fmt), ops.quantize(wlp, fmt)
    scale = dk ** -0.5

    qkv = ops.bsgemm(a, wq, epilogue=ops.EPI_BIAS, bias=bias, out_dtype=torch.bfloat16)
    p0 = ops.bsgemm(ap, wl, out_dtype=torch.bfloat16)
    want = ops.qkv_pack(qkv, p0, u, v, scale)

    packed = torch.full((3, h, T, 2 * dk), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.bsgemm_qkv_pack(a, wq, bias, u, v, scale, packed=packed)
    ops.bsgemm_heads(ap, wl, None, packed[1], col_off=dk)
    torch.cuda.synchronize()
    for i, name in enumerate(("q2", "k2", "v2")):
        assert torch.equal(packed[i], want[i]), name

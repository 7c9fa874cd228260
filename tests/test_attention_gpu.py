"""vx_relpos_attention (tcgen05 bf16 attention on the fold pack) against the CPU oracle and torch SDPA."""

import numpy as np
import pytest
import torch

from oracle import attention as A

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from velox_voice_b200 import ops as o

    return o


def _inputs(h, T, dk, seed, spread=1.0):
    torch.manual_seed(seed)
    q2 = (torch.randn(h, T, 2 * dk, device="cuda") * 0.25 * spread).bfloat16()
    k2 = torch.randn(h, T, 2 * dk, device="cuda").bfloat16()
    v2 = torch.cat([torch.randn(h, T, dk, device="cuda"), torch.zeros(h, T, dk, device="cuda")], dim=-1).bfloat16()
    return q2, k2, v2


@pytest.mark.parametrize("T,kv_len", [(1, None), (64, None), (128, None), (129, None), (300, None), (1000, 777), (3750, None)])
def test_attention_matches_the_oracle(ops, T, kv_len):
    """bf16 operands, fp32 accumulation, probabilities rounded to bf16 before the second product and a bf16
    result: 2e-2 of the largest output value (north star: 1e-2 relative on bf16 GEMM outputs; the bf16
    rounding of P adds its own 2^-9)."""
    h, dk = 8, 64
    q2, k2, v2 = _inputs(h, T, dk, seed=T)
    out = ops.relpos_attention(q2, k2, v2, kv_len=kv_len)
    torch.cuda.synchronize()
    assert out.shape == (T, h * dk) and out.dtype == torch.bfloat16
    ref = A.relpos_attention_ref(q2.float().cpu().numpy(), k2.float().cpu().numpy(), v2.float().cpu().numpy(), kv_len)
    got = out.float().cpu().numpy()
    err = np.abs(got - ref).max() / np.abs(ref).max()
    print(f"[T={T}, kv_len={kv_len}] max err / max |ref| = {err:.3g}")
    assert np.isfinite(got).all() and err < 2e-2


def test_attention_peaked_rows_and_torch_sdpa(ops):
    """Large logits (a peaked softmax: the row maximum must come out exactly) and agreement with the call the
    model makes, scaled_dot_product_attention on the same bf16 tensors."""
    h, T, dk = 8, 515, 64
    q2, k2, v2 = _inputs(h, T, dk, seed=3, spread=6.0)
    out = ops.relpos_attention(q2, k2, v2)
    x = torch.nn.functional.scaled_dot_product_attention(q2[None], k2[None], v2[None], scale=1.0)[..., :dk]
    want = x.transpose(1, 2).reshape(T, h * dk)
    ref = A.relpos_attention_ref(q2.float().cpu().numpy(), k2.float().cpu().numpy(), v2.float().cpu().numpy())
    scale = np.abs(ref).max()
    assert np.abs(out.float().cpu().numpy() - ref).max() / scale < 2e-2
    assert (out.float() - want.float()).abs().max().item() / scale < 3e-2


def test_attention_consumes_the_fold_pack(ops):
    """qkv_pack -> relpos_attention equals the model's chain on the unpacked projection."""
    from oracle import gemm as G

    torch.manual_seed(8)
    T, h, dk = 333, 8, 64
    d = h * dk
    qkv = (torch.randn(T, 3 * d, device="cuda") * 0.5).bfloat16()
    p0 = (torch.randn(T, d, device="cuda") * 0.5).bfloat16()
    pos_u, pos_v = (torch.randn(h, dk, device="cuda") * 0.1).bfloat16(), (torch.randn(h, dk, device="cuda") * 0.1).bfloat16()
    q2, k2, v2 = ops.qkv_pack(qkv, p0, pos_u, pos_v, dk ** -0.5)
    out = ops.relpos_attention(q2, k2, v2)
    rq, rk, rv = G.qkv_pack_ref(qkv.float().cpu().numpy(), p0.float().cpu().numpy(), pos_u.float().cpu().numpy(),
                                pos_v.float().cpu().numpy(), dk ** -0.5, h)
    ref = A.relpos_attention_ref(rq, rk, rv)
    assert np.abs(out.float().cpu().numpy() - ref).max() / np.abs(ref).max() < 2e-2


def test_attention_argument_errors(ops):
    q2, k2, v2 = _inputs(8, 16, 64, seed=0)
    with pytest.raises(ValueError):
        ops.relpos_attention(q2, k2[:, :8], v2)
    with pytest.raises(ValueError):
        ops.relpos_attention(q2[..., :64].contiguous(), k2[..., :64].contiguous(), v2[..., :64].contiguous())
    with pytest.raises(ValueError):
        ops.relpos_attention(q2.float(), k2.float(), v2.float())

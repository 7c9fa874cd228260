"""The attention oracle against the reference model's own torch formulation (CPU)."""

import numpy as np
import torch

from oracle import attention as A


def _torch_attention_chain(q2, k2, v2, dk, mask=None):
    """veloxvoice/models/wenet/torch_conformer.py:514-519 for n = 1 on the folded tensors [h, T, 2 dk]."""
    x = torch.nn.functional.scaled_dot_product_attention(q2[None], k2[None], v2[None], attn_mask=mask, scale=1.0)
    x = x[..., :dk]
    return x.transpose(1, 2).reshape(1, -1, q2.shape[0] * dk)[0]


def test_oracle_attention_equals_the_torch_formulation():
    torch.manual_seed(0)
    h, T, dk = 8, 150, 64
    q2 = torch.randn(h, T, 2 * dk) * 0.3
    k2 = torch.randn(h, T, 2 * dk)
    v2 = torch.cat([torch.randn(h, T, dk), torch.zeros(h, T, dk)], dim=-1)
    want = _torch_attention_chain(q2, k2, v2, dk).numpy()
    got = A.relpos_attention_ref(q2.numpy(), k2.numpy(), v2.numpy())
    assert got.shape == (T, h * dk)
    assert np.abs(got - want).max() < 1e-5
    # a padded span: keys beyond kv_len masked (boolean key mask in the torch call)
    n = 97
    mask = torch.zeros(1, 1, T, T, dtype=torch.bool)
    mask[..., :n] = True
    want = _torch_attention_chain(q2, k2, v2, dk, mask).numpy()
    got = A.relpos_attention_ref(q2.numpy(), k2.numpy(), v2.numpy(), kv_len=n)
    assert np.abs(got - want).max() < 1e-5

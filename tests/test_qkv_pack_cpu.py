"""The oracle's attention fold chain against the reference model's own torch formulation."""

import numpy as np
import torch

from oracle import gemm as G


def _torch_fold_chain(qkv, p_raw, pos_u, pos_v, scale, h):
    """veloxvoice/models/wenet/torch_conformer.py:488-510 for n = n_pos = 1, bf16 tensors."""
    d = qkv.shape[-1] // 3
    dk = d // h
    n = 1
    qkv = qkv[None]
    q, k, v = (qkv[:, :, :d].view(n, -1, h, dk), qkv[:, :, d:2 * d].view(n, -1, h, dk), qkv[:, :, 2 * d:].view(n, -1, h, dk))
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    p = p_raw[None].view(1, -1, h, dk).transpose(1, 2)
    u = pos_u.view(1, h, 1, dk)
    vb = pos_v.view(1, h, 1, dk)
    q = torch.cat([(q + u), (q + vb)], dim=-1) * scale
    k = torch.cat([k, p], dim=-1)
    v = torch.cat([v, torch.zeros_like(v)], dim=-1)
    return q[0], k[0], v[0]


def test_oracle_fold_chain_equals_the_torch_formulation():
    torch.manual_seed(0)
    T, h, dk = 77, 8, 64
    d = h * dk
    qkv = (torch.randn(T, 3 * d) * 2).bfloat16()
    p0 = torch.randn(T, d).bfloat16()
    pos_u, pos_v = torch.randn(h, dk).bfloat16(), torch.randn(h, dk).bfloat16()
    scale = dk ** -0.5
    want = _torch_fold_chain(qkv, p0, pos_u, pos_v, scale, h)
    got = G.qkv_pack_ref(qkv.float().numpy(), p0.float().numpy(), pos_u.float().numpy(), pos_v.float().numpy(), scale, h)
    for w, g in zip(want, got):
        assert w.shape == g.shape
        assert np.array_equal(w.float().numpy(), g)

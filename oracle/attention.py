"""TEST INFRASTRUCTURE: CPU restatement of the encoder's attention on the fold pack.

``x = scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=1.0)[..., :head_dim]`` then
``x.transpose(1, 2).reshape(n, -1, d)`` (``veloxvoice/models/wenet/torch_conformer.py:514-519``) with
``q = ((q + u) | (q + v)) * scale``, ``k = k | p``, ``v = v | 0`` (``:488-510``): plain fp32 matmul, softmax over the
keys, matmul.  Pinned by running the reference module's own chain (torch CPU,
``tests/test_attention_cpu.py``).  Only tests and the smoke check may import this module.
"""

from __future__ import annotations

import numpy as np


def relpos_attention_ref(q2: np.ndarray, k2: np.ndarray, v2: np.ndarray, kv_len=None) -> np.ndarray:
    """q2, k2, v2 [h, T, 2 dk] -> [T, h dk] (fp32 throughout); keys >= kv_len masked."""
    q2 = np.asarray(q2, np.float32)
    k2 = np.asarray(k2, np.float32)
    v2 = np.asarray(v2, np.float32)
    h, T, d2 = q2.shape
    dk = d2 // 2
    n = T if kv_len is None or kv_len <= 0 or kv_len > T else int(kv_len)
    out = np.empty((T, h * dk), np.float32)
    for i in range(h):
        s = q2[i] @ k2[i, :n].T
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[:, i * dk:(i + 1) * dk] = p @ v2[i, :n, :dk]
    return out

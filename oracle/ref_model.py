"""A random-init instance of the REFERENCE's own model class.  TEST INFRASTRUCTURE.

No WeNet checkpoint exists in this repository or in its build container, so the end-to-end
drop-in test builds ``WenetConformerASR`` (``veloxvoice/models/wenet/torch_conformer.py:748-843``)
from a synthetic state dict: every tensor the constructors read, with the checkpoint's key names
and shapes, filled from a seeded generator.  The class comes from the copy of the reference
package in ``oracle/_ref`` (``oracle/make_ref.py``); nothing of it is restated here.
"""

from __future__ import annotations

import math
from typing import Dict

import torch

from . import make_ref


def random_state(d: int = 512, heads: int = 8, ffn: int = 2048, blocks: int = 12, kernel: int = 15, vocab: int = 5538,
                 mel: int = 80, max_len: int = 5000, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Checkpoint-shaped tensors (CPU fp32).  Linear / conv weights ~ N(0, 1/fan_in), LayerNorm
    affine near identity, sinusoidal position table, CMVN = identity."""
    g = torch.Generator().manual_seed(seed)

    def w(*shape, fan_in=None):
        fan_in = fan_in or shape[-1]
        return torch.randn(*shape, generator=g) / math.sqrt(fan_in)

    def ln(prefix, st):
        st[prefix + ".weight"] = 1.0 + 0.1 * torch.randn(d, generator=g)
        st[prefix + ".bias"] = 0.1 * torch.randn(d, generator=g)

    st: Dict[str, torch.Tensor] = {}
    f2 = ((mel - 1) // 2 - 1) // 2  # frequency bins left after the two stride-2 convolutions
    st["encoder.embed.conv.0.weight"] = w(d, 1, 3, 3, fan_in=9)
    st["encoder.embed.conv.0.bias"] = 0.1 * torch.randn(d, generator=g)
    st["encoder.embed.conv.2.weight"] = w(d, d, 3, 3, fan_in=9 * d)
    st["encoder.embed.conv.2.bias"] = 0.1 * torch.randn(d, generator=g)
    st["encoder.embed.out.0.weight"] = w(d, d * f2)
    st["encoder.embed.out.0.bias"] = 0.1 * torch.randn(d, generator=g)
    pos = torch.arange(max_len, dtype=torch.float32)[:, None]
    div = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * -(math.log(10000.0) / d))
    pe = torch.zeros(max_len, d)
    pe[:, 0::2] = torch.sin(pos * div)
    pe[:, 1::2] = torch.cos(pos * div)
    st["encoder.embed.pos_enc.pe"] = pe[None]
    dk = d // heads
    for i in range(blocks):
        p = f"encoder.encoders.{i}."
        for n in ("norm_ff", "norm_mha", "norm_conv", "norm_ff_macaron", "norm_final"):
            ln(p + n, st)
        for ff in ("feed_forward", "feed_forward_macaron"):
            st[p + ff + ".w_1.weight"], st[p + ff + ".w_1.bias"] = w(ffn, d), 0.1 * torch.randn(ffn, generator=g)
            st[p + ff + ".w_2.weight"], st[p + ff + ".w_2.bias"] = w(d, ffn), 0.1 * torch.randn(d, generator=g)
        a = p + "self_attn."
        st[a + "pos_bias_u"] = 0.1 * torch.randn(heads, dk, generator=g)
        st[a + "pos_bias_v"] = 0.1 * torch.randn(heads, dk, generator=g)
        for n in ("linear_q", "linear_k", "linear_v", "linear_out"):
            st[a + n + ".weight"], st[a + n + ".bias"] = w(d, d), 0.1 * torch.randn(d, generator=g)
        st[a + "linear_pos.weight"] = w(d, d)
        c = p + "conv_module."
        ln(c + "norm", st)
        st[c + "pointwise_conv1.weight"], st[c + "pointwise_conv1.bias"] = w(2 * d, d, 1, fan_in=d), 0.1 * torch.randn(2 * d, generator=g)
        st[c + "depthwise_conv.weight"], st[c + "depthwise_conv.bias"] = w(d, 1, kernel, fan_in=kernel), 0.1 * torch.randn(d, generator=g)
        st[c + "pointwise_conv2.weight"], st[c + "pointwise_conv2.bias"] = w(d, d, 1, fan_in=d), 0.1 * torch.randn(d, generator=g)
    ln("encoder.after_norm", st)
    st["encoder.global_cmvn.mean"] = torch.zeros(mel)
    st["encoder.global_cmvn.istd"] = torch.ones(mel)
    st["ctc.ctc_lo.weight"], st["ctc.ctc_lo.bias"] = w(vocab, d), 0.1 * torch.randn(vocab, generator=g)
    return st


def build_reference_asr(state: Dict[str, torch.Tensor], device: str, d: int = 512, heads: int = 8, ffn: int = 2048,
                        blocks: int = 12, kernel: int = 15, vocab: int = 5538, model_dir: str = "/nonexistent-model-dir"):
    """``WenetConformerASR`` of the reference (full-context, non-causal depthwise conv) on ``device``."""
    if not make_ref.add_to_path():
        raise RuntimeError("oracle/_ref is absent: run `python oracle/make_ref.py <reference checkout>`")
    from veloxvoice.models.wenet.config import WeNetConfig
    from veloxvoice.models.wenet.torch_conformer import WenetConformerASR

    cfg = WeNetConfig(output_size=d, attention_heads=heads, linear_units=ffn, num_blocks=blocks, cnn_module_kernel=kernel,
                      causal_conv=False)
    return WenetConformerASR(model_dir, device=device, cfg=cfg, vocab=vocab, state=state)

"""The encoder's linear stack built from the REFERENCE's own classes, on the CPU.  TEST INFRASTRUCTURE.

``DenseLinear`` and ``WenetConformerFF`` are imported from the copy of the reference package in
``oracle/_ref`` (see ``oracle/make_ref.py``) and run in their fp32 lane, which is the
reference's CPU path: ``DenseLinear.forward`` ends in ``torch.nn.functional.linear``
(``veloxvoice/models/wenet/torch_conformer.py:270``).  The data flow between the linears is the
model's (``torch_conformer.py:705-713``) with attention and the depthwise convolution left out,
exactly like :class:`oracle.stack.OracleStack` and the GPU stack.

Only ``bench.py --impl reference`` / its ``cpu_baseline`` leg and the tests use this.
"""

from __future__ import annotations

from typing import Dict

import numpy as np

from . import make_ref


def available() -> bool:
    return make_ref.available()


class ReferenceCpuStack:
    def __init__(self, weights: Dict[str, np.ndarray], blocks: int, d_model: int = 512, eps: float = 1e-5):
        import torch

        if not make_ref.add_to_path():
            raise RuntimeError("oracle/_ref is absent: run `python oracle/make_ref.py <reference checkout>`")
        from veloxvoice.models.wenet.torch_conformer import DenseLinear, WenetConformerFF

        t = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in weights.items()}
        self.t = t
        self.blocks, self.d, self.eps = blocks, d_model, eps
        self.ff, self.lin = {}, {}
        for i in range(blocks):
            b = f"b{i}."
            for ff in ("ffm", "ff"):
                states = {"p.w_1.weight": t[b + ff + ".w1"], "p.w_1.bias": t[b + ff + ".b1"],
                          "p.w_2.weight": t[b + ff + ".w2"], "p.w_2.bias": t[b + ff + ".b2"]}
                m = WenetConformerFF(None, states, "p")
                m.w1.precision = m.w2.precision = "fp32"
                self.ff[b + ff] = m
            for name, bias in (("qkv", True), ("lo", True), ("pw1", True), ("pw2", True)):
                m = DenseLinear(t[b + name + ".w"], t[b + name + ".b"] if bias else None)
                m.precision = "fp32"
                self.lin[b + name] = m
        m = DenseLinear(t["ctc.w"], t["ctc.b"])
        m.precision = "fp32"
        self.lin["ctc"] = m

    def forward(self, x: np.ndarray) -> np.ndarray:
        import torch
        import torch.nn.functional as Fn

        t, d = self.t, self.d

        def ln(v, key):
            return Fn.layer_norm(v, (d,), t[key + ".g"], t[key + ".b"], self.eps)

        with torch.no_grad():
            x = torch.from_numpy(np.asarray(x, dtype=np.float32))
            for i in range(self.blocks):
                b = f"b{i}."
                x = x + 0.5 * self.ff[b + "ffm"](ln(x, b + "ln_ffm"))
                qkv = self.lin[b + "qkv"](ln(x, b + "ln_mha"))
                x = x + self.lin[b + "lo"](qkv[:, 2 * d:])
                x = x + self.lin[b + "pw2"](Fn.glu(self.lin[b + "pw1"](ln(x, b + "ln_conv")), dim=1))
                x = x + 0.5 * self.ff[b + "ff"](ln(x, b + "ln_ff"))
                x = ln(x, b + "ln_final")
            return self.lin["ctc"](ln(x, "after")).numpy()

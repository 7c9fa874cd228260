"""Generate golden vectors from the reference's own Python code (run once, CPU only).

Usage::

    python tests/golden/make_golden.py --reference /path/to/velox-voice [--out tests/golden]

What runs, unmodified, from the reference tree:

* ``veloxvoice/kernels/ops/triton_ops.py``: ``per_row_col_quantize``,
  ``mxfp4_block_quantize`` (modes "A" and "B") and ``mxfp4_dequant`` -- the Triton kernels
  execute through Triton's CPU interpreter (``TRITON_INTERPRET=1``);
* ``veloxvoice/kernels/ops/cuda_ops.py``: ``_dequantize_to_bf16``;
* ``veloxvoice/models/wenet/nvfp4_linear.py``: ``_encode_codes``, ``decode_codes``;
* ``tests/kernels/test_dgx_mxfp4_gemm.py``: ``unpack`` and ``torch_matmul_ref`` (the
  reference's definition of the FP4 GEMM result);
* ``veloxvoice/kernels/ops/cuda_ops.py``: ``reference_power_mel_log`` and
  ``tests/kernels/test_power_mel_log.py``: ``emulated_power_mel_log``, ``_tf32_rz`` (the fp32 formula
  of the filterbank projection and the reference's restatement of its tensor-core kernel).

The two reference modules create a lookup table with ``device="cuda"`` at import time; the
only accommodation made here is to map that one ``torch.tensor(..., device="cuda")`` call to
the CPU while the modules are imported (and to answer the compute-capability query a skip mark
of the mel test file makes at import).  No reference source is copied.

Outputs (small ``.npz`` files next to this script) hold the seeded inputs and the bytes the
reference produced for them.
"""

from __future__ import annotations

import argparse
import importlib
import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402


def _import_reference(ref_root: str):
    orig_tensor = torch.tensor

    def tensor_on_cpu(*a, **k):
        if str(k.get("device", "")).startswith("cuda"):
            k["device"] = "cpu"
        return orig_tensor(*a, **k)

    torch.tensor = tensor_on_cpu
    orig_cap = torch.cuda.get_device_capability
    torch.cuda.get_device_capability = lambda *a, **k: (0, 0)  # a skip mark of the mel test file asks for it at import
    sys.path.insert(0, ref_root)
    try:
        tri = importlib.import_module("veloxvoice.kernels.ops.triton_ops")
        cu = importlib.import_module("veloxvoice.kernels.ops.cuda_ops")
        nv = importlib.import_module("veloxvoice.models.wenet.nvfp4_linear")
        spec = importlib.util.spec_from_file_location(
            "_ref_test_gemm", os.path.join(ref_root, "tests/kernels/test_dgx_mxfp4_gemm.py")
        )
        tg = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(tg)
        spec = importlib.util.spec_from_file_location(
            "_ref_test_mel", os.path.join(ref_root, "tests/kernels/test_power_mel_log.py")
        )
        tm = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(tm)
    finally:
        torch.tensor = orig_tensor
        torch.cuda.get_device_capability = orig_cap
    return tri, cu, nv, tg, tm


def _edge_rows(K: int) -> torch.Tensor:
    """Rows that exercise ties, exact power-of-two scales, zeros and extreme magnitudes."""
    rows = []
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 0.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -0.0, 6.0, 4.0])
    for sh in (0, -3, 5):  # amax = 6 * 2**sh -> s is an exact power of two
        rows.append((ties * 2.0**sh).repeat(K // 16))
    rows.append(torch.zeros(K))  # all-zero row -> scale byte 108
    r = torch.zeros(K)
    r[3] = 1.5 * 2.0**-20  # tiny amax: below the 1e-6 floor
    r[5] = -1e-9
    rows.append(r)
    r = torch.linspace(-1.0, 1.0, K) * 3.0e38  # near the bf16/fp32 maximum
    rows.append(r)
    r = torch.full((K,), 1.5)  # amax/6 = 0.25 exactly
    r[1::2] = -0.37
    rows.append(r)
    r = torch.linspace(-6.0, 6.0, K)
    rows.append(r)
    return torch.stack(rows).float()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()
    tri, cu, nv, tg, tm = _import_reference(os.path.abspath(args.reference))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from oracle import mel as mel_oracle

    # ---------------- per-row quantizer (per_row_col_quantize) + _dequantize_to_bf16
    row = {}
    cases = []
    for seed, (M, K), dt in [(0, (64, 512), "bf16"), (1, (32, 128), "f32"), (2, (16, 96), "bf16"), (3, (128, 64), "bf16")]:
        torch.manual_seed(seed)
        x = torch.randn(M, K)
        if seed == 1:
            x = x * torch.logspace(-6, 6, M).unsqueeze(1)
        if dt == "bf16":
            x = x.bfloat16()
        cases.append((f"s{seed}", x))
    cases.append(("edge", _edge_rows(64).bfloat16()))
    cases.append(("edge_f32", _edge_rows(64)))
    torch.manual_seed(7)
    cases.append(("w002", (0.02 * torch.randn(48, 512))))
    for name, x in cases:
        q, s = tri.per_row_col_quantize(x)
        row[f"{name}_x"] = x.float().numpy()
        row[f"{name}_isbf16"] = np.array(x.dtype == torch.bfloat16)
        row[f"{name}_q"] = q.numpy()
        row[f"{name}_s"] = s.numpy()
        row[f"{name}_deq_bf16_as_f32"] = cu._dequantize_to_bf16(q, s).float().numpy()
    np.savez_compressed(os.path.join(args.out, "rowscale.npz"), **row)

    # ---------------- per-16 block quantizer (mxfp4_block_quantize) + mxfp4_dequant
    blk = {}
    cases = []
    for seed, (R, K) in [(0, (32, 128)), (1, (64, 64)), (2, (16, 48))]:
        torch.manual_seed(seed)
        x = torch.randn(R, K)
        if seed == 1:
            x = x * torch.logspace(-4, 4, K).unsqueeze(0)
        cases.append((f"s{seed}", x.bfloat16()))
    cases.append(("edge", _edge_rows(64).bfloat16()))
    torch.manual_seed(11)
    cases.append(("pos_f32", torch.rand(16, 64) * 1000.0))  # power-spectrum-like, fp32
    for name, x in cases:
        blk[f"{name}_x"] = x.float().numpy()
        for mode in ("A", "B"):
            q, s = tri.mxfp4_block_quantize(x, mode=mode)
            blk[f"{name}_{mode}_q"] = q.numpy()
            blk[f"{name}_{mode}_s"] = s.numpy()
            blk[f"{name}_{mode}_deq"] = tri.mxfp4_dequant(q, s, mode).numpy()
    np.savez_compressed(os.path.join(args.out, "blk16.npz"), **blk)

    # ---------------- E2M1 helpers + the reference's GEMM definition
    g = {}
    v = torch.cat([torch.linspace(-7, 7, 1121), torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, -0.0, 0.0])])
    g["enc_in"] = v.numpy()
    g["enc_out"] = nv._encode_codes(v).numpy()
    allb = torch.arange(256, dtype=torch.uint8).reshape(8, 32)
    g["dec_in"] = allb.numpy()
    g["dec_out"] = nv.decode_codes(allb).numpy()
    g["unpack_out"] = tg.unpack(allb).numpy()
    for seed, (M, N, K) in [(0, (128, 128, 64)), (1, (64, 96, 256)), (2, (32, 48, 2048))]:
        torch.manual_seed(seed)
        x = torch.randn(M, K).bfloat16()
        w = torch.randn(N, K).bfloat16()
        xq, xs = tri.per_row_col_quantize(x)
        wq, ws = tri.per_row_col_quantize(w)
        ref = tg.torch_matmul_ref(xq, wq, xs, ws)
        g[f"gemm{seed}_x"] = x.float().numpy()
        g[f"gemm{seed}_w"] = w.float().numpy()
        g[f"gemm{seed}_xq"] = xq.numpy()
        g[f"gemm{seed}_xs"] = xs.numpy()
        g[f"gemm{seed}_wq"] = wq.numpy()
        g[f"gemm{seed}_ws"] = ws.numpy()
        g[f"gemm{seed}_ref"] = ref.numpy()
    np.savez_compressed(os.path.join(args.out, "gemm_rowscale.npz"), **g)
    # ---------------- filterbank projection: the reference's fp32 formula and its test's tf32 emulation
    m = {}
    for name, seed, (T, F, M), bank, cmvn in [("rand", 42, (40, 257, 80), "randn", True), ("tri", 5, (24, 201, 80), "triangles", False),
                                              ("small", 3, (7, 64, 3), "randn", False)]:
        torch.manual_seed(seed)
        spec_t = torch.randn(T, F, dtype=torch.cfloat)
        mel_t = torch.randn(M, F) if bank == "randn" else torch.from_numpy(mel_oracle.mel_filterbank(F, M, seed))
        mean = torch.randn(M) if cmvn else None
        istd = (torch.rand(M) + 0.5) if cmvn else None
        m[f"{name}_spec"] = torch.view_as_real(spec_t).numpy()
        m[f"{name}_mel"] = mel_t.numpy()
        if cmvn:
            m[f"{name}_mean"], m[f"{name}_istd"] = mean.numpy(), istd.numpy()
        m[f"{name}_fp32"] = cu.reference_power_mel_log(spec_t.real, spec_t.imag, mel_t, mean, istd).numpy()
        m[f"{name}_tf32"] = tm.emulated_power_mel_log(spec_t, mel_t, mean, istd).numpy()
        m[f"{name}_rz_bits"] = tm._tf32_rz(mel_t).numpy()
    np.savez_compressed(os.path.join(args.out, "mel.npz"), **m)
    print("golden vectors written to", args.out)


if __name__ == "__main__":
    main()

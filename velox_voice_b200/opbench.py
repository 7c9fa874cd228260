"""Per-launch micro-benchmark of the quantized-linear path (the counterpart of the reference's
``benchmark/kernels/bench_*.py``: CUDA-event timings of single launches at the encoder's shapes).

    python -m velox_voice_b200.opbench                     # every launch of one Conformer block + CTC
    python -m velox_voice_b200.opbench --ops ffn-up        # only launches whose name contains "ffn-up"
    python -m velox_voice_b200.opbench --ops mel           # the front-end's filterbank projection (4 x frames rows)
    python -m velox_voice_b200.opbench --ops attention     # one 3,750-frame span of the rel-pos attention, and torch's SDPA
    python -m velox_voice_b200.opbench --configs           # the three single-GPU benchmark configurations
    python -m velox_voice_b200.opbench --frames 11250 --fmt nv16

Each launch is timed alone with the L2 flushed before it (a 512 MB buffer is overwritten), median
of five; bytes and FLOPs are the algorithmic ones (operands + scales read once, result written
once).  Prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os


def _timed(fn, flush, n=5, warm=2):
    import torch

    for _ in range(warm):
        fn()
    ts = []
    for _ in range(n):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def op_breakdown(stack, T, fmt_name, only=""):
    """Times every distinct launch of one block (+ CTC) alone, L2 flushed before each timed
    launch, and returns [(name, count_per_step, us, algorithmic_bytes, flops)]."""
    import torch

    from . import ops

    cfg = stack.cfg
    dev = stack.device
    d, f, V = cfg.d_model, cfg.ffn, cfg.vocab
    nb = cfg.blocks
    fmt = stack.fmt
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    x = torch.randn(T, d, device=dev).bfloat16()
    g, b = stack.ln["b0.ln_ffm"]
    sfb = 1 / 32 if fmt_name == "mx32" else (1 / 16 if fmt_name == "nv16" else 4 / 128)
    ebytes = 1.0 if fmt_name == "fp8_1x128" else 0.5

    def qbytes(rows, k):
        return rows * k * (ebytes + sfb)

    am = stack.amax.get("b0.ln_ffm")
    xq = ops.ln_quantize(x, g, b, cfg.eps, fmt, amax_t=am)
    res = torch.randn(T, d, device=dev).bfloat16()
    cases = []

    def add(name, count, fn, nbytes, flops):
        if only and only not in name:
            return
        cases.append((name, count, _timed(fn, flush), nbytes, flops))

    # the LayerNorms behind residual GEMMs run in those GEMMs (long inputs only, see StackConfig)
    fused = bool(getattr(stack, "fuse_ln", False)) and T >= getattr(stack, "fuse_ln_min_frames", cfg.fuse_ln_min_frames)
    add("ln_quantize [T,512]", 1 if fused else 3 * nb + 1, lambda: ops.ln_quantize(x, g, b, cfg.eps, fmt, amax_t=am),
        T * d * 2 + qbytes(T, d), 0)
    add("ln2_quantize [T,512] (norm_final + next LayerNorm + quantize)", 0 if fused else nb,
        lambda: ops.ln2_quantize(x, g, b, g, b, cfg.eps, fmt, y=x, amax_t=am), T * d * 4 + qbytes(T, d), 0)
    add("quantize [T,512]", 2 * nb + 1, lambda: ops.quantize(x, fmt, natural=fmt_name == "fp8_1x128", amax_t=am),
        T * d * 2 + qbytes(T, d), 0)
    w1, w2 = stack.p["b0.ffm.w1"], stack.p["b0.ffm.w2"]
    if stack.fuse_ffn:
        hq = w1(xq, act="swish", out_fmt=fmt, out_amax=stack.amax.get("b0.ffm.h"))
        add("gemm ffn-up 512->2048 swish, FP4 out", 2 * nb,
            lambda: w1(xq, act="swish", out_fmt=fmt, out_amax=stack.amax.get("b0.ffm.h")),
            qbytes(T, d) + qbytes(f, d) + qbytes(T, f), 2 * T * d * f)
    else:
        h = w1(xq, act="swish")
        hq = ops.quantize(h, fmt, natural=fmt_name == "fp8_1x128")
        add("gemm ffn-up 512->2048 swish, bf16 out", 2 * nb, lambda: w1(xq, act="swish"),
            qbytes(T, d) + qbytes(f, d) + T * f * 2, 2 * T * d * f)
        add("quantize [T,2048]", 2 * nb, lambda: ops.quantize(h, fmt, natural=fmt_name == "fp8_1x128"),
            T * f * 2 + qbytes(T, f), 0)
    add("gemm ffn-down 2048->512 +0.5 residual", 0 if fused else 2 * nb, lambda: w2(hq, residual=res, alpha=0.5, out=res),
        qbytes(T, f) + qbytes(d, f) + T * d * 4, 2 * T * d * f)
    add("gemm qkv 512->1536 bias", nb, lambda: stack.p["b0.qkv"](xq), qbytes(T, d) + qbytes(3 * d, d) + T * 3 * d * 2,
        2 * T * d * 3 * d)
    if fused:
        add("gemm ffn-down 2048->512 +0.5 residual + LayerNorm + quantize (2-CTA clusters)", nb,
            lambda: w2.residual_ln(hq, residual=res, gamma=g, beta=b, eps=cfg.eps, alpha=0.5, out=res),
            qbytes(T, f) + qbytes(d, f) + T * d * 4 + qbytes(T, d), 2 * T * d * f)
        add("gemm ffn-down 2048->512 +0.5 residual + 2 LayerNorms + quantize (2-CTA clusters)", nb,
            lambda: w2.residual_ln(hq, residual=res, gamma=g, beta=b, eps=cfg.eps, alpha=0.5, out=res, gamma2=g, beta2=b),
            qbytes(T, f) + qbytes(d, f) + T * d * 4 + qbytes(T, d), 2 * T * d * f)
        add("gemm lo/pw2 512->512 +residual + LayerNorm + quantize (2-CTA clusters)", 2 * nb,
            lambda: stack.p["b0.lo"].residual_ln(xq, residual=res, gamma=g, beta=b, eps=cfg.eps, alpha=1.0, out=res),
            qbytes(T, d) + qbytes(d, d) + T * d * 4 + qbytes(T, d), 2 * T * d * d)
    add("gemm lo/pw2 512->512 +residual", 0 if fused else 2 * nb, lambda: stack.p["b0.lo"](xq, residual=res, alpha=1.0, out=res),
        qbytes(T, d) + qbytes(d, d) + T * d * 4, 2 * T * d * d)
    add("gemm lp 512->512", nb, lambda: stack.p["b0.lp"](xq), qbytes(T, d) + qbytes(d, d) + T * d * 2, 2 * T * d * d)
    add("gemm pw1 512->1024 GLU", nb, lambda: stack.p["b0.pw1"](xq), qbytes(T, d) + qbytes(2 * d, d) + T * d * 2,
        2 * T * d * 2 * d)
    add("gemm ctc 512->5538 bias + argmax (no logits written)", 1, lambda: stack.p["ctc"].argmax(xq),
        qbytes(T, d) + qbytes(V, d) + T * 12, 2 * T * d * V)
    if only and "mel" in only:
        # the audio front-end's filterbank projection (not part of the encoder step): one hour of 10 ms frames
        Tm, Fm, Mm = 4 * T, 257, 80
        spec = torch.randn(Tm, Fm, dtype=torch.cfloat, device=dev)
        bank = torch.rand(Mm, Fm, device=dev)
        mean, istd = torch.randn(Mm, device=dev), torch.rand(Mm, device=dev) + 0.5
        add(f"power_mel_log [{Tm} x {Fm}] -> {Mm} mel (tf32)", 0, lambda: ops.power_mel_log_tf32(spec, bank, mean, istd),
            Tm * Fm * 8 + Tm * Mm * 4 + Mm * Fm * 4, 2 * Tm * Fm * Mm)
    if only and "attention" in only:
        # one span of one layer (not part of the linear-stack step): 3,750 frames, 8 heads of 64, on the fold pack
        Ta, h, dk = 3750, 8, 64
        q2 = (torch.randn(h, Ta, 2 * dk, device=dev) * 0.25).bfloat16()
        k2 = torch.randn(h, Ta, 2 * dk, device=dev).bfloat16()
        v2 = torch.randn(h, Ta, 2 * dk, device=dev).bfloat16()
        fl = 2 * h * Ta * Ta * (2 * dk + dk)
        nbytes = 3 * h * Ta * 2 * dk * 2 + Ta * h * dk * 2
        add(f"relpos attention [{h} x {Ta} x {2 * dk}] (tcgen05 bf16)", 0, lambda: ops.relpos_attention(q2, k2, v2), nbytes, fl)
        add("relpos attention, torch scaled_dot_product_attention on the same tensors", 0,
            lambda: torch.nn.functional.scaled_dot_product_attention(q2[None], k2[None], v2[None], scale=1.0), nbytes, fl)
    del flush
    return cases


def baseline_configs(dev, hbm_peak_gbs):
    """The three single-GPU benchmark configurations as single (chains of) launches: us,
    algorithmic TFLOP/s and GB/s, and the fraction of the roofline (slower of bytes at the measured
    HBM peak and FLOPs at the measured tensor-core peak of that operand type).  The first one is
    also timed as a CUDA-graph replay of 20 back-to-back calls (the reference's method for
    launch-bound shapes, ``benchmark/kernels/bench_fused_qkv.py:167-198``)."""
    import torch

    from . import ops

    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    peak = {"fp4": ops.mma_peak_tflops("fp4", 256, 2048), "fp8": ops.mma_peak_tflops("fp8", 256, 2048)}

    def entry(name, us, flops, nbytes, kind, **extra):
        t_roof = max(nbytes / (hbm_peak_gbs * 1e3), flops / (peak[kind] * 1e6))  # us
        e = {"config": name, "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1), "GBps": round(nbytes / us / 1e3, 1),
             "roofline_us": round(t_roof, 2), "roofline_frac": round(t_roof / us, 3)}
        e.update(extra)
        return e

    out = []
    torch.manual_seed(0)
    # single MXFP4 linear, x [1024, 512] -> [1024, 2048] bf16 (quantize on the fly + GEMM)
    x = torch.randn(1024, 512, device=dev).bfloat16()
    w = ops.quantize(0.02 * torch.randn(2048, 512, device=dev), "mx32")
    o1 = torch.empty(1024, 2048, device=dev, dtype=torch.bfloat16)

    def cfg1():
        ops.bsgemm(ops.quantize(x, "mx32", natural=False), w, out=o1)

    us = _timed(cfg1, flush, n=7)
    # graph replay: 20 calls per replay, caches warm (launch overhead out of the picture)
    cfg1()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        cfg1()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(20):
                cfg1()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us_graph = e0.elapsed_time(e1) * 1e3 / 200
    out.append(entry("cfg1 mxfp4 linear 1024x2048x512 (quantize + GEMM)", us, 2 * 1024 * 2048 * 512,
                     1024 * 512 * 2 + 2048 * 512 * (0.5 + 1 / 32) + 1024 * 2048 * 2, "fp4",
                     us_graph_replay=round(us_graph, 2)))
    # fused QKV, FP8 1x128, T = 90000 (activations already quantized; GEMM + bias -> bf16)
    T = 90000
    xa = torch.nn.functional.layer_norm(torch.randn(T, 512, device=dev), (512,)).bfloat16()
    bound = (6.0 / (512 + 1536)) ** 0.5
    wq = ops.quantize((torch.rand(1536, 512, device=dev) * 2 - 1) * bound, "fp8_1x128")
    aq = ops.quantize(xa, "fp8_1x128")
    bias = torch.zeros(1536, device=dev)
    o = torch.empty(T, 1536, device=dev, dtype=torch.bfloat16)
    us = _timed(lambda: ops.bsgemm(aq, wq, epilogue=ops.EPI_BIAS, bias=bias, out=o), flush, n=7)
    out.append(entry("cfg2 fused QKV fp8_1x128 90000x1536x512 (GEMM + bias)", us, 2 * T * 1536 * 512,
                     T * 512 * (1 + 4 / 128) + 1536 * 512 * (1 + 4 / 128) + T * 1536 * 2, "fp8"))
    us = _timed(lambda: ops.quantize(xa, "fp8_1x128"), flush, n=7)
    out.append(entry("cfg2 activation quantize fp8_1x128 [90000, 512]", us, 0, T * 512 * (2 + 1 + 4 / 128), "fp8"))
    # macaron FFN, NVFP4: y = x + 0.5 * W2 swish(W1 LN(x)); 3 launches, FP4 intermediate
    xf = torch.randn(T, 512, device=dev).bfloat16()
    w1 = ops.quantize(0.02 * torch.randn(2048, 512, device=dev), "nv16")
    w2 = ops.quantize(0.02 * torch.randn(512, 2048, device=dev), "nv16")
    b1, b2 = torch.zeros(2048, device=dev), torch.zeros(512, device=dev)
    g_, be = torch.ones(512, device=dev), torch.zeros(512, device=dev)
    am_x = torch.tensor([6.0], device=dev)
    am_h = torch.tensor([8.0], device=dev)
    y = torch.empty_like(xf)

    def ffn():
        q = ops.ln_quantize(xf, g_, be, 1e-5, "nv16", amax_t=am_x)
        h = ops.bsgemm(q, w1, epilogue=ops.EPI_BIAS_SWISH, bias=b1, out_fmt="nv16", out_amax=am_h)
        ops.bsgemm(h, w2, epilogue=ops.EPI_BIAS_RESIDUAL, bias=b2, residual=xf, alpha=0.5, out=y)

    us = _timed(ffn, flush, n=7)
    nb = T * 512 * 2 + T * 512 * (0.5 + 1 / 16) * 2 + T * 2048 * (0.5 + 1 / 16) * 2 + T * 512 * 4
    out.append(entry("cfg3 macaron FFN nv16 T=90000 (ln_quant + up/swish/FP4 + down/residual)", us, 2 * 2 * T * 512 * 2048, nb, "fp4"))
    del flush
    return out, peak


def measured_hbm_peak(root: str):
    """(GB/s, where it came from): the pool's measured copy bandwidth when its record is
    present beside the package, else the documented fallback."""
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback 6650 GB/s"


def main():
    import torch

    from .stack import ConformerLinearStack, StackConfig, make_weights

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--frames", type=int, default=90000)
    ap.add_argument("--fmt", default="mx32", choices=["mx32", "nv16", "fp8_1x128"])
    ap.add_argument("--ops", default="", help="substring filter on the launch name")
    ap.add_argument("--configs", action="store_true", help="time the three single-GPU benchmark configurations instead")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA GPU: this library has no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hbm, src = measured_hbm_peak(root)
    if a.configs:
        cfgs, peak = baseline_configs(dev, hbm)
        print(json.dumps({"baseline_configs": cfgs, "mma_peak_tflops_measured": peak, "hbm_peak": hbm, "hbm_peak_source": src}))
        return
    cfg = StackConfig(blocks=1, fmt=a.fmt)
    stack = ConformerLinearStack(cfg, make_weights(cfg, seed=0), device=dev)
    if a.fmt == "nv16":
        stack.calibrate(torch.randn(4096, cfg.d_model, device=dev).bfloat16(), torch.randn(4096, cfg.d_model, device=dev).bfloat16())
    cases = op_breakdown(stack, a.frames, a.fmt, a.ops)
    print(json.dumps({"frames": a.frames, "format": a.fmt,
                      "launches": [{"op": n, "us": round(us, 1), "GBps": round(nb / us / 1e3, 1), "TFLOPs": round(fl / us / 1e6, 1),
                                    "hbm_frac": round(nb / us / 1e3 / hbm, 3)} for n, _, us, nb, fl in cases]}))


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the quantized-linear path: encoder frames per second of the full linear stack.

A step = one pass of the MXFP4 encoder linear stack (12 Conformer blocks' linears + CTC head,
greedy argmax) over ONE HOUR of synthetic 16 kHz audio (89,999 encoder frames: seeded PCM ->
80-bin Kaldi fbank -> fixed seeded stand-in for the subsampling front, velox_voice_b200/synth.py),
random-init weights (seed 0).  With N GPUs the hour is cut into N equal frame shards (strong
scaling), weights replicated; the only collective is the gather of the per-frame CTC ids (a
second leg gathers the bf16 logits instead, a third gives the weak-scaling number).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference        # the path's CPU restatement on the host cores

Prints ONE JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "encoder_frames_per_s"
UNIT = "frames/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--frames", type=int, default=0,
                    help="encoder frames of the whole job (default: the synthetic hour, 89,999)")
    ap.add_argument("--fmt", default="mx32", choices=["mx32", "nv16", "fp8_1x128"])
    ap.add_argument("--blocks", type=int, default=12)
    ap.add_argument("--cpu-frames", type=int, default=65536, help="frames per step of the CPU arms' sample")
    ap.add_argument("--no-breakdown", action="store_true", help="skip the per-launch timings (no roofline object)")
    ap.add_argument("--no-extras", action="store_true", help="skip the logits-gather and weak-scaling legs")
    ap.add_argument("--traffic-bytes", type=float, default=None,
                    help="dram bytes (read + write) of one launch of the dominant kernel from an ncu capture of THIS build")
    return ap.parse_args()


def total_frames(a) -> int:
    from velox_voice_b200 import synth

    return a.frames if a.frames > 0 else synth.total_encoder_frames()


def workload_name(a) -> str:
    return (f"cfg5: one hour of synthetic 16 kHz audio (seed 1) -> 80-bin Kaldi fbank -> fixed seeded 4x80->512 "
            f"stand-in for the subsampling front -> cfg4 encoder linear stack, {a.fmt}, {a.blocks} blocks + CTC 512->5538 "
            f"greedy ids; T={total_frames(a)} encoder frames in total, cut into equal frame shards over the GPUs; "
            f"attention / depthwise conv left out")


# ----------------------------------------------------------------------------- clocks


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            p = [c.strip() for c in r.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- CPU arms

_CPU_STACKS = {}


def cpu_reference_sample(a, frames: int):
    """The reference's CPU path of the stack on `frames` frames with every host thread torch can
    use: its own DenseLinear / WenetConformerFF classes in their fp32 lane (F.linear) when the
    copy of the reference package is present in oracle/_ref, else this repository's fp32
    restatement of the same lane.  Returns (frames/s, threads, seconds, kind)."""
    import numpy as np
    import torch

    from oracle import ref_stack
    from oracle.stack import cpu_linear_stack_fp32
    from velox_voice_b200.stack import StackConfig, make_weights

    torch.set_num_threads(os.cpu_count() or 1)
    cfg = StackConfig(blocks=a.blocks, fmt=a.fmt)
    key = ("fp32", a.blocks)
    st = _CPU_STACKS.get(key)
    if st is None:
        w = {k: v.numpy() for k, v in make_weights(cfg, seed=0).items()}
        if ref_stack.available():
            rs = ref_stack.ReferenceCpuStack(w, cfg.blocks)
            st = (rs.forward, "reference")
        else:
            st = ((lambda x: cpu_linear_stack_fp32(w, x, cfg.blocks)), "port")
        _CPU_STACKS[key] = st
    fn, kind = st
    g = torch.Generator().manual_seed(1)
    x = torch.randn(frames, cfg.d_model, generator=g).bfloat16().float().numpy()
    t0 = time.perf_counter()
    fn(x)
    dt = time.perf_counter() - t0
    return frames / dt, torch.get_num_threads(), dt, kind


def cpu_quantized_port_sample(a, frames: int):
    """The quantized path's CPU restatement (oracle: quantize -> dequantize -> fp32 matmul per
    linear) on `frames` frames.  Returns (frames/s, threads, seconds)."""
    import numpy as np
    import torch

    from oracle import formats as F
    from oracle.stack import OracleStack
    from velox_voice_b200.stack import StackConfig, make_weights

    torch.set_num_threads(os.cpu_count() or 1)
    cfg = StackConfig(blocks=a.blocks, fmt=a.fmt)
    key = ("q", a.blocks, a.fmt)
    st = _CPU_STACKS.get(key)
    if st is None:
        w = {k: v.numpy() for k, v in make_weights(cfg, seed=0).items()}
        st = OracleStack(w, F.FMT_NAMES[a.fmt], cfg.blocks, amax={} if a.fmt == "nv16" else None)
        st.forward(np.zeros((8, cfg.d_model), np.float32))  # quantize the weights once, untimed
        _CPU_STACKS[key] = st
    g = torch.Generator().manual_seed(1)
    x = torch.randn(frames, cfg.d_model, generator=g).bfloat16().float().numpy()
    t0 = time.perf_counter()
    st.forward(x)
    dt = time.perf_counter() - t0
    return frames / dt, torch.get_num_threads(), dt


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = []
    for _ in range(max(a.warmup, 1)):
        _, threads, _, kind = cpu_reference_sample(a, min(a.cpu_frames, 512))
    t0 = time.perf_counter()
    for _ in range(a.steps):
        _, threads, dt, kind = cpu_reference_sample(a, a.cpu_frames)
        per_step.append(dt)
    wall = time.perf_counter() - t0
    dt = sum(per_step) / len(per_step)
    value = a.cpu_frames / dt
    what = ("the reference's own DenseLinear / WenetConformerFF classes, fp32 lane (F.linear)" if kind == "reference"
            else "fp32 F.linear restatement of the reference's CPU lane")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "sample": f"{a.cpu_frames} frames per step on the host cores"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"{a.cpu_frames} frames of the same stack per step through {what}, "
                                   f"{a.steps} steps, wall {wall:.1f} s"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm


def run_ours(a):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.gpus > 1 and world == 1:
        # convenience: relaunch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29591", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from velox_voice_b200 import _lib, opbench, synth
    from velox_voice_b200.stack import ConformerLinearStack, StackConfig, make_weights, shard_capacity, shard_rows

    T = total_frames(a)                       # the whole job
    s0, s1 = shard_rows(T, world, rank)       # this rank's frames
    cap = shard_capacity(T, world)            # rows of every rank's slot in the gathers
    Tl = s1 - s0
    cfg = StackConfig(blocks=a.blocks, fmt=a.fmt)
    stack = ConformerLinearStack(cfg, make_weights(cfg, seed=0), device=dev)
    feats, _ = synth.encoder_features(s0, s1, device=dev)
    feats_host = torch.zeros((cap, cfg.d_model), dtype=torch.bfloat16).pin_memory()
    feats_host[:Tl].copy_(feats)
    del feats
    g = torch.Generator().manual_seed(1000 + rank)
    pos = torch.randn(cap, cfg.d_model, generator=g).bfloat16().to(dev)
    if a.fmt == "nv16":
        stack.calibrate(feats_host[:4096].to(dev), pos[:4096])
    comp = stack.compile(cap)
    comp.pos.copy_(pos)
    comp.x_in.copy_(feats_host)
    ids_all = torch.empty((world * cap,), dtype=torch.int32, device=dev)

    def gather_ids():
        if world > 1:
            dist.all_gather_into_tensor(ids_all, comp.ids)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(step_fn, steps, warmup):
        """K steps bracketed by barrier + synchronize, CUDA events, max over ranks -> ms."""
        for _ in range(warmup):
            step_fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        torch.cuda.synchronize(dev)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- device-resident timing: this rank's shard already in HBM; ids gathered every step
    def step_ids():
        comp.run()
        gather_ids()

    for _ in range(max(a.warmup, 3)):
        step_ids()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = timed(step_ids, a.steps, 0)
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.device_status()
    ms_per_step = ms / a.steps
    value = T * a.steps / (ms * 1e-3)

    # ---- end to end through the public call: pinned host features in, host ids out
    for _ in range(2):
        comp.encode_ctc_host(feats_host)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(a.steps):
        comp.encode_ctc_host(feats_host)
        gather_ids()
    e1.record()
    torch.cuda.synchronize(dev)
    seq_ms = max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3))
    # the same K steps as a queue of shards: copy of shard i+1 overlaps the stack of shard i
    queue = [feats_host] * a.steps
    comp.reserve_host_ids(len(queue))  # pinned result buffers: allocated outside the timed region
    comp.encode_ctc_host_batches(queue[:2])
    barrier()
    t0 = time.perf_counter()
    e0.record()
    comp.encode_ctc_host_batches(queue, after_each=lambda i: gather_ids())
    e1.record()
    torch.cuda.synchronize(dev)
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3))
    e2e_value = T * a.steps / (e2e_ms * 1e-3)
    e2e_seq_value = T * a.steps / (seq_ms * 1e-3)

    # ---- the same job with the bf16 CTC logits gathered instead of the ids, and (N > 1) the
    #      weak-scaling number: every GPU takes a whole hour of its own
    extras = {}
    if not a.no_extras:
        ldv = (cfg.vocab + 7) // 8 * 8
        logits = [torch.empty((cap, ldv), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        full = [torch.empty((world * cap, ldv), dtype=torch.bfloat16, device=dev) for _ in range(2)] if world > 1 else None
        comm = torch.cuda.Stream(device=dev)
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]
        for e in ev_free:
            e.record()
        state = {"i": 0}
        xw = torch.empty_like(comp.x_in)

        def logits_pass(buf):
            xw.copy_(comp.x_in)
            stack.forward(xw, comp.pos, out_logits=buf[:, : cfg.vocab])

        def step_logits_serial():
            logits_pass(logits[0])
            if world > 1:
                dist.all_gather_into_tensor(full[0], logits[0])

        def step_logits_overlapped():
            # the gather of step i runs on a side stream under the stack of step i + 1
            k = state["i"] & 1
            state["i"] += 1
            main = torch.cuda.current_stream()
            main.wait_event(ev_free[k])
            logits_pass(logits[k])
            ev_done[k].record(main)
            if world > 1:
                with torch.cuda.stream(comm):
                    comm.wait_event(ev_done[k])
                    dist.all_gather_into_tensor(full[k], logits[k])
                    ev_free[k].record(comm)

        def drain():
            torch.cuda.current_stream().wait_stream(comm)

        k_extra = max(2, min(a.steps, 5))
        ms_ser = timed(step_logits_serial, k_extra, 2)
        extras["logits_gather_serial"] = {"value": T * k_extra / (ms_ser * 1e-3), "ms_per_step": ms_ser / k_extra}

        def steps_overlapped():
            step_logits_overlapped()

        for _ in range(2):
            steps_overlapped()
        drain()
        barrier()
        e0.record()
        for _ in range(k_extra):
            steps_overlapped()
        drain()
        e1.record()
        torch.cuda.synchronize(dev)
        barrier()
        ms_ovl = max_over_ranks(e0.elapsed_time(e1))
        extras["logits_gather_overlapped"] = {"value": T * k_extra / (ms_ovl * 1e-3), "ms_per_step": ms_ovl / k_extra}
        extras["logits_bytes_gathered_per_step"] = world * cap * ldv * 2
        extras["note"] = ("eager launches (no CUDA graph); bf16 logits [T, 5538] written and, for N > 1, all-gathered "
                          "(NCCL all_gather_into_tensor of equal row slots); overlapped = gather of step i under the stack of step i+1")
        del logits, full
        if world > 1:
            comp_w = stack.compile(T)
            gw = torch.Generator().manual_seed(7 + rank)
            comp_w.x_in.copy_(torch.randn(T, cfg.d_model, generator=gw).bfloat16())
            comp_w.pos.copy_(torch.randn(T, cfg.d_model, generator=gw).bfloat16())
            ids_w = torch.empty((world * T,), dtype=torch.int32, device=dev)

            def step_weak():
                comp_w.run()
                dist.all_gather_into_tensor(ids_w, comp_w.ids)

            ms_w = timed(step_weak, k_extra, 2)
            extras["weak_scaling"] = {"value": world * T * k_extra / (ms_w * 1e-3), "ms_per_step": ms_w / k_extra,
                                      "frames_per_gpu": T, "note": "every GPU takes T frames of its own (randn features), ids gathered"}
            del comp_w, ids_w

    line = None
    if rank == 0:
        flops_per_frame = cfg.flops_per_frame()
        hbm_peak, peak_src = opbench.measured_hbm_peak(ROOT)
        roofline, breakdown, cfgs, mma_peak = None, None, None, None
        if not a.no_breakdown:
            cases = opbench.op_breakdown(stack, cap, a.fmt)
            total_us = sum(c * us for _, c, us, _, _ in cases)
            breakdown = [{"op": n, "launches_per_step": c, "us": round(us, 1), "share": round(c * us / total_us, 3),
                          "GBps": round(nb / us / 1e3, 1), "TFLOPs": round(fl / us / 1e6, 1)} for n, c, us, nb, fl in cases]
            top = max(cases, key=lambda t: t[1] * t[2])
            kind = "fp8" if a.fmt == "fp8_1x128" else "fp4"
            from velox_voice_b200 import ops

            mma_peak = {"fp4": ops.mma_peak_tflops("fp4", 256, 2048), "fp8": ops.mma_peak_tflops("fp8", 256, 2048)}
            # the dominant launch against both roofs; the one that gives the longer time binds
            gbs, tfs = top[3] / top[2] / 1e3, top[4] / top[2] / 1e6
            t_hbm, t_tc = top[3] / (hbm_peak * 1e3), top[4] / (mma_peak[kind] * 1e6)
            tensor_bound = t_tc > t_hbm
            roofline = {
                "kernel": top[0], "bound": "tensor" if tensor_bound else "hbm",
                "achieved": round(tfs if tensor_bound else gbs, 1),
                "peak": round(mma_peak[kind], 1) if tensor_bound else hbm_peak,
                "unit": "TFLOP/s" if tensor_bound else "GB/s",
                "frac": round((tfs / mma_peak[kind]) if tensor_bound else (gbs / hbm_peak), 4),
                "traffic": a.traffic_bytes,
                "peak_source": ("vx_mma_peak_probe in this run (measured, dense, back-to-back MMAs)" if tensor_bound else peak_src),
                "us_per_launch": round(top[2], 1), "roofline_us": round(max(t_hbm, t_tc), 1),
                "algorithmic_bytes_per_launch": int(top[3]), "algorithmic_flops_per_launch": int(top[4]),
                "hbm": {"achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(gbs / hbm_peak, 4), "peak_source": peak_src},
                "tensor": {"achieved": round(tfs, 1), "peak": round(mma_peak[kind], 1), "unit": "TFLOP/s",
                           "frac": round(tfs / mma_peak[kind], 4)},
                "rows_per_launch": cap,
            }
            if world == 1:
                cfgs, _ = opbench.baseline_configs(dev, hbm_peak)
        cpu_base = None
        if world == 1:
            cpu_fps, cores, cpu_dt, kind_cpu = cpu_reference_sample(a, a.cpu_frames)
            q_fps, _, q_dt = cpu_quantized_port_sample(a, min(a.cpu_frames, 1024))
            cpu_base = {"value": cpu_fps, "unit": UNIT, "cores": cores, "kind": kind_cpu,
                        "sample": f"{a.cpu_frames} frames of the same stack on the host cores ({cpu_dt:.1f} s), fp32 F.linear lane "
                                  + ("through the reference's own DenseLinear / WenetConformerFF classes" if kind_cpu == "reference"
                                     else "(restatement: the reference package copy is absent)"),
                        "quantized_port": {"value": q_fps, "unit": UNIT, "kind": "port",
                                           "sample": f"{min(a.cpu_frames, 1024)} frames through the CPU oracle "
                                                     f"(quantize -> dequantize -> fp32 matmul), {q_dt:.1f} s"}}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"mx32": "fp4 (e2m1, ue8m0 per 32) x fp4 -> f32", "nv16": "fp4 (e2m1, e4m3 per 16) -> f32",
                      "fp8_1x128": "fp8 (e4m3, f32 per 1x128) -> f32"}[a.fmt],
            "data": "synthetic",
            "config": {"workload": workload_name(a), "total_frames": T, "frames_per_gpu": cap, "format": a.fmt, "blocks": a.blocks,
                       "l2": ("working set per launch > L2 (126 MB) at one GPU; per-launch timings flush L2 (512 MB write) "
                              "before every timed launch"),
                       "parallelism": f"{world} equal frame shards of one {T}-frame job, weights replicated, ids all-gather"},
            "tflops": value * flops_per_frame / 1e12,
            "flops_per_frame": flops_per_frame,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": cap * cfg.d_model * 2, "d2h_bytes_per_step": cap * 4,
                    "ms_per_step": e2e_ms / a.steps, "call": "CompiledStack.encode_ctc_host_batches (K jobs queued, "
                    "copy of job i+1 overlaps the stack of job i); bytes are per GPU",
                    "sequential_value": e2e_seq_value, "sequential_call": "CompiledStack.encode_ctc_host per step"},
            "gpu_launches": comp.launches * a.steps,
            "gpu_launches_per_step": comp.launches,
            "device_status": status,
            "clocks": clocks,
            "roofline": roofline,
            "breakdown": breakdown,
            "baseline_configs": cfgs,
            "mma_peak_tflops_measured": mma_peak,
            "cpu_baseline": cpu_base,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()

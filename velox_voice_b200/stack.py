"""The encoder's linear stack on the quantized path, and its frame-sharded multi-GPU driver.

What runs per Conformer block (``veloxvoice/models/wenet/torch_conformer.py:705-713``):

    x += 0.5 * w2(swish(w1(LN(x))))            macaron FFN      (:657-658, :706)
    qkv = [lq|lk|lv](LN(x)); x += lo(ctx)      attention linears (:439-459, :519); lp(pos) (:472)
    x += pw2(f(glu(pw1(LN(x)))))               conv-module pointwise convs (:594-642)
    x += 0.5 * w2(swish(w1(LN(x))))            FFN              (:712)
    x  = LN(x)                                 norm_final       (:713)

followed by ``after_norm`` (:745) and the CTC head (:810-814).  Attention itself, the depthwise
convolution and its norm/activation are NOT linear layers and are outside this library: the
stack passes the value projection straight to ``lo`` and the GLU output straight to ``pw2``,
so it measures and validates every linear of the encoder with the real operand shapes.

Kernel sequence per block (13 launches; the reference issues >= 4 per linear):
``GEMM(bias, swish, FP4 out) -> GEMM(bias, 0.5 residual)`` for each FFN (the second one behind
its ``ln_quant``), ``ln_quant -> GEMM(bias) [qkv] -> quant -> GEMM(bias, residual) [lo]``,
``GEMM [lp]``, ``ln_quant -> GEMM(bias, GLU) -> quant -> GEMM(bias, residual)``, and one
``ln2_quant`` kernel that applies norm_final, stores the residual stream and hands the next
block's first FFN (or the CTC head, through after_norm) its quantized input.  The greedy head
(:meth:`ConformerLinearStack.forward_ids`) takes the per-frame argmax inside the CTC GEMM's
epilogue, so the [T, vocab] logits are never written.

Multi-GPU: every operation is row-wise in the frames, so frames are cut into contiguous equal
shards (:func:`shard_rows`), weights are replicated, and the only collective is the final
gather of the logits (:func:`gather_rows`, NCCL through ``torch.distributed``).  The reference
moves work between GPUs as files and subprocesses (``tools/bench_wenet_multi_worker.py:257-377``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import ops
from .linear import PackedLinear, glu_tile
from .ops import FMT_FP8_1X128, FMT_MX32, FMT_NV16


@dataclass
class StackConfig:
    d_model: int = 512
    heads: int = 8
    ffn: int = 2048
    blocks: int = 12
    conv_pw: int = 1024
    vocab: int = 5538
    fmt: str = "mx32"
    eps: float = 1e-5
    fuse_ffn: bool = True  # keep the FFN intermediate in FP4 (re-quantized in the up-GEMM epilogue)
    fuse_ln: bool = True   # MX32, d_model 512: the residual GEMMs also run the LayerNorm + quantizer behind them
    # ... from this many frames on: the fused kernel walks 128-row blocks with 74 two-CTA clusters at ~5 us a
    # block, which pays once every cluster has a few blocks (per step: 8.64 vs 9.13 ms at 90,000 frames, 2.82
    # vs 2.89 ms at 22,500) and no longer does on a short shard (11,250 frames, 88 blocks: 1.81 vs 1.80 ms)
    fuse_ln_min_frames: int = 16384

    def flops_per_frame(self) -> int:
        """Algorithmic FLOPs of the linears per encoder frame (2 * N * K each)."""
        d, f = self.d_model, self.ffn
        per_block = 4 * (2 * d * f) + 2 * d * 3 * d + 2 * d * d + 2 * d * d + 2 * d * self.conv_pw + 2 * d * d
        return self.blocks * per_block + 2 * d * self.vocab


def make_weights(cfg: StackConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init fp32 weights of the stack on the CPU (N(0, 0.02), zero biases, LN = identity
    affine), generated in a fixed order so every rank and the CPU oracle see the same values."""
    g = torch.Generator().manual_seed(seed)
    d, f = cfg.d_model, cfg.ffn

    def w(n, k):
        return torch.randn(n, k, generator=g) * 0.02

    out: Dict[str, torch.Tensor] = {}
    for i in range(cfg.blocks):
        p = f"b{i}."
        for ff in ("ffm", "ff"):
            out[p + ff + ".w1"], out[p + ff + ".b1"] = w(f, d), torch.zeros(f)
            out[p + ff + ".w2"], out[p + ff + ".b2"] = w(d, f), torch.zeros(d)
        out[p + "qkv.w"], out[p + "qkv.b"] = w(3 * d, d), torch.zeros(3 * d)
        out[p + "lo.w"], out[p + "lo.b"] = w(d, d), torch.zeros(d)
        out[p + "lp.w"] = w(d, d)
        out[p + "pw1.w"], out[p + "pw1.b"] = w(cfg.conv_pw, d), torch.zeros(cfg.conv_pw)
        out[p + "pw2.w"], out[p + "pw2.b"] = w(d, cfg.conv_pw // 2), torch.zeros(d)
        for n in ("ln_ffm", "ln_mha", "ln_conv", "ln_ff", "ln_final"):
            out[p + n + ".g"], out[p + n + ".b"] = torch.ones(d), torch.zeros(d)
    out["after.g"], out["after.b"] = torch.ones(d), torch.zeros(d)
    out["ctc.w"], out["ctc.b"] = w(cfg.vocab, d), torch.zeros(cfg.vocab)
    return out


class ConformerLinearStack:
    """All linears of the encoder on packed weights, fused quantize / GEMM / epilogue chain."""

    def __init__(self, cfg: StackConfig, weights: Dict[str, torch.Tensor], device="cuda",
                 amax: Optional[Dict[str, float]] = None):
        self.cfg = cfg
        self.fmt = ops._fmt(cfg.fmt)
        if self.fmt not in (FMT_MX32, FMT_NV16, FMT_FP8_1X128):
            raise ValueError("the stack runs in mx32, nv16 or fp8_1x128")
        self.device = torch.device(device)
        self.fuse_ffn = cfg.fuse_ffn and self.fmt != FMT_FP8_1X128
        # (environment: VELOX_B200_FUSE_LN=0 switches the fused residual + LayerNorm launches off and
        # VELOX_B200_FUSE_LN_MIN_FRAMES overrides their frame threshold, for A/B timing)
        self.fuse_ln = (bool(cfg.fuse_ln) and os.environ.get("VELOX_B200_FUSE_LN", "1") != "0"
                        and ops.residual_ln_supported(self.fmt, cfg.d_model, cfg.d_model))
        self.fuse_ln_min_frames = int(os.environ.get("VELOX_B200_FUSE_LN_MIN_FRAMES", cfg.fuse_ln_min_frames))
        dev = self.device
        self.p: Dict[str, PackedLinear] = {}
        self.ln: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}

        def pack(name, wkey, bkey=None, glu=False):
            wt = weights[wkey].to(dev)
            bt = weights[bkey].to(dev) if bkey else None
            self.p[name] = PackedLinear(wt, bt, self.fmt, glu=glu)

        for i in range(cfg.blocks):
            b = f"b{i}."
            for ff in ("ffm", "ff"):
                pack(b + ff + ".w1", b + ff + ".w1", b + ff + ".b1")
                pack(b + ff + ".w2", b + ff + ".w2", b + ff + ".b2")
            pack(b + "qkv", b + "qkv.w", b + "qkv.b")
            pack(b + "lo", b + "lo.w", b + "lo.b")
            pack(b + "lp", b + "lp.w")
            pack(b + "pw1", b + "pw1.w", b + "pw1.b", glu=True)
            pack(b + "pw2", b + "pw2.w", b + "pw2.b")
            for n in ("ln_ffm", "ln_mha", "ln_conv", "ln_ff", "ln_final"):
                self.ln[b + n] = (weights[b + n + ".g"].to(dev).float(), weights[b + n + ".b"].to(dev).float())
        self.ln["after"] = (weights["after.g"].to(dev).float(), weights["after.b"].to(dev).float())
        pack("ctc", "ctc.w", "ctc.b")
        # NV16 needs a per-tensor amax for every activation it quantizes: calibrated once
        self.amax: Dict[str, torch.Tensor] = {}
        if amax:
            for k, v in amax.items():
                self.amax[k] = torch.tensor([v], dtype=torch.float32, device=dev)

    # ---- helpers
    def _amax(self, key: str, x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if self.fmt != FMT_NV16:
            return None
        t = self.amax.get(key)
        if t is None:
            raise RuntimeError(f"nv16 stack: no calibrated amax for {key!r} (run calibrate())")
        return t

    def _lnq(self, key: str, x: torch.Tensor):
        g, b = self.ln[key]
        return ops.ln_quantize(x, g, b, self.cfg.eps, self.fmt, amax_t=self._amax(key, None))

    def _q(self, key: str, x: torch.Tensor):
        return ops.quantize(x, self.fmt, natural=self.fmt == FMT_FP8_1X128, amax_t=self._amax(key, x))

    def _residual(self, name: str, a, x: torch.Tensor, alpha: float, next_ln: Optional[str],
                  then_ln: Optional[str] = None):
        """``x <- alpha * linear(a) + x`` and, when ``next_ln`` names the LayerNorm that reads x next, its
        quantized output: one launch where the fused kernel covers the layer, else two.  With ``then_ln`` (the
        end of a block): ``x <- LN_next_ln(x)`` is what is stored and the quantized output is that of
        ``LN_then_ln`` of it."""
        lin = self.p[name]
        if next_ln is None:
            return lin(a, residual=x, alpha=alpha, out=x), None
        g, be = self.ln[next_ln]
        g2, be2 = self.ln[then_ln] if then_ln is not None else (None, None)
        if self.fuse_ln and x.shape[0] >= self.fuse_ln_min_frames and lin.residual_ln_supported():
            return lin.residual_ln(a, residual=x, gamma=g, beta=be, eps=self.cfg.eps, alpha=alpha, out=x,
                                   gamma2=g2, beta2=be2)
        x = lin(a, residual=x, alpha=alpha, out=x)
        if then_ln is None:
            return x, self._lnq(next_ln, x)
        # norm_final of this block + the LayerNorm that reads it next, one kernel
        return x, ops.ln2_quantize(x, g, be, g2, be2, self.cfg.eps, self.fmt, y=x, amax_t=self._amax(then_ln, None))

    def _ffn(self, b: str, ff: str, ln: str, x: torch.Tensor, q=None, next_ln: Optional[str] = None,
             then_ln: Optional[str] = None):
        if q is None:
            q = self._lnq(b + ln, x)
        if self.fuse_ffn:
            h = self.p[b + ff + ".w1"](q, act="swish", out_fmt=self.fmt, out_amax=self._amax(b + ff + ".h", None))
        else:
            h = self._q(b + ff + ".h", self.p[b + ff + ".w1"](q, act="swish"))
        return self._residual(b + ff + ".w2", h, x, 0.5, next_ln, then_ln)

    # ---- forward
    def forward(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None, *, return_hidden: bool = False,
                ids_only: bool = False, keys=None, ids=None, out_logits: Optional[torch.Tensor] = None):
        """x: bf16 [T, d_model] residual stream (overwritten in place); returns bf16 logits [T, vocab]
        (written into ``out_logits`` when given: bf16 [T, vocab], unit column stride)."""
        cfg = self.cfg
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != cfg.d_model:
            raise ValueError("x must be bf16 [T, d_model]")
        d = cfg.d_model
        pos_q = self._q("pos", pos) if pos is not None else None
        q_in = None  # first LayerNorm of the block, already applied by the previous block's last kernel
        for i in range(cfg.blocks):
            b = f"b{i}."
            x, q = self._ffn(b, "ffm", "ln_ffm", x, q_in, next_ln=b + "ln_mha")
            qkv = self.p[b + "qkv"](q)
            if pos_q is not None:
                self.p[b + "lp"](pos_q)  # feeds the attention scores only
            ctx = self._q(b + "ctx", qkv[:, 2 * d:])
            x, q = self._residual(b + "lo", ctx, x, 1.0, b + "ln_conv")
            gl = self.p[b + "pw1"](q)
            x, q = self._residual(b + "pw2", self._q(b + "glu", gl), x, 1.0, b + "ln_ff")
            # norm_final of this block + the LayerNorm that reads it next (first of the next block, or
            # after_norm) behind the second FFN: x <- LN_final(x), q_in <- quantize(LN_next(x))
            nxt = f"b{i + 1}.ln_ffm" if i + 1 < cfg.blocks else "after"
            x, q_in = self._ffn(b, "ff", "ln_ff", x, q, next_ln=b + "ln_final", then_ln=nxt)
        if q_in is None:  # zero blocks
            q_in = self._lnq("after", x)
        if ids_only:
            return self.p["ctc"].argmax(q_in, keys=keys, ids=ids)
        logits = self.p["ctc"](q_in, out=out_logits)
        return (logits, x) if return_hidden else logits

    def forward_ids(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None, *, keys=None, ids=None):
        """Greedy CTC ids int32 [T] of ``forward(x, pos).argmax(1)`` without writing the logits."""
        return self.forward(x, pos, ids_only=True, keys=keys, ids=ids)

    __call__ = forward

    # ---- captured execution (launch-bound at small T; the reference keeps a CUDA-graph cache
    # for the same reason, torch_conformer.py:1055-1066)
    def compile(self, frames: int, with_pos: bool = True):
        """Capture one forward + per-frame argmax for ``frames`` rows into a CUDA graph with
        static buffers.  Returns the :class:`CompiledStack`."""
        return CompiledStack(self, frames, with_pos)

    def calibrate(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None) -> Dict[str, float]:
        """One bf16 pass with plain torch ops recording max |.| of every tensor the NV16 path
        quantizes; fills ``self.amax`` (host sync; run once, outside any timed region)."""
        cfg = self.cfg
        rec: Dict[str, float] = {}

        def ln(key, t):
            g, b = self.ln[key]
            y = torch.nn.functional.layer_norm(t.float(), (cfg.d_model,), g, b, cfg.eps)
            rec[key] = float(y.abs().max())
            return y

        def lin(name, t):
            q = self.p[name].q
            w = ops._decode_e2m1(q.codes)  # dequantized weight rows (GLU rows stay interleaved)
            from_e4m3 = q.scales.view(torch.float8_e4m3fn).float()
            w = w * from_e4m3.repeat_interleave(16, dim=1) * (q.amax / 2688.0)
            y = t.float() @ w.T
            if self.p[name].bias is not None:
                y = y + self.p[name].bias
            return y

        if self.fmt != FMT_NV16:
            return rec
        x = x.float().clone()
        d = cfg.d_model
        if pos is not None:
            rec["pos"] = float(pos.abs().max())
        for i in range(cfg.blocks):
            b = f"b{i}."
            for ff, lnk in (("ffm", "ln_ffm"),):
                h = torch.nn.functional.silu(lin(b + ff + ".w1", ln(b + lnk, x)))
                rec[b + ff + ".h"] = float(h.abs().max())
                x = x + 0.5 * lin(b + ff + ".w2", h)
            qkv = lin(b + "qkv", ln(b + "ln_mha", x))
            ctx = qkv[:, 2 * d:]
            rec[b + "ctx"] = float(ctx.abs().max())
            x = x + lin(b + "lo", ctx)
            z = lin(b + "pw1", ln(b + "ln_conv", x))
            half = glu_tile(self.fmt) // 2  # pw1's rows are stored interleaved per GEMM tile
            z = z.view(z.shape[0], -1, 2, half)
            gl = (z[:, :, 0] * torch.sigmoid(z[:, :, 1])).reshape(z.shape[0], -1)
            rec[b + "glu"] = float(gl.abs().max())
            x = x + lin(b + "pw2", gl)
            h = torch.nn.functional.silu(lin(b + "ff.w1", ln(b + "ln_ff", x)))
            rec[b + "ff.h"] = float(h.abs().max())
            x = x + 0.5 * lin(b + "ff.w2", h)
            g, be = self.ln[b + "ln_final"]
            x = torch.nn.functional.layer_norm(x, (d,), g, be, cfg.eps)
        ln("after", x)
        for k, v in rec.items():
            # head-room so that unseen frames rarely exceed the calibrated range
            self.amax[k] = torch.tensor([v * 1.25], dtype=torch.float32, device=self.device)
        return rec


class CompiledStack:
    """A forward pass over a fixed number of frames captured in a CUDA graph.

    ``x_in`` (bf16 [T, d]) is the device input buffer, ``logits`` / ``ids`` the outputs;
    :meth:`run` replays on the current stream, :meth:`encode_ctc_host` is the end-to-end call:
    pinned host features in, greedy CTC ids on the host out.

    """

    def __init__(self, stack: "ConformerLinearStack", frames: int, with_pos: bool = True):
        self.stack = stack
        self.frames = frames
        cfg = stack.cfg
        dev = stack.device
        self.x_in = torch.zeros((frames, cfg.d_model), dtype=torch.bfloat16, device=dev)
        self.pos = torch.zeros((frames, cfg.d_model), dtype=torch.bfloat16, device=dev) if with_pos else None
        self._x = torch.empty_like(self.x_in)
        self._keys = torch.empty((frames,), dtype=torch.int64, device=dev)
        self._ids = torch.empty((frames,), dtype=torch.int32, device=dev)
        self.ids_host = torch.empty((frames,), dtype=torch.int32).pin_memory()
        self._stage = None
        self._ids_pool: List[torch.Tensor] = []
        ops.reset_launch_count()
        self._body()  # warm-up: lazy module loading and one-time attribute calls happen here
        self.launches = ops.launch_count()
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._body()
        torch.cuda.synchronize(dev)

    def _body(self):
        self._x.copy_(self.x_in)
        self.ids = self.stack.forward_ids(self._x, self.pos, keys=self._keys, ids=self._ids)

    def run(self):
        self.graph.replay()
        return self.ids

    def encode_ctc_host(self, feats_host: torch.Tensor) -> torch.Tensor:
        """Host bf16 [T, d] features (pinned for full copy speed) -> host int32 [T] greedy ids."""
        self.x_in.copy_(feats_host, non_blocking=True)
        self.graph.replay()
        self.ids_host.copy_(self.ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.ids_host

    def reserve_host_ids(self, n: int) -> None:
        """Pinned host id buffers for ``n`` queued batches (pinning is slow and synchronises the
        device: call this once, outside any latency-sensitive region)."""
        if len(self._ids_pool) < n:
            block = torch.empty((n - len(self._ids_pool), self.frames), dtype=torch.int32).pin_memory()
            self._ids_pool.extend(block.unbind(0))

    def encode_ctc_host_batches(self, batches: Sequence[torch.Tensor],
                                out: Optional[List[torch.Tensor]] = None, after_each=None) -> List[torch.Tensor]:
        """Throughput form of :meth:`encode_ctc_host` for a queue of utterance shards.

        ``batches``: host bf16 [T, d] tensors (pinned for full copy speed); returns one pinned
        host int32 [T] id tensor per batch (``out`` re-uses caller buffers).  The host->device
        copy of batch i+1 runs on a copy stream into one of two staging buffers while the
        stack of batch i runs, so per batch the cost is max(copy, compute) instead of their sum.
        ``after_each(i)``, if given, is called after batch i has been enqueued (multi-GPU callers
        enqueue their gather of ``self.ids`` there).  Results are complete when the call returns.
        """
        if self._stage is None:
            self._stage = [torch.empty_like(self.x_in) for _ in range(2)]
            self._h2d = torch.cuda.Stream(device=self.stack.device)
            self._ev_in = [torch.cuda.Event() for _ in range(2)]
            self._ev_free = [torch.cuda.Event() for _ in range(2)]
        if out is None:
            self.reserve_host_ids(len(batches))
            out = self._ids_pool[: len(batches)]
        main = torch.cuda.current_stream()
        self._h2d.wait_stream(main)
        for i, feats in enumerate(batches):
            s = i & 1
            with torch.cuda.stream(self._h2d):
                if i >= 2:
                    self._h2d.wait_event(self._ev_free[s])
                self._stage[s].copy_(feats, non_blocking=True)
                self._ev_in[s].record(self._h2d)
            main.wait_event(self._ev_in[s])
            self.x_in.copy_(self._stage[s])
            self._ev_free[s].record(main)
            self.graph.replay()
            out[i].copy_(self.ids, non_blocking=True)
            if after_each is not None:
                after_each(i)
        main.synchronize()
        return list(out)


# --------------------------------------------------------------------------------------
# frame sharding


def shard_rows(total: int, world: int, rank: int, multiple: int = 2) -> Tuple[int, int]:
    """Contiguous shard [start, stop) of ``total`` frames for ``rank`` of ``world``.

    Shards are equal up to rounding to ``multiple`` frames (2 keeps the row pairs of the
    per-16 "A"-side format inside one shard); trailing ranks may get fewer (or zero) frames.
    """
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world / rank")
    per = -(-total // world)
    per = -(-per // multiple) * multiple
    start = min(rank * per, total)
    stop = min(start + per, total)
    return start, stop


def shard_capacity(total: int, world: int, multiple: int = 2) -> int:
    per = -(-total // world)
    return -(-per // multiple) * multiple


def gather_rows(local: torch.Tensor, total: int, world: int, rank: int, group=None) -> torch.Tensor:
    """All-gather row shards (cut by :func:`shard_rows`) into the full [total, C] tensor.

    One ``all_gather_into_tensor`` over equal-capacity slots (NCCL on GPUs, gloo on CPU); the
    short last shards are padded in the slot and trimmed after the collective.
    """
    import torch.distributed as dist

    cap = shard_capacity(total, world)
    cols = local.shape[1]
    slot = local
    if local.shape[0] != cap or not local.is_contiguous():
        slot = torch.zeros((cap, cols), dtype=local.dtype, device=local.device)
        slot[: local.shape[0]] = local
    full = torch.empty((world * cap, cols), dtype=local.dtype, device=local.device)
    if world == 1:
        full.copy_(slot)
    else:
        dist.all_gather_into_tensor(full, slot, group=group)
    return full[:total]

"""Synthetic long-audio input of the multi-GPU benchmark configuration.

What the configuration describes: one hour of 16 kHz mono PCM -- uniform [-1, 1] noise mixed with
100-4000 Hz sines, seed 1 -- turned into 80-bin Kaldi filterbank features exactly the way the
reference's front-end does it (``torchaudio.compliance.kaldi.fbank`` on ``wav * 32768`` with a
25 ms window, 10 ms hop and ``energy_floor = 0``;
``veloxvoice/audio/frontend_torch.py:206-213``), subsampled 4x and fed to the encoder's linear
stack.  No real audio or checkpoint exists in this repository, so:

* the PCM is generated here, in blocks of ten seconds that are seeded one by one, so that a
  rank can make exactly the samples its frame shard needs and still get the samples a
  single-GPU run gets;
* the encoder's conv2d subsampling front (``torch_conformer.py:273-327``) is not a quantized
  linear and is outside this library.  It is replaced by a FIXED, seeded stand-in with the same
  shape contract: four consecutive mel frames (4 x 80 values, shifted and scaled by the
  constants below) are multiplied by a seeded N(0, 1/320) matrix [512, 320], which gives one
  512-wide encoder frame per 40 ms with roughly unit variance.

The functions are deterministic on a given device type (the sines and the filterbank are
evaluated on the device asked for); every rank calls them with its own frame range.
"""

from __future__ import annotations

import math
from typing import Tuple

import torch

SAMPLE_RATE = 16000
HOP = 160  # 10 ms
WINDOW = 400  # 25 ms
MEL_BINS = 80
SUBSAMPLE = 4
BLOCK_SAMPLES = 10 * SAMPLE_RATE  # PCM is seeded per block of ten seconds
N_SINES = 8
NOISE_GAIN = 0.05
SINE_GAIN = 0.08
# log-mel values of this signal sit around MEL_SHIFT with a spread of about MEL_SCALE
MEL_SHIFT = 19.0
MEL_SCALE = 4.0
PROJ_SEED = 20240531
HOUR_SAMPLES = 3600 * SAMPLE_RATE


def total_encoder_frames(n_samples: int = HOUR_SAMPLES) -> int:
    """Encoder frames of ``n_samples`` of audio: Kaldi frames without edge padding, 4x subsampled."""
    mel = 1 + (n_samples - WINDOW) // HOP if n_samples >= WINDOW else 0
    return mel // SUBSAMPLE


def sine_table(seed: int = 1) -> torch.Tensor:
    """[N_SINES, 3]: frequency in Hz (uniform 100-4000), phase, tremolo rate in Hz (0.05-0.5)."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(N_SINES, 3, generator=g, dtype=torch.float64)
    freq = 100.0 + 3900.0 * u[:, 0]
    phase = 2 * math.pi * u[:, 1]
    trem = 0.05 + 0.45 * u[:, 2]
    return torch.stack([freq, phase, trem], dim=1)


def pcm_block(index: int, seed: int = 1, device="cpu") -> torch.Tensor:
    """Samples [index * BLOCK_SAMPLES, (index + 1) * BLOCK_SAMPLES) of the signal, float32 in [-1, 1].

    The noise always comes from the CPU generator (so it does not depend on the device); the
    sines are evaluated in float64 on ``device``."""
    g = torch.Generator().manual_seed(seed * 1000003 + index)
    noise = torch.rand(BLOCK_SAMPLES, generator=g, dtype=torch.float32) * 2.0 - 1.0
    t = (torch.arange(BLOCK_SAMPLES, dtype=torch.float64, device=device) + float(index) * BLOCK_SAMPLES) / SAMPLE_RATE
    x = NOISE_GAIN * noise.to(device).double()
    for f, ph, tr in sine_table(seed).tolist():
        x += SINE_GAIN * (0.5 + 0.5 * torch.sin(2 * math.pi * tr * t)) * torch.sin(2 * math.pi * f * t + ph)
    return x.clamp_(-1.0, 1.0).float()


def pcm_range(start: int, stop: int, seed: int = 1, device="cpu") -> torch.Tensor:
    """Samples [start, stop) of the signal (float32 on ``device``)."""
    b0, b1 = start // BLOCK_SAMPLES, (stop - 1) // BLOCK_SAMPLES
    x = torch.cat([pcm_block(b, seed, device) for b in range(b0, b1 + 1)])
    off = start - b0 * BLOCK_SAMPLES
    return x[off: off + (stop - start)]


def projection(d_model: int = 512, device="cpu") -> torch.Tensor:
    """The stand-in for the subsampling front: seeded N(0, 1/320) matrix [d_model, 4 * 80]."""
    g = torch.Generator().manual_seed(PROJ_SEED)
    k = SUBSAMPLE * MEL_BINS
    return (torch.randn(d_model, k, generator=g) / math.sqrt(k)).to(device)


def encoder_features(frame_start: int, frame_stop: int, device="cpu", seed: int = 1,
                     d_model: int = 512) -> Tuple[torch.Tensor, torch.Tensor]:
    """Encoder input frames [frame_start, frame_stop) of the synthetic hour.

    Returns ``(features bf16 [n, d_model], mel f32 [4 n, 80])`` on ``device``.  Only the PCM that
    these frames cover is generated.
    """
    import torchaudio.compliance.kaldi as kaldi

    n = frame_stop - frame_start
    if n <= 0:
        return (torch.zeros((0, d_model), dtype=torch.bfloat16, device=device),
                torch.zeros((0, MEL_BINS), dtype=torch.float32, device=device))
    m0, m1 = frame_start * SUBSAMPLE, frame_stop * SUBSAMPLE  # mel frames
    s0, s1 = m0 * HOP, (m1 - 1) * HOP + WINDOW
    wav = pcm_range(s0, s1, seed, device)
    mel = kaldi.fbank((wav * 32768.0).unsqueeze(0), num_mel_bins=MEL_BINS, frame_length=25, frame_shift=10,
                      energy_floor=0.0, sample_frequency=SAMPLE_RATE)
    if mel.shape[0] != m1 - m0:
        raise RuntimeError(f"fbank gave {mel.shape[0]} frames for {m1 - m0}")
    stacked = ((mel - MEL_SHIFT) / MEL_SCALE).reshape(n, SUBSAMPLE * MEL_BINS)
    feats = stacked @ projection(d_model, device).T
    return feats.to(torch.bfloat16), mel

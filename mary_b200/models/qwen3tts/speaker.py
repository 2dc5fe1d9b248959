"""ECAPA-TDNN speaker encoder of Qwen3-TTS and the mel front end it consumes (src/models/qwen3tts/speaker.rs).

Mel: 24 kHz, ``n_fft = win = 1024`` (periodic Hann), hop 256, 128 Slaney-scale filters with Slaney (area) normalisation between 0
and 12 kHz; no centring — the signal is reflect-padded by ``(n_fft - hop) / 2`` on both sides; ``log(clamp(sqrt(re^2 + im^2 + 1e-9),
1e-5))``.  The STFT is two matrix products with the windowed DFT basis.

Encoder (an x-vector of 2048 dims): TDNN(128 -> 512, kernel 5) -> three SE-Res2Net blocks (kernel 3, dilations 2 / 3 / 4, Res2Net
scale 8, squeeze-excitation bottleneck 128) -> concatenate the three block outputs -> TDNN(1536, kernel 1) -> attentive statistics
pooling (attention bottleneck 128 over ``[x, mean, std]``) -> ``[mean, std]`` = 3072 -> 1 x 1 convolution -> 2048.  Every
convolution pads "same" by reflection and is followed by ReLU; there is no normalisation layer."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class EcapaConfig:
    n_mels: int = 128
    channels: int = 512
    kernel0: int = 5
    dilations: tuple = (2, 3, 4)
    res2net_scale: int = 8
    se_channels: int = 128
    att_channels: int = 128
    out_dim: int = 2048

    @staticmethod
    def tiny():
        return EcapaConfig(n_mels=16, channels=32, res2net_scale=4, se_channels=8, att_channels=8, out_dim=24)


def slaney_mel_filters(n_mels: int, n_fft: int, sr: int, fmin: float = 0.0, fmax: float | None = None):
    """Slaney-scale triangles with area normalisation ``[n_mels, n_fft / 2 + 1]``."""
    fmax = sr / 2 if fmax is None else fmax

    def to_mel(f):
        return f / (200.0 / 3) if f < 1000.0 else 15.0 + math.log(f / 1000.0) / (math.log(6.4) / 27.0)

    def to_hz(m):
        return torch.where(m >= 15.0, 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))
    pts = to_hz(torch.linspace(to_mel(fmin), to_mel(fmax), n_mels + 2, dtype=torch.float64))
    freqs = torch.linspace(0, sr / 2, n_fft // 2 + 1, dtype=torch.float64)
    lo, mid, hi = pts[:-2, None], pts[1:-1, None], pts[2:, None]
    tri = torch.minimum((freqs - lo) / (mid - lo), (hi - freqs) / (hi - mid)).clamp_min(0.0)
    return (tri * (2.0 / (hi - lo))).float()


def speaker_mel(wave, n_mels: int = 128, n_fft: int = 1024, hop: int = 256, sr: int = 24000, fmax: float = 12000.0):
    """``wave [L]`` -> ``[n_mels, frames]`` with ``frames = L / hop`` for ``L`` a multiple of ``hop``."""
    pad = (n_fft - hop) // 2
    x = F.pad(torch.as_tensor(wave, dtype=torch.float32)[None, None], (pad, pad), mode="reflect")[0, 0]
    frames = x.unfold(0, n_fft, hop) * torch.hann_window(n_fft, device=x.device)
    n = torch.arange(n_fft, dtype=torch.float64, device=x.device)
    k = torch.arange(n_fft // 2 + 1, dtype=torch.float64, device=x.device)
    ang = 2.0 * math.pi * n[:, None] * k[None, :] / n_fft
    re, im = frames @ ang.cos().float(), frames @ ang.sin().float()
    mag = torch.sqrt(re * re + im * im + 1e-9).T
    return (slaney_mel_filters(n_mels, n_fft, sr, 0.0, fmax).to(x.device) @ mag).clamp_min(1e-5).log()


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


class TDNN(nn.Module):
    def __init__(self, cin, cout, k, dilation=1):
        super().__init__()
        self.w, self.b, self.k, self.d = _P(cout, cin, k), _P(cout), k, dilation

    def forward(self, x, act=True):
        """``x [C, T]`` -> ``[C', T]`` (reflect "same" padding)."""
        p = self.d * (self.k - 1) // 2
        y = F.conv1d(F.pad(x[None], (p, p), mode="reflect") if p else x[None], self.w, self.b, dilation=self.d)[0]
        return F.relu(y) if act else y


class SERes2NetBlock(nn.Module):
    def __init__(self, c: EcapaConfig, dilation: int):
        super().__init__()
        C, s = c.channels, c.res2net_scale
        self.scale = s
        self.tdnn1, self.tdnn2 = TDNN(C, C, 1), TDNN(C, C, 1)
        self.res = nn.ModuleList([TDNN(C // s, C // s, 3, dilation) for _ in range(s - 1)])
        self.se1, self.se2 = TDNN(C, c.se_channels, 1), TDNN(c.se_channels, C, 1)

    def forward(self, x):
        h = self.tdnn1(x)
        parts, prev, out = h.chunk(self.scale, 0), None, []
        for i, p in enumerate(parts):                      # chunk 0 passes through; chunk i sees chunk i plus the previous result
            if i == 0:
                y = p
            else:
                y = self.res[i - 1](p if i == 1 else p + prev)
                prev = y
            out.append(y)
        h = self.tdnn2(torch.cat(out, 0))
        s = torch.sigmoid(self.se2(self.se1(h.mean(1, keepdim=True)), act=False))
        return x + h * s


class Ecapa(nn.Module):
    def __init__(self, c: EcapaConfig):
        super().__init__()
        self.c = c
        C = c.channels
        self.tdnn0 = TDNN(c.n_mels, C, c.kernel0)
        self.blocks = nn.ModuleList([SERes2NetBlock(c, d) for d in c.dilations])
        n = C * len(c.dilations)
        self.mfa = TDNN(n, n, 1)
        self.att1, self.att2 = TDNN(3 * n, c.att_channels, 1), TDNN(c.att_channels, n, 1)
        self.fc = TDNN(2 * n, c.out_dim, 1)

    def pool(self, x):
        """Attentive statistics: attention logits from ``[x, mean, std]`` through a ReLU time-delay layer, then tanh, then a plain
        convolution (speaker.rs:186); softmax over time; weighted mean and std."""
        T = x.shape[1]
        mean, std = x.mean(1, keepdim=True), x.var(1, unbiased=False, keepdim=True).clamp_min(1e-12).sqrt()
        a = self.att2(torch.tanh(self.att1(torch.cat([x, mean.expand(-1, T), std.expand(-1, T)], 0))), act=False)
        w = torch.softmax(a, dim=1)
        m = (w * x).sum(1, keepdim=True)
        s = ((w * (x - m) ** 2).sum(1, keepdim=True)).clamp_min(1e-12).sqrt()
        return torch.cat([m, s], 0)

    @torch.no_grad()
    def forward(self, mel):
        """``mel [n_mels, T]`` -> speaker vector ``[out_dim]``."""
        x = self.tdnn0(mel.to(self.tdnn0.w.dtype))
        outs = []
        for b in self.blocks:
            x = b(x)
            outs.append(x)
        x = self.mfa(torch.cat(outs, 0))
        return self.fc(self.pool(x), act=False)[:, 0]


def load_into(m: Ecapa, loader, prefix: str = "speaker_encoder.") -> None:
    """Checkpoint names of the released speaker encoder (speaker.rs:60-165): time-delay layers keep their convolution under
    ``.conv``; the squeeze-excitation pair, the attention's output convolution and the final projection are bare convolutions:
    ``blocks.0.conv``, ``blocks.<i>.{tdnn1.conv, res2net_block.blocks.<j>.conv, tdnn2.conv, se_block.conv1, se_block.conv2}``,
    ``mfa.conv``, ``asp.tdnn.conv``, ``asp.conv``, ``fc``."""
    def put(t: TDNN, name: str):
        for p, leaf in ((t.w, ".weight"), (t.b, ".bias")):
            x = loader.load_tensor(prefix + name + leaf, p.dtype)
            if tuple(x.shape) != tuple(p.shape):
                raise ValueError(f"{prefix}{name}{leaf}: stored {tuple(x.shape)}, expected {tuple(p.shape)}")
            p.data.copy_(x)
    put(m.tdnn0, "blocks.0.conv")
    for i, b in enumerate(m.blocks, start=1):
        put(b.tdnn1, f"blocks.{i}.tdnn1.conv"), put(b.tdnn2, f"blocks.{i}.tdnn2.conv")
        for j, r in enumerate(b.res):
            put(r, f"blocks.{i}.res2net_block.blocks.{j}.conv")
        put(b.se1, f"blocks.{i}.se_block.conv1"), put(b.se2, f"blocks.{i}.se_block.conv2")
    put(m.mfa, "mfa.conv"), put(m.att1, "asp.tdnn.conv"), put(m.att2, "asp.conv"), put(m.fc, "fc")

"""Vocos vocoder: mel -> waveform through an inverse STFT head (the separate model F5-TTS decodes with; src/models/f5).

Backbone: 1-D convolution (kernel 7) into ``dim`` channels, LayerNorm, ``layers`` ConvNeXt blocks (depthwise kernel-7 convolution,
LayerNorm, ``dim -> 3 dim`` GELU MLP back to ``dim``, learned per-channel layer scale, residual), LayerNorm.  Head: a linear layer
to ``n_fft + 2`` channels = log-magnitude and phase of every bin; ``exp`` (clipped at 100) and ``cos / sin`` give the complex
spectrum, the inverse STFT (as matrix products, ``spectral.istft_matmul``) the samples."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from .spectral import istft_matmul


@dataclass
class VocosConfig:
    n_mels: int = 100
    dim: int = 512
    ffn: int = 1536
    layers: int = 8
    n_fft: int = 1024
    hop: int = 256

    @staticmethod
    def tiny():
        return VocosConfig(n_mels=12, dim=16, ffn=32, layers=2, n_fft=64, hop=16)


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


class VocosBlock(nn.Module):
    def __init__(self, c: VocosConfig):
        super().__init__()
        self.dw_w, self.dw_b = _P(c.dim, 1, 7), _P(c.dim)
        self.ln_w, self.ln_b = _P(c.dim), _P(c.dim)
        self.w1, self.b1, self.w2, self.b2, self.gamma = _P(c.ffn, c.dim), _P(c.ffn), _P(c.dim, c.ffn), _P(c.dim), _P(c.dim)

    def forward(self, x):
        """``x [T, dim]``."""
        h = F.conv1d(x.T[None], self.dw_w, self.dw_b, padding=3, groups=x.shape[1])[0].T
        h = F.layer_norm(h, (x.shape[1],), self.ln_w, self.ln_b, 1e-6)
        h = ops.linear(F.gelu(ops.linear(h.contiguous(), self.w1, self.b1)), self.w2, self.b2)
        return x + self.gamma * h


class Vocos(nn.Module):
    def __init__(self, c: VocosConfig):
        super().__init__()
        self.c = c
        self.embed_w, self.embed_b = _P(c.dim, c.n_mels, 7), _P(c.dim)
        self.ln0_w, self.ln0_b, self.lnf_w, self.lnf_b = _P(c.dim), _P(c.dim), _P(c.dim), _P(c.dim)
        self.blocks = nn.ModuleList([VocosBlock(c) for _ in range(c.layers)])
        self.out_w, self.out_b = _P(c.n_fft + 2, c.dim), _P(c.n_fft + 2)

    def spectrum(self, mel):
        c = self.c
        x = F.conv1d(mel[None].to(self.embed_w.dtype), self.embed_w, self.embed_b, padding=3)[0].T
        x = F.layer_norm(x, (c.dim,), self.ln0_w, self.ln0_b, 1e-6)
        for b in self.blocks:
            x = b(x)
        x = F.layer_norm(x, (c.dim,), self.lnf_w, self.lnf_b, 1e-6)
        y = ops.linear(x.contiguous(), self.out_w, self.out_b).float().T                       # [n_fft + 2, T]
        mag, phase = y[:c.n_fft // 2 + 1].exp().clamp_max(1e2), y[c.n_fft // 2 + 1:]
        return torch.complex(mag * phase.cos(), mag * phase.sin())

    @torch.no_grad()
    def forward(self, mel):
        """``mel [n_mels, T]`` -> waveform ``[T * hop]``."""
        return istft_matmul(self.spectrum(mel), self.c.n_fft, self.c.hop, length=mel.shape[1] * self.c.hop)


def load_into(m: Vocos, loader) -> None:
    """Names of the ``charactr/vocos-mel-24khz`` checkpoint (``backbone.*``, ``head.out``)."""
    dt = m.embed_w.dtype

    def put(p, n):
        p.data.copy_(loader.load_tensor(n, dt).reshape(p.shape))
    for p, n in ((m.embed_w, "backbone.embed.weight"), (m.embed_b, "backbone.embed.bias"), (m.ln0_w, "backbone.norm.weight"), (m.ln0_b, "backbone.norm.bias"),
                 (m.lnf_w, "backbone.final_layer_norm.weight"), (m.lnf_b, "backbone.final_layer_norm.bias"), (m.out_w, "head.out.weight"),
                 (m.out_b, "head.out.bias")):
        put(p, n)
    for i, b in enumerate(m.blocks):
        t = f"backbone.convnext.{i}."
        for p, n in ((b.dw_w, "dwconv.weight"), (b.dw_b, "dwconv.bias"), (b.ln_w, "norm.weight"), (b.ln_b, "norm.bias"), (b.w1, "pwconv1.weight"),
                     (b.b1, "pwconv1.bias"), (b.w2, "pwconv2.weight"), (b.b2, "pwconv2.bias"), (b.gamma, "gamma")):
            put(p, t + n)

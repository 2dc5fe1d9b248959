"""Gemma-4 audio tower: log-mel frames -> soft tokens in the decoder's embedding space (src/models/gemma/gemma4/audio.rs:364-526,
a Conformer / Universal-Speech-Model encoder).

Pipeline for one utterance ``mel [T, n_mels]``: two 3 x 3 stride-2 convolutions over (time, frequency), each followed by a
LayerNorm over channels and ReLU, flatten (frequency, channel) and project -> ``T / 4`` frames.  Every block is
half-step FFN -> local attention -> light convolution -> half-step FFN -> RMSNorm:

* FFN: RMSNorm, 4x SiLU MLP, RMSNorm, added with weight 0.5.
* attention: every frame attends to itself and the ``left - 2`` frames before it.  Queries are scaled per dimension by
  ``softplus(per_dim_scale) / (sqrt(d) ln 2)``, keys by ``log2(1 + e)``; a relative-position term ``q . W_rel sinusoid(distance)`` is
  added to the content logits; the sum is soft-capped with ``cap * tanh(x / cap)`` before the softmax.  (The checkpoint's code
  evaluates this in blocks of 12 queries with a shifted bias matrix; per query it is the windowed form used here.)
* light convolution: RMSNorm, linear to 2H, GLU, causal depthwise convolution (kernel 5), RMSNorm, SiLU, linear, residual.

A biased output projection and the multimodal embedder (weightless RMSNorm + projection) map frames to the decoder's width:
one soft token per 40 ms of audio."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from .vision import ClipLinear


@dataclass
class Gemma4AudioConfig:
    n_mels: int = 128
    hidden: int = 1024
    layers: int = 12
    heads: int = 8
    conv_channels: tuple = (128, 32)
    conv_kernel: int = 5
    residual_weight: float = 0.5
    context_left: int = 13
    logit_cap: float = 50.0
    eps: float = 1e-6
    out_dims: int = 1536
    text_hidden: int = 2304

    @staticmethod
    def tiny():
        return Gemma4AudioConfig(n_mels=16, hidden=32, layers=2, heads=4, conv_channels=(16, 8), context_left=5, out_dims=24, text_hidden=20)


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


def usm_log_mel(wave, sr: int = 16000, n_mels: int = 128, frame_ms: float = 20.0, hop_ms: float = 10.0, fmin: float = 0.0, fmax: float = 8000.0,
                mel_floor: float = 1e-3):
    """The tower's front end (the ``gemma_hear`` / ``gemma_listen`` mel): ``frame_length // 2`` zeros are prepended (semi-causal
    framing), frames of ``frame_ms`` every ``hop_ms``, periodic Hann window, FFT of the next power of two, MAGNITUDE spectrum, HTK
    mel triangles without normalisation, ``log(mel + floor)``.  Returns ``[frames, n_mels]``."""
    from ..f5.spectral import mel_filterbank_htk
    x = torch.as_tensor(wave, dtype=torch.float32)
    fl, hop = int(round(sr * frame_ms / 1000.0)), int(round(sr * hop_ms / 1000.0))
    n_fft = 1 << (fl - 1).bit_length()
    x = F.pad(x, (fl // 2, 0))
    if x.shape[0] < fl + 1:
        return torch.zeros(0, n_mels)
    frames = x.unfold(0, fl + 1, hop)[:, :fl] * torch.hann_window(fl, periodic=True)
    mag = torch.fft.rfft(frames, n=n_fft).abs()
    fb = mel_filterbank_htk(n_mels, n_fft, sr, fmin, fmax)
    return torch.log(mag @ fb.T + mel_floor)


class FFN(nn.Module):
    def __init__(self, H):
        super().__init__()
        self.l1, self.l2, self.pre, self.post = ClipLinear(4 * H, H), ClipLinear(H, 4 * H), _P(H), _P(H)

    def forward(self, x, c):
        h = self.l2(F.silu(self.l1(ops.rmsnorm(x, self.pre, c.eps)).float()).to(x.dtype))
        return x + ops.rmsnorm(h, self.post, c.eps) * c.residual_weight


class AudioLayer(nn.Module):
    def __init__(self, c: Gemma4AudioConfig):
        super().__init__()
        H = c.hidden
        self.ff1, self.ff2 = FFN(H), FFN(H)
        self.q, self.k, self.v, self.post = ClipLinear(H, H), ClipLinear(H, H), ClipLinear(H, H), ClipLinear(H, H)
        self.rel_k, self.per_dim_scale = _P(H, H), _P(H // c.heads)
        self.n_pre_attn, self.n_post_attn, self.n_out = _P(H), _P(H), _P(H)
        self.lc_start, self.lc_end, self.lc_conv = ClipLinear(2 * H, H), ClipLinear(H, H), _P(H, 1, c.conv_kernel)
        self.lc_pre, self.lc_norm = _P(H), _P(H)


class Gemma4AudioTower(nn.Module):
    def __init__(self, c: Gemma4AudioConfig):
        super().__init__()
        self.c = c
        c0, c1 = c.conv_channels
        self.conv0, self.ln0, self.conv1, self.ln1 = _P(c0, 1, 3, 3), _P(c0), _P(c1, c0, 3, 3), _P(c1)
        self.in_proj = _P(c.hidden, (c.n_mels // 4) * c1)
        self.layers = nn.ModuleList([AudioLayer(c) for _ in range(c.layers)])
        self.out_w, self.out_b, self.embed_proj = _P(c.out_dims, c.hidden), _P(c.out_dims), _P(c.text_hidden, c.out_dims)
        n = c.hidden // 2
        inc = math.log(10000.0) / max(n - 1, 1)
        d = torch.arange(c.context_left - 1, -1, -1, dtype=torch.float32)[:, None]                  # window slot w holds distance left-1-w
        t = d * torch.exp(torch.arange(n, dtype=torch.float32) * -inc)
        self.register_buffer("rel_code", torch.cat([t.sin(), t.cos()], -1), persistent=False)      # [left, hidden]

    def subsample(self, mel):
        c = self.c
        x = mel.T[None, None].transpose(2, 3).to(self.conv0.dtype)                                  # [1, 1, T, F]
        for w, g in ((self.conv0, self.ln0), (self.conv1, self.ln1)):
            x = F.conv2d(x, w, stride=2, padding=1)
            x = F.relu(F.layer_norm(x.permute(0, 2, 3, 1), (w.shape[0],), g, None, c.eps)).permute(0, 3, 1, 2)
        T4 = x.shape[2]
        return ops.linear(x[0].permute(1, 2, 0).reshape(T4, -1).contiguous(), self.in_proj)

    def attention(self, L: AudioLayer, x):
        c = self.c
        T, nh, W = x.shape[0], c.heads, c.context_left
        hd = c.hidden // nh
        q = L.q(x).float().view(T, nh, hd) * ((hd ** -0.5) / math.log(2.0)) * F.softplus(L.per_dim_scale.float())
        k = L.k(x).float().view(T, nh, hd) * (math.log(1.0 + math.e) / math.log(2.0))
        v = L.v(x).float().view(T, nh, hd)
        # window slot w of query t is key t - (W - 1) + w
        kw = F.pad(k, (0, 0, 0, 0, W - 1, 0)).unfold(0, W, 1)                                      # [T, nh, hd, W]
        vw = F.pad(v, (0, 0, 0, 0, W - 1, 0)).unfold(0, W, 1)
        rel = ops.linear(self.rel_code.to(L.rel_k.dtype), L.rel_k).float().view(W, nh, hd)
        logits = torch.einsum("thd,thdw->thw", q, kw) + torch.einsum("thd,whd->thw", q, rel)
        logits = c.logit_cap * torch.tanh(logits / c.logit_cap)
        # the checkpoint's mask admits distances 0 .. left - 2: the slot of distance left - 1 exists in the bias table but is never seen
        valid = ((torch.arange(T)[:, None] - (W - 1) + torch.arange(W)[None, :] >= 0) & (torch.arange(W)[None, :] >= 1)).to(x.device)
        p = torch.softmax(logits.masked_fill(~valid[:, None, :], -1e9), -1)
        return L.post(torch.einsum("thw,thdw->thd", p, vw).reshape(T, c.hidden).to(x.dtype))

    def light_conv(self, L: AudioLayer, x):
        c = self.c
        h = F.glu(L.lc_start(ops.rmsnorm(x, L.lc_pre, c.eps)), dim=-1)
        h = F.conv1d(F.pad(h.T[None], (c.conv_kernel - 1, 0)), L.lc_conv, groups=c.hidden)[0].T.contiguous()
        return x + L.lc_end(F.silu(ops.rmsnorm(h, L.lc_norm, c.eps).float()).to(x.dtype))

    def encode(self, mel):
        """``mel [T, n_mels]`` -> ``[T / 4, out_dims]``."""
        c = self.c
        x = self.subsample(mel)
        for L in self.layers:
            x = L.ff1(x, c)
            x = x + ops.rmsnorm(self.attention(L, ops.rmsnorm(x, L.n_pre_attn, c.eps)), L.n_post_attn, c.eps)
            x = L.ff2(self.light_conv(L, x), c)
            x = ops.rmsnorm(x, L.n_out, c.eps)
        return ops.linear(x, self.out_w, self.out_b)

    def forward(self, mel):
        """Soft tokens of one utterance in the decoder's width."""
        return ops.linear(ops.rmsnorm(self.encode(mel), None, self.c.eps), self.embed_proj)


def load_into(m: Gemma4AudioTower, loader, prefix: str = "model.audio_tower.", embed_prefix: str = "model.embed_audio.") -> None:
    """Names of the Hugging Face ``Gemma4ForConditionalGeneration`` layout (``audio_tower.*`` and ``embed_audio.*``)."""
    dt = m.in_proj.dtype

    def get(n):
        return loader.load_tensor(n, dt)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))

    def lin(l, n):
        put(l.w, n + ".linear.weight")
        if loader.has_weight(n + ".input_min"):
            l.bounds.copy_(torch.stack([get(n + "." + b).float().reshape(()) for b in ("input_min", "input_max", "output_min", "output_max")]))
            l.clipped = bool(torch.isfinite(l.bounds).any())
    s = prefix + "subsample_conv_projection."
    for ours, theirs in (("conv0", "layer0.conv.weight"), ("ln0", "layer0.norm.weight"), ("conv1", "layer1.conv.weight"),
                         ("ln1", "layer1.norm.weight"), ("in_proj", "input_proj_linear.weight")):
        put(getattr(m, ours), s + theirs)
    put(m.out_w, prefix + "output_proj.weight")
    put(m.out_b, prefix + "output_proj.bias")
    put(m.embed_proj, embed_prefix + "embedding_projection.weight")
    for i, L in enumerate(m.layers):
        p = f"{prefix}layers.{i}."
        for ff, name in ((L.ff1, "feed_forward1."), (L.ff2, "feed_forward2.")):
            lin(ff.l1, p + name + "ffw_layer_1")
            lin(ff.l2, p + name + "ffw_layer_2")
            put(ff.pre, p + name + "pre_layer_norm.weight")
            put(ff.post, p + name + "post_layer_norm.weight")
        for l, name in ((L.q, "self_attn.q_proj"), (L.k, "self_attn.k_proj"), (L.v, "self_attn.v_proj"), (L.post, "self_attn.post"),
                        (L.lc_start, "lconv1d.linear_start"), (L.lc_end, "lconv1d.linear_end")):
            lin(l, p + name)
        for ours, theirs in (("rel_k", "self_attn.relative_k_proj.weight"), ("per_dim_scale", "self_attn.per_dim_scale"),
                             ("n_pre_attn", "norm_pre_attn.weight"), ("n_post_attn", "norm_post_attn.weight"), ("n_out", "norm_out.weight"),
                             ("lc_conv", "lconv1d.depthwise_conv1d.weight"), ("lc_pre", "lconv1d.pre_layer_norm.weight"),
                             ("lc_norm", "lconv1d.conv_norm.weight")):
            put(getattr(L, ours), p + theirs)

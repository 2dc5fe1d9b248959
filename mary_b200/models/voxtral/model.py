"""Voxtral realtime: streaming speech-to-text (src/models/voxtral/*: mel front end, causal convolution stem, 32-layer audio
encoder with a 750-frame attention window, 4-frame projector, 26-layer decoder whose MLP input is modulated by the transcription
delay).

Data flow of one 80 ms step: 8 new mel frames -> causal conv stem (kernel 3, then kernel 3 stride 2; the stem keeps the last
input frames of the previous chunk instead of zero padding) -> 4 encoder frames appended to the encoder's paged KV cache (RoPE,
causal sliding window, biased q / v / o and down projections) -> the 4 frames concatenated and projected (GELU MLP) to ONE vector
in the decoder's width -> added to the embedding of the previous output token -> one decoder step.  Every decoder layer scales
its post-attention-normed activations by ``1 + W2 gelu(W1 t)`` where ``t`` is the sinusoidal code of the delay (in tokens)
between audio and text: the same weights transcribe with different latencies.

Both transformers run on the package's paged-cache ops, so a stream is a sequence in the cache and many streams batch like
decoder sequences."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...ops import reference as ref
from ...runtime.batch import BatchMeta
from ...runtime.kv_cache import PagedKVCache


@dataclass
class VoxtralConfig:
    n_mels: int = 128
    a_hidden: int = 1280
    a_layers: int = 32
    a_heads: int = 32
    a_head_dim: int = 64
    a_ffn: int = 5120
    a_window: int = 750
    a_theta: float = 1e6
    downsample: int = 4
    vocab: int = 131072
    hidden: int = 3072
    layers: int = 26
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 9216
    theta: float = 1e6
    window: int = 8192
    ada_dim: int = 32
    eps: float = 1e-5
    delay_tokens: int = 6
    tie: bool = True
    bos: int = 1
    pad: int = 32            # the streaming pad token that fills the delay

    @staticmethod
    def tiny():
        return VoxtralConfig(n_mels=16, a_hidden=32, a_layers=2, a_heads=4, a_head_dim=8, a_ffn=64, a_window=12, a_theta=1e4, vocab=90,
                             hidden=48, layers=2, heads=4, kv_heads=2, head_dim=12, ffn=80, theta=1e4, window=64, delay_tokens=2, pad=5)


def log_mel(wave, n_mels: int = 128, n_fft: int = 400, hop: int = 160, sr: int = 16000, global_max: float | None = 1.5):
    """Whisper-style log-mel spectrogram ``[n_mels, frames]`` of a mono waveform: Hann window, power spectrum, Slaney mel filters,
    ``log10`` clamped at 1e-10, floored 8 below the maximum (a FIXED maximum when streaming, since the true one is not known yet),
    then ``(x + 4) / 4``."""
    wave = torch.as_tensor(wave, dtype=torch.float32)
    spec = torch.stft(wave, n_fft, hop, window=torch.hann_window(n_fft), return_complex=True)[:, :-1].abs() ** 2
    mel = mel_filters(n_mels, n_fft, sr) @ spec
    x = mel.clamp_min(1e-10).log10()
    top = x.max() if global_max is None else torch.tensor(global_max)
    return (torch.maximum(x, top - 8.0) + 4.0) / 4.0


def mel_filters(n_mels: int, n_fft: int, sr: int):
    """Slaney-scale triangular filters with area normalisation ``[n_mels, n_fft / 2 + 1]``."""
    def hz_to_mel(f):
        f = torch.as_tensor(f, dtype=torch.float64)
        lin = f / (200.0 / 3)
        return torch.where(f >= 1000.0, 15.0 + torch.log(f / 1000.0) / (math.log(6.4) / 27.0), lin)

    def mel_to_hz(m):
        lin = m * (200.0 / 3)
        return torch.where(m >= 15.0, 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0)), lin)
    freqs = torch.linspace(0, sr / 2, n_fft // 2 + 1, dtype=torch.float64)
    pts = mel_to_hz(torch.linspace(float(hz_to_mel(0.0)), float(hz_to_mel(sr / 2)), n_mels + 2, dtype=torch.float64))
    lo, mid, hi = pts[:-2, None], pts[1:-1, None], pts[2:, None]
    tri = torch.minimum((freqs - lo) / (mid - lo), (hi - freqs) / (hi - mid)).clamp_min(0.0)
    return (tri * (2.0 / (hi - lo))).float()


def _P(*s, **kw):
    return nn.Parameter(torch.empty(*s, **kw), requires_grad=False)


class Layer(nn.Module):
    """Pre-RMSNorm block over the paged cache.  ``audio`` layers have q / v / o / down biases and no delay modulation."""

    def __init__(self, H, heads, kv_heads, D, ffn, audio: bool, ada_dim: int, kw):
        super().__init__()
        self.heads, self.kv, self.D, self.audio = heads, kv_heads, D, audio
        n = (heads + 2 * kv_heads) * D
        self.ln1, self.ln2 = _P(H, **kw), _P(H, **kw)
        self.w_qkv, self.w_o, self.w_gu, self.w_down = _P(n, H, **kw), _P(H, heads * D, **kw), _P(2 * ffn, H, **kw), _P(H, ffn, **kw)
        if audio:
            self.b_qkv, self.b_o, self.b_down = _P(n, **kw), _P(H, **kw), _P(H, **kw)         # the k slice of b_qkv stays zero
        else:
            self.ada1, self.ada2 = _P(ada_dim, H, **kw), _P(H, ada_dim, **kw)

    def forward(self, h, meta, kc, vc, inv_freq, window, eps, mod=None):
        x = ops.rmsnorm(h, self.ln1, eps)
        qkv = ops.linear(x, self.w_qkv, self.b_qkv if self.audio else None)
        q = ops.qk_norm_rope_append(qkv, self.heads, self.kv, self.D, None, None, False, inv_freq, meta, kc, vc, eps)
        o = ops.paged_attention(q, kc, vc, meta, self.D ** -0.5, window)
        h = h + ops.linear(o.reshape(o.shape[0], -1), self.w_o, self.b_o if self.audio else None)
        x = ops.rmsnorm(h, self.ln2, eps)
        if mod is not None:
            x = (x.float() * mod).to(h.dtype)
        return h + ops.linear(ops.linear_glu(x, self.w_gu, "swiglu"), self.w_down, self.b_down if self.audio else None)


class VoxtralModel(nn.Module):
    def __init__(self, c: VoxtralConfig, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.c = c
        kw = dict(dtype=dtype, device=device)
        A, H = c.a_hidden, c.hidden
        self.conv1_w, self.conv1_b, self.conv2_w, self.conv2_b = _P(A, c.n_mels, 3, **kw), _P(A, **kw), _P(A, A, 3, **kw), _P(A, **kw)
        self.a_layers = nn.ModuleList([Layer(A, c.a_heads, c.a_heads, c.a_head_dim, c.a_ffn, True, 0, kw) for _ in range(c.a_layers)])
        self.a_norm = _P(A, **kw)
        self.proj1, self.proj2 = _P(H, A * c.downsample, **kw), _P(H, H, **kw)
        self.embed, self.norm = _P(c.vocab, H, **kw), _P(H, **kw)
        self.lm_head = None if c.tie else _P(c.vocab, H, **kw)
        self.layers = nn.ModuleList([Layer(H, c.heads, c.kv_heads, c.head_dim, c.ffn, False, c.ada_dim, kw) for _ in range(c.layers)])
        self.register_buffer("a_inv_freq", ref.rope_inv_freq(c.a_head_dim, c.a_theta, 1.0, device), persistent=False)
        self.register_buffer("inv_freq", ref.rope_inv_freq(c.head_dim, c.theta, 1.0, device), persistent=False)

    # -- pieces
    def stem(self, mel, state=None):
        """``mel [n_mels, 2k]`` -> ``[k, A]`` encoder inputs.  ``state`` = (last 2 mel frames, last conv1 output frame) of the stream so
        far (zeros at its start); returns the new state."""
        c = self.c
        dt = self.conv1_w.dtype
        if state is None:
            state = (torch.zeros(c.n_mels, 2, dtype=dt, device=mel.device), torch.zeros(c.a_hidden, 1, dtype=dt, device=mel.device))
        x = torch.cat([state[0], mel.to(dt)], 1)
        y1 = F.gelu(F.conv1d(x[None], self.conv1_w, self.conv1_b))[0]
        z = torch.cat([state[1], y1], 1)
        y2 = F.gelu(F.conv1d(z[None], self.conv2_w, self.conv2_b, stride=2))[0]
        return y2.T.contiguous(), (x[:, -2:], z[:, -1:])

    def encode(self, x, meta, cache):
        for i, L in enumerate(self.a_layers):
            x = L(x, meta, cache.k[i], cache.v[i], self.a_inv_freq, self.c.a_window, self.c.eps)
        return ops.rmsnorm(x, self.a_norm, self.c.eps)

    def project(self, enc):
        """``enc [4k, A]`` -> ``[k, H]``: every ``downsample`` consecutive frames become one decoder-width vector."""
        c = self.c
        y = ops.linear(enc.reshape(-1, c.a_hidden * c.downsample), self.proj1)
        return ops.linear(F.gelu(y.float()).to(enc.dtype), self.proj2)

    def delay_code(self, delay_tokens: float, device):
        H = self.c.hidden
        inv = torch.exp(-math.log(10000.0) * torch.arange(H // 2, dtype=torch.float32, device=device) / (H // 2))
        return torch.cat([(delay_tokens * inv).cos(), (delay_tokens * inv).sin()])

    def modulations(self, delay_tokens: float):
        """Per decoder layer ``1 + W2 gelu(W1 t)`` (f32 ``[H]``); depends only on the delay, so it is computed once per stream."""
        t = self.delay_code(delay_tokens, self.embed.device).to(self.embed.dtype)[None]
        return [1.0 + ops.linear(F.gelu(ops.linear(t, L.ada1).float()).to(t.dtype), L.ada2).float()[0] for L in self.layers]

    def decode(self, h, meta, cache, mods):
        for i, L in enumerate(self.layers):
            h = L(h, meta, cache.k[i], cache.v[i], self.inv_freq, self.c.window, self.c.eps, mods[i])
        return ops.rmsnorm(h, self.norm, self.c.eps)

    def logits(self, x):
        return ops.linear(x, self.embed if self.lm_head is None else self.lm_head).float()

    @torch.no_grad()
    def forward(self, ids, mel, delay_tokens: float | None = None, page: int = 16):
        """Teacher-forced logits ``[T, vocab]`` of a whole utterance: ``ids [T]`` input tokens, ``mel [n_mels, 8 T]``."""
        c = self.c
        T = len(ids)
        n_pages = -(-max(mel.shape[1] // 2, T) // page) + 1
        ac, tc = self.caches(n_pages, page)

        def meta(cache, n):
            cache.alloc.extend(0, n)
            table, lens = cache.alloc.page_table([0])
            return BatchMeta.build([n], lens, table, page, device=self.embed.device)
        x, _ = self.stem(mel.to(self.embed.device))
        audio = self.project(self.encode(x, meta(ac, x.shape[0]), ac))
        h = (self.embed[torch.as_tensor(ids, device=self.embed.device).long()].float() + audio[:T].float()).to(self.embed.dtype)
        mods = self.modulations(float(c.delay_tokens if delay_tokens is None else delay_tokens))
        return self.logits(self.decode(h, meta(tc, T), tc, mods))

    def caches(self, n_pages=64, page=16, dtype=None, device=None):
        c, dt, dev = self.c, dtype or self.embed.dtype, device or self.embed.device
        return (PagedKVCache(c.a_layers, n_pages, page, c.a_heads, c.a_head_dim, dtype=dt, device=dev),
                PagedKVCache(c.layers, n_pages, page, c.kv_heads, c.head_dim, dtype=dt, device=dev))


class VoxtralListener:
    """One stream: ``feed(mel_chunk)`` with ``2 * downsample`` mel frames per text position, returns the greedy tokens of the new positions."""

    def __init__(self, model: VoxtralModel, delay_tokens: int | None = None, n_pages: int = 64, page: int = 16):
        self.m, self.page = model, page
        self.acache, self.tcache = model.caches(n_pages, page)
        self.state = None
        self.delay = model.c.delay_tokens if delay_tokens is None else delay_tokens
        self.mods = model.modulations(float(self.delay))
        self.prev = model.c.bos
        self.tokens: list[int] = []

    def _meta(self, cache, n):
        cache.alloc.extend(0, n)
        table, lens = cache.alloc.page_table([0])
        return BatchMeta.build([n], lens, table, self.page, device=self.m.embed.device)

    @torch.no_grad()
    def feed(self, mel, forced=None):
        """``mel [n_mels, 8k]`` -> ``k`` tokens.  ``forced``: ids to feed back instead of the model's own choices (teacher forcing)."""
        m, c = self.m, self.m.c
        x, self.state = m.stem(mel.to(m.embed.device), self.state)
        enc = m.encode(x, self._meta(self.acache, x.shape[0]), self.acache)
        audio = m.project(enc)
        out = []
        for j in range(audio.shape[0]):
            h = (m.embed[self.prev].float() + audio[j].float()).to(audio.dtype)[None]
            tok = int(m.logits(m.decode(h, self._meta(self.tcache, 1), self.tcache, self.mods))[0].argmax())
            out.append(tok)
            pos = len(self.tokens) + len(out)
            self.prev = forced[pos - 1] if forced is not None else (c.pad if pos <= self.delay else tok)
        self.tokens += out
        return out


def load_into(m: VoxtralModel, loader) -> None:
    """Names of the Hugging Face ``VoxtralRealtimeForConditionalGeneration`` layout."""
    dt = m.embed.dtype

    def get(n):
        return loader.load_tensor(n, dt)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    a = "audio_tower."
    for ours, theirs in (("conv1_w", "embedder.conv1.weight"), ("conv1_b", "embedder.conv1.bias"), ("conv2_w", "embedder.conv2.weight"),
                         ("conv2_b", "embedder.conv2.bias"), ("a_norm", "norm.weight")):
        put(getattr(m, ours), a + theirs)
    for i, L in enumerate(m.a_layers):
        p = f"{a}layers.{i}."
        L.w_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
        bq, bv = get(p + "self_attn.q_proj.bias"), get(p + "self_attn.v_proj.bias")
        L.b_qkv.data.copy_(torch.cat([bq, torch.zeros_like(bv), bv], 0))
        for ours, theirs in (("w_o", "self_attn.o_proj.weight"), ("b_o", "self_attn.o_proj.bias"), ("w_down", "mlp.down_proj.weight"),
                             ("b_down", "mlp.down_proj.bias"), ("ln1", "self_attn_layer_norm.weight"), ("ln2", "final_layer_norm.weight")):
            put(getattr(L, ours), p + theirs)
        L.w_gu.data.copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
    put(m.proj1, "multi_modal_projector.linear_1.weight")
    put(m.proj2, "multi_modal_projector.linear_2.weight")
    t = "language_model.model."
    put(m.embed, t + "embed_tokens.weight")
    put(m.norm, t + "norm.weight")
    if m.lm_head is not None:
        put(m.lm_head, "language_model.lm_head.weight")
    for i, L in enumerate(m.layers):
        p = f"{t}layers.{i}."
        L.w_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
        L.w_gu.data.copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
        for ours, theirs in (("w_o", "self_attn.o_proj.weight"), ("w_down", "mlp.down_proj.weight"), ("ln1", "input_layernorm.weight"),
                             ("ln2", "post_attention_layernorm.weight"), ("ada1", "ada_rms_norm.linear1.weight"), ("ada2", "ada_rms_norm.linear2.weight")):
            put(getattr(L, ours), p + theirs)

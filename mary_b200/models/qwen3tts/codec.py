"""The 12 Hz speech codec of Qwen3-TTS: decoder (codes -> 24 kHz waveform) and encoder (reference audio -> codes).

Reference: src/models/qwen3tts/codec.rs (decoder) and encoder.rs (encoder); dimensions from config.rs:44-62.

Decoder (codec.rs:283-466), fully causal: split residual-VQ lookup (1 semantic + 15 acoustic codebooks, each table =
``embedding_sum / clamp(cluster_usage, 1e-5)``, summed per bank, 1x1 ``output_proj``) -> causal conv 512->1024 k3 -> 8-layer
sliding-window (72) transformer at width 512 with LayerScale -> 2 x (transposed conv x2 + ConvNeXt block) -> SEANet-style stack
(conv k7, four SnakeBeta / transposed-conv / 3 dilated residual units blocks upsampling 8*5*4*3, SnakeBeta, conv k7 to 1 channel)
-> clamp to [-1, 1]; 1920 samples per frame.  ``chunked_decode`` walks 300-frame chunks with 25 frames of left context.

Encoder (encoder.rs:1-499): causal SEANet conv encoder (x960), 8-layer LayerNorm / GELU transformer with LayerScale at width 512,
stride-2 ``downsample`` conv with replicate padding (12.5 Hz), split residual-VQ ENCODE (nearest codebook row by
``|e|^2 - 2 <r, e>``, residual chain).

Activations are kept TIME-MAJOR ``[T, C]`` here, so every dense convolution is one row-major GEMM over ``k`` shifted copies of its
input and every transposed convolution one GEMM followed by an overlap-add: on the GPU these run on this package's tcgen05 GEMM
(``ops.linear``), the rest is elementwise.  The reference runs the same im2col form because its direct conv path measured 3 %
efficiency (codec.rs:36-40).  Parameters live in a dictionary under their CHECKPOINT names, so a loader fills them by name."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from ... import ops


@dataclass
class CodecConfig:
    num_code_groups: int = 16
    codebook_size: int = 2048
    code_dim: int = 256                      # per-quantiser embedding width
    quant_out: int = 512                     # after ``output_proj``
    latent: int = 1024
    hidden: int = 512                        # transformer width (decoder and encoder)
    tr_layers: int = 8
    tr_heads: int = 16
    tr_head_dim: int = 64
    tr_inter: int = 1024
    tr_window: int = 72
    tr_eps: float = 1e-5
    rope_theta: float = 10_000.0
    decoder_dim: int = 1536
    upsample_rates: list = field(default_factory=lambda: [8, 5, 4, 3])
    upsampling_ratios: list = field(default_factory=lambda: [2, 2])
    # encoder
    enc_stem: int = 64
    enc_ratios: list = field(default_factory=lambda: [4, 5, 6, 8])
    enc_heads: int = 8
    enc_head_dim: int = 64
    enc_layers: int = 8
    enc_inter: int = 2048
    enc_eps: float = 1e-5
    enc_acoustic_stored: int = 31            # the checkpoint holds 31 acoustic quantisers; 15 are used

    @property
    def samples_per_frame(self) -> int:
        return math.prod(self.upsample_rates) * math.prod(self.upsampling_ratios)

    @staticmethod
    def tiny() -> "CodecConfig":
        return CodecConfig(num_code_groups=4, codebook_size=32, code_dim=16, quant_out=32, latent=64, hidden=32, tr_layers=2, tr_heads=2,
                           tr_head_dim=16, tr_inter=64, tr_window=6, decoder_dim=64, upsample_rates=[3, 2], upsampling_ratios=[2],
                           enc_stem=8, enc_ratios=[2, 3], enc_heads=2, enc_head_dim=16, enc_layers=2, enc_inter=64, enc_acoustic_stored=5)


# --------------------------------------------------------------------------------------------------------------------------------
# building blocks on time-major activations x[T, C]
def _mm(x, w, b=None):
    """``x @ w^T (+ b)``: the package GEMM for bf16 on the GPU when the row pitch allows a TMA load, else a plain matmul."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0:
        return ops.linear(x.contiguous(), w, b)
    y = x @ w.t()
    return y if b is None else y + b


def shifted(x, k: int, dilation: int = 1):
    """``[T, k * C]``: copy ``j`` holds the rows ``(k - 1 - j) * dilation`` steps back, zeros before the start."""
    if k == 1:
        return x
    T, C = x.shape
    pad = (k - 1) * dilation
    xp = torch.cat([x.new_zeros(pad, C), x], 0)
    return torch.cat([xp[j * dilation:j * dilation + T] for j in range(k)], 1)


def conv_weight(w):
    """``[out, in, k]`` -> ``[out, k * in]`` in the order :func:`shifted` lays the copies out."""
    o, i, k = w.shape
    return w.permute(0, 2, 1).reshape(o, k * i).contiguous()


def causal_conv(x, w2, b, k: int, dilation: int = 1):
    """Causal convolution, stride 1: left padding ``(k - 1) * dilation`` (codec.rs:70-99); ``w2 = conv_weight(w)``."""
    return _mm(shifted(x, k, dilation), w2, b)


def depthwise_causal_conv(x, w, b):
    """``groups = C`` causal convolution; ``w [C, 1, k]``.  A handful of fused multiply-adds per element: no GEMM."""
    T, C = x.shape
    k = w.shape[-1]
    xp = torch.cat([x.new_zeros(k - 1, C), x], 0).float()
    acc = b.float().expand(T, C).clone()
    for j in range(k):
        acc = acc + xp[j:j + T] * w[:, 0, j].float()
    return acc.to(x.dtype)


def transconv_weight(w):
    """``[in, out, k]`` -> ``[k * out, in]``."""
    i, o, k = w.shape
    return w.permute(2, 1, 0).reshape(k * o, i).contiguous()


def causal_transconv(x, w2, b, out_ch: int, k: int, stride: int):
    """Causal transposed convolution with ``k = m * stride``, ``m`` in {1, 2}: one GEMM ``[T, k * out]``, overlap-add of the
    stride blocks and interleave; the causal right trim ``k - stride`` drops the dangling tail (codec.rs:101-156):
    ``out[t * s + j] = z[t, j] + z[t - 1, j + s]``."""
    if k % stride or k // stride > 2:
        raise ValueError(f"transposed conv with k={k}, stride={stride} is outside the codec's forms")
    T = x.shape[0]
    z = _mm(x, w2).view(T, k, out_ch)
    acc = z[:, :stride]
    if k == 2 * stride:
        acc = acc + torch.cat([z.new_zeros(1, stride, out_ch), z[:-1, stride:]], 0)
    out = acc.reshape(T * stride, out_ch)
    return (out.float() + b.float()).to(x.dtype)


def snake_beta(x, alpha, beta):
    """``x + sin^2(x e^alpha) / (e^beta + 1e-9)`` per channel (codec.rs:158-179)."""
    xf = x.float()
    return (xf + torch.sin(xf * alpha.float().exp()).square() / (beta.float().exp() + 1e-9)).to(x.dtype)


def rope_half(x, pos, theta: float):
    """Split-half rotary embedding of ``x [T, H, D]`` at positions ``pos [T]``."""
    D = x.shape[-1]
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = pos.float()[:, None] * inv[None]
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    a, b = x.float()[..., :D // 2], x.float()[..., D // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)


def windowed_attention(q, k, v, window: int | None):
    """Causal attention of one stream; ``q, k, v [T, H, D]`` (already rotated); key ``j`` is visible to row ``i`` iff ``j <= i`` and
    ``i - j < window`` (layers.rs:398-417).  A few hundred rows at most per chunk: plain f32 arithmetic."""
    T, H, D = q.shape
    s = torch.einsum("thd,shd->hts", q.float(), k.float()) * D ** -0.5
    i = torch.arange(T, device=q.device)
    blocked = i[None, :] > i[:, None]
    if window is not None:
        blocked = blocked | (i[:, None] - i[None, :] >= window)
    s = s.masked_fill(blocked[None], float("-inf"))
    return torch.einsum("hts,shd->thd", torch.softmax(s, -1), v.float()).to(q.dtype)


def rms(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype) if w is not None else y.to(x.dtype)


class _Params:
    """Name -> tensor store with the declared shapes; derived (re-laid-out) weights are cached and dropped on ``set_tensor``."""

    def __init__(self, dtype, device):
        self.dtype, self.dev = dtype, torch.device(device)
        self.P: dict[str, torch.Tensor] = {}
        self.shapes: dict[str, tuple] = {}
        self._derived: dict = {}

    def declare(self, name: str, *shape):
        self.shapes[name] = tuple(shape)

    def expected(self) -> list[tuple[str, tuple]]:
        return sorted(self.shapes.items())

    def set_tensor(self, name: str, value) -> None:
        if name not in self.shapes:
            raise KeyError(f"codec has no tensor named {name!r}")
        if tuple(value.shape) != self.shapes[name]:
            raise ValueError(f"{name}: shape {tuple(value.shape)} != declared {self.shapes[name]}")
        keep_f32 = name.endswith(("cluster_usage", "embedding_sum", "embed_sum"))
        self.P[name] = value.to(self.dev, torch.float32 if keep_f32 else self.dtype)
        self._derived.clear()

    def load_from(self, loader) -> None:
        for name in self.shapes:
            self.set_tensor(name, loader.load_tensor(name, torch.float32))

    def missing(self) -> list[str]:
        return [n for n in self.shapes if n not in self.P]

    def init_random_(self, seed: int = 0, std: float = 0.05):
        g = torch.Generator().manual_seed(seed)
        for name, shape in self.expected():
            last = name.rsplit(".", 1)[-1]
            if name.endswith("cluster_usage"):
                v = torch.rand(shape, generator=g) + 0.5
            elif last in ("alpha", "beta"):
                v = torch.randn(shape, generator=g) * 0.1
            elif last in ("gamma", "scale"):
                v = torch.full(shape, 0.5)
            elif name.endswith(("norm.weight", "layernorm.weight")):
                v = torch.ones(shape) + torch.randn(shape, generator=g) * 0.02
            elif last == "bias":
                v = torch.randn(shape, generator=g) * 0.01
            else:
                fan_in = max(math.prod(shape[1:]), 1) if len(shape) > 1 else 1
                v = torch.randn(shape, generator=g) * (std if len(shape) == 1 else 1.0 / math.sqrt(fan_in))
            self.set_tensor(name, v)
        return self

    def d(self, key, make):
        if key not in self._derived:
            self._derived[key] = make()
        return self._derived[key]

    def conv(self, x, prefix: str, dilation: int = 1):
        w = self.P[prefix + ".weight"]
        w2 = self.d(prefix, lambda: conv_weight(w))
        return causal_conv(x, w2, self.P.get(prefix + ".bias"), w.shape[-1], dilation)

    def snake(self, x, prefix: str):
        return snake_beta(x, self.P[prefix + ".alpha"], self.P[prefix + ".beta"])


# --------------------------------------------------------------------------------------------------------------------------------
class CodecDecoder(_Params):
    """``codes [T, 16]`` -> waveform ``[T * 1920]`` in [-1, 1] (codec.rs:283-466)."""

    def __init__(self, cfg: CodecConfig | None = None, dtype=torch.float32, device="cpu"):
        super().__init__(dtype, device)
        c = self.cfg = cfg or CodecConfig()
        for bank, n in (("rvq_first", 1), ("rvq_rest", c.num_code_groups - 1)):
            for i in range(n):
                self.declare(f"decoder.quantizer.{bank}.vq.layers.{i}._codebook.embedding_sum", c.codebook_size, c.code_dim)
                self.declare(f"decoder.quantizer.{bank}.vq.layers.{i}._codebook.cluster_usage", c.codebook_size)
            self.declare(f"decoder.quantizer.{bank}.output_proj.weight", c.quant_out, c.code_dim, 1)
        self.declare("decoder.pre_conv.conv.weight", c.latent, c.quant_out, 3)
        self.declare("decoder.pre_conv.conv.bias", c.latent)
        t = "decoder.pre_transformer"
        self.declare(f"{t}.input_proj.weight", c.hidden, c.latent)
        self.declare(f"{t}.input_proj.bias", c.hidden)
        hd = c.tr_heads * c.tr_head_dim
        for i in range(c.tr_layers):
            p = f"{t}.layers.{i}"
            self.declare(f"{p}.input_layernorm.weight", c.hidden)
            self.declare(f"{p}.post_attention_layernorm.weight", c.hidden)
            for n in "qkv":
                self.declare(f"{p}.self_attn.{n}_proj.weight", hd, c.hidden)
            self.declare(f"{p}.self_attn.o_proj.weight", c.hidden, hd)
            self.declare(f"{p}.self_attn_layer_scale.scale", c.hidden)
            self.declare(f"{p}.mlp.gate_proj.weight", c.tr_inter, c.hidden)
            self.declare(f"{p}.mlp.up_proj.weight", c.tr_inter, c.hidden)
            self.declare(f"{p}.mlp.down_proj.weight", c.hidden, c.tr_inter)
            self.declare(f"{p}.mlp_layer_scale.scale", c.hidden)
        self.declare(f"{t}.norm.weight", c.hidden)
        self.declare(f"{t}.output_proj.weight", c.latent, c.hidden)
        self.declare(f"{t}.output_proj.bias", c.latent)
        for i, r in enumerate(c.upsampling_ratios):
            u = f"decoder.upsample.{i}"
            self.declare(f"{u}.0.conv.weight", c.latent, c.latent, r)
            self.declare(f"{u}.0.conv.bias", c.latent)
            self.declare(f"{u}.1.dwconv.conv.weight", c.latent, 1, 7)
            self.declare(f"{u}.1.dwconv.conv.bias", c.latent)
            self.declare(f"{u}.1.norm.weight", c.latent)
            self.declare(f"{u}.1.norm.bias", c.latent)
            self.declare(f"{u}.1.pwconv1.weight", 4 * c.latent, c.latent)
            self.declare(f"{u}.1.pwconv1.bias", 4 * c.latent)
            self.declare(f"{u}.1.pwconv2.weight", c.latent, 4 * c.latent)
            self.declare(f"{u}.1.pwconv2.bias", c.latent)
            self.declare(f"{u}.1.gamma", c.latent)
        self.declare("decoder.decoder.0.conv.weight", c.decoder_dim, c.latent, 7)
        self.declare("decoder.decoder.0.conv.bias", c.decoder_dim)
        dim = c.decoder_dim
        for i, r in enumerate(c.upsample_rates):
            b = f"decoder.decoder.{i + 1}.block"
            self.declare(f"{b}.0.alpha", dim)
            self.declare(f"{b}.0.beta", dim)
            self.declare(f"{b}.1.conv.weight", dim, dim // 2, 2 * r)
            self.declare(f"{b}.1.conv.bias", dim // 2)
            dim //= 2
            for u in (2, 3, 4):
                for a in ("act1", "act2"):
                    self.declare(f"{b}.{u}.{a}.alpha", dim)
                    self.declare(f"{b}.{u}.{a}.beta", dim)
                self.declare(f"{b}.{u}.conv1.conv.weight", dim, dim, 7)
                self.declare(f"{b}.{u}.conv1.conv.bias", dim)
                self.declare(f"{b}.{u}.conv2.conv.weight", dim, dim, 1)
                self.declare(f"{b}.{u}.conv2.conv.bias", dim)
        n = len(c.upsample_rates)
        self.declare(f"decoder.decoder.{n + 1}.alpha", dim)
        self.declare(f"decoder.decoder.{n + 1}.beta", dim)
        self.declare(f"decoder.decoder.{n + 2}.conv.weight", 1, dim, 7)
        self.declare(f"decoder.decoder.{n + 2}.conv.bias", 1)

    # ------------------------------------------------------------------ stages
    def _bank(self, bank: str, codes):
        """One residual-VQ bank: the tables' rows summed, then the 1x1 output projection (codec.rs:236-281)."""
        acc = None
        for i in range(codes.shape[1]):
            p = f"decoder.quantizer.{bank}.vq.layers.{i}._codebook."
            table = self.d(p, lambda p=p: self.P[p + "embedding_sum"] / self.P[p + "cluster_usage"].clamp_min(1e-5)[:, None])
            e = table[codes[:, i].long()]
            acc = e if acc is None else acc + e
        w = self.P[f"decoder.quantizer.{bank}.output_proj.weight"]
        return _mm(acc.to(self.dtype), w[:, :, 0].contiguous())

    def quantizer_decode(self, codes):
        """``codes [T, groups]`` -> ``[T, quant_out]``: semantic bank (codebook 0) plus acoustic bank (the rest)."""
        return (self._bank("rvq_first", codes[:, :1]).float() + self._bank("rvq_rest", codes[:, 1:]).float()).to(self.dtype)

    def _transformer(self, h):
        c, t = self.cfg, "decoder.pre_transformer"
        x = _mm(h, self.P[f"{t}.input_proj.weight"], self.P[f"{t}.input_proj.bias"])
        T = x.shape[0]
        pos = torch.arange(T, device=x.device)
        for i in range(c.tr_layers):
            p = f"{t}.layers.{i}"
            wqkv = self.d(p + ".qkv", lambda p=p: torch.cat([self.P[f"{p}.self_attn.{n}_proj.weight"] for n in "qkv"], 0).contiguous())
            wgu = self.d(p + ".gu", lambda p=p: torch.cat([self.P[f"{p}.mlp.gate_proj.weight"], self.P[f"{p}.mlp.up_proj.weight"]], 0).contiguous())
            y = rms(x, self.P[f"{p}.input_layernorm.weight"], c.tr_eps)
            q, k, v = _mm(y, wqkv).view(T, 3, c.tr_heads, c.tr_head_dim).unbind(1)
            a = windowed_attention(rope_half(q, pos, c.rope_theta), rope_half(k, pos, c.rope_theta), v, c.tr_window)
            a = _mm(a.reshape(T, -1), self.P[f"{p}.self_attn.o_proj.weight"])
            x = (x.float() + a.float() * self.P[f"{p}.self_attn_layer_scale.scale"].float()).to(x.dtype)
            y = rms(x, self.P[f"{p}.post_attention_layernorm.weight"], c.tr_eps)
            g, u = _mm(y, wgu).float().chunk(2, -1)
            m = _mm((F.silu(g) * u).to(x.dtype), self.P[f"{p}.mlp.down_proj.weight"])
            x = (x.float() + m.float() * self.P[f"{p}.mlp_layer_scale.scale"].float()).to(x.dtype)
        y = rms(x, self.P[f"{t}.norm.weight"], c.tr_eps)
        return _mm(y, self.P[f"{t}.output_proj.weight"], self.P[f"{t}.output_proj.bias"])

    def _convnext(self, x, p: str):
        """causal depthwise k7 -> LayerNorm (eps 1e-6) -> 4x pointwise, GELU, pointwise -> gamma -> residual (codec.rs:181-234)."""
        h = depthwise_causal_conv(x, self.P[f"{p}.dwconv.conv.weight"], self.P[f"{p}.dwconv.conv.bias"])
        h = F.layer_norm(h.float(), (h.shape[-1],), self.P[f"{p}.norm.weight"].float(), self.P[f"{p}.norm.bias"].float(), 1e-6).to(x.dtype)
        h = _mm(h, self.P[f"{p}.pwconv1.weight"], self.P[f"{p}.pwconv1.bias"])
        h = _mm(F.gelu(h.float()).to(x.dtype), self.P[f"{p}.pwconv2.weight"], self.P[f"{p}.pwconv2.bias"])
        return (x.float() + h.float() * self.P[f"{p}.gamma"].float()).to(x.dtype)

    def _transconv(self, x, prefix: str, stride: int):
        w = self.P[prefix + ".weight"]
        return causal_transconv(x, self.d(prefix, lambda: transconv_weight(w)), self.P[prefix + ".bias"], w.shape[1], w.shape[2], stride)

    @torch.no_grad()
    def decode(self, codes) -> torch.Tensor:
        """Whole-sequence decode of ``codes [T, groups]`` (any integer tensor / array) -> f32 waveform ``[T * samples_per_frame]``."""
        c = self.cfg
        codes = torch.as_tensor(codes, device=self.dev).long()
        if codes.dim() != 2 or codes.shape[1] != c.num_code_groups or codes.shape[0] == 0:
            raise ValueError(f"codes must be [T > 0, {c.num_code_groups}], got {tuple(codes.shape)}")
        if int(codes.min()) < 0 or int(codes.max()) >= c.codebook_size:
            raise ValueError("code outside the codebook")
        h = self.conv(self.quantizer_decode(codes), "decoder.pre_conv.conv")
        h = self._transformer(h)
        for i, r in enumerate(c.upsampling_ratios):
            h = self._convnext(self._transconv(h, f"decoder.upsample.{i}.0.conv", r), f"decoder.upsample.{i}.1")
        w = self.conv(h, "decoder.decoder.0.conv")
        for i, r in enumerate(c.upsample_rates):
            b = f"decoder.decoder.{i + 1}.block"
            w = self._transconv(self.snake(w, f"{b}.0"), f"{b}.1.conv", r)
            for u, dil in ((2, 1), (3, 3), (4, 9)):
                res = w
                w = self.conv(self.snake(w, f"{b}.{u}.act1"), f"{b}.{u}.conv1.conv", dil)
                w = self.conv(self.snake(w, f"{b}.{u}.act2"), f"{b}.{u}.conv2.conv")
                w = (w.float() + res.float()).to(w.dtype)
        n = len(c.upsample_rates)
        w = self.conv(self.snake(w, f"decoder.decoder.{n + 1}"), f"decoder.decoder.{n + 2}.conv")
        return w.float().clamp(-1.0, 1.0).reshape(-1)

    def chunked_decode(self, codes, chunk: int = 300, context: int = 25) -> torch.Tensor:
        """Long sequences in ``chunk``-frame pieces, each decoded with ``context`` earlier frames whose samples are dropped
        (codec.rs:451-465)."""
        codes = torch.as_tensor(codes)
        spf, out, start = self.cfg.samples_per_frame, [], 0
        while start < codes.shape[0]:
            end = min(start + chunk, codes.shape[0])
            c = min(context, start)
            out.append(self.decode(codes[start - c:end])[c * spf:])
            start = end
        return torch.cat(out)


# --------------------------------------------------------------------------------------------------------------------------------
def strided_causal_conv(x, w, b, stride: int, replicate: bool = False):
    """The encoder's convolution on ``x [T, C]``: left padding ``k - stride``, right padding up to a whole number of output frames
    (zeros, or the edge values for the ``downsample`` conv), then one GEMM over the gathered windows (encoder.rs:44-118)."""
    T, C = x.shape
    o, i, k = w.shape
    pad_left = k - stride
    n_frames = max(math.ceil((T + pad_left - k) / stride + 1) - 1, 0)
    pad_right = max(n_frames * stride + k - pad_left - T, 0)
    if replicate:
        xp = torch.cat([x[:1].expand(pad_left, C), x, x[-1:].expand(pad_right, C)], 0)
    else:
        xp = torch.cat([x.new_zeros(pad_left, C), x, x.new_zeros(pad_right, C)], 0)
    n_out = (xp.shape[0] - k) // stride + 1
    win = xp.unfold(0, k, stride)                                  # [n_out, C, k]
    cols = win.permute(0, 2, 1).reshape(n_out, k * C)             # copy j-major, as conv_weight lays the weight out
    return _mm(cols.contiguous(), conv_weight(w), b)


def rvq_encode(residual, codebooks):
    """Residual-VQ encode: per quantiser the nearest row by ``|e|^2 - 2 <r, e>`` (first minimum), then ``r -= e``
    (encoder.rs:189-232).  ``residual [T, D]`` f32; returns ``codes [T, n_q]``."""
    r = residual.float().clone()
    out = []
    for cb in codebooks:
        cb = cb.float()
        dist = cb.square().sum(-1)[None] - 2.0 * (r @ cb.t())
        m = dist.min(-1, keepdim=True).values
        idx = torch.where(dist == m, torch.arange(cb.shape[0], device=r.device)[None], cb.shape[0]).min(-1).values
        out.append(idx)
        r = r - cb[idx]
    return torch.stack(out, 1)


class CodecEncoder(_Params):
    """Waveform ``[N]`` at 24 kHz -> ``codes [ceil(N / 1920), 16]`` (encoder.rs:234-499).  Runs in f32: encoding happens once per
    reference clip, so determinism counts for more than throughput (encoder.rs:23-25)."""

    def __init__(self, cfg: CodecConfig | None = None, dtype=torch.float32, device="cpu"):
        super().__init__(dtype, device)
        c = self.cfg = cfg or CodecConfig()
        p = "encoder.encoder.layers"
        self.declare(f"{p}.0.conv.weight", c.enc_stem, 1, 7)
        self.declare(f"{p}.0.conv.bias", c.enc_stem)
        dim = c.enc_stem
        for i, r in enumerate(c.enc_ratios):
            self.declare(f"{p}.{3 * i + 1}.block.1.conv.weight", dim // 2, dim, 3)
            self.declare(f"{p}.{3 * i + 1}.block.1.conv.bias", dim // 2)
            self.declare(f"{p}.{3 * i + 1}.block.3.conv.weight", dim, dim // 2, 1)
            self.declare(f"{p}.{3 * i + 1}.block.3.conv.bias", dim)
            self.declare(f"{p}.{3 * i + 3}.conv.weight", 2 * dim, dim, 2 * r)
            self.declare(f"{p}.{3 * i + 3}.conv.bias", 2 * dim)
            dim *= 2
        self.final_index = 3 * len(c.enc_ratios) + 2
        self.declare(f"{p}.{self.final_index}.conv.weight", c.hidden, dim, 3)
        self.declare(f"{p}.{self.final_index}.conv.bias", c.hidden)
        hd = c.enc_heads * c.enc_head_dim
        for i in range(c.enc_layers):
            t = f"encoder.encoder_transformer.layers.{i}"
            for n in ("input_layernorm", "post_attention_layernorm"):
                self.declare(f"{t}.{n}.weight", c.hidden)
                self.declare(f"{t}.{n}.bias", c.hidden)
            for n in "qkv":
                self.declare(f"{t}.self_attn.{n}_proj.weight", hd, c.hidden)
            self.declare(f"{t}.self_attn.o_proj.weight", c.hidden, hd)
            self.declare(f"{t}.mlp.fc1.weight", c.enc_inter, c.hidden)
            self.declare(f"{t}.mlp.fc2.weight", c.hidden, c.enc_inter)
            self.declare(f"{t}.self_attn_layer_scale.scale", c.hidden)
            self.declare(f"{t}.mlp_layer_scale.scale", c.hidden)
        self.declare("encoder.downsample.conv.weight", c.hidden, c.hidden, 4)
        for bank, n in (("semantic", 1), ("acoustic", c.enc_acoustic_stored)):
            q = f"encoder.quantizer.{bank}_residual_vector_quantizer"
            self.declare(f"{q}.input_proj.weight", c.code_dim, c.hidden, 1)
            for i in range(n):
                self.declare(f"{q}.layers.{i}.codebook.embed_sum", c.codebook_size, c.code_dim)
                self.declare(f"{q}.layers.{i}.codebook.cluster_usage", c.codebook_size)

    def _sconv(self, x, prefix: str, stride: int = 1, replicate: bool = False):
        return strided_causal_conv(x, self.P[prefix + ".weight"], self.P.get(prefix + ".bias"), stride, replicate)

    def _transformer(self, h):
        """LayerNorm (biased) / full causal attention / GELU MLP, LayerScale on both branches (encoder.rs:330-425).  The
        checkpoint's config names a sliding window of 250, but the path the reference follows never applies it."""
        c = self.cfg
        T = h.shape[0]
        pos = torch.arange(T, device=h.device)
        for i in range(c.enc_layers):
            t = f"encoder.encoder_transformer.layers.{i}"
            y = F.layer_norm(h, (c.hidden,), self.P[f"{t}.input_layernorm.weight"], self.P[f"{t}.input_layernorm.bias"], c.enc_eps)
            q, k, v = ((y @ self.P[f"{t}.self_attn.{n}_proj.weight"].t()).view(T, c.enc_heads, c.enc_head_dim) for n in "qkv")
            a = windowed_attention(rope_half(q, pos, c.rope_theta), rope_half(k, pos, c.rope_theta), v, None)
            h = h + (a.reshape(T, -1) @ self.P[f"{t}.self_attn.o_proj.weight"].t()) * self.P[f"{t}.self_attn_layer_scale.scale"]
            y = F.layer_norm(h, (c.hidden,), self.P[f"{t}.post_attention_layernorm.weight"], self.P[f"{t}.post_attention_layernorm.bias"], c.enc_eps)
            m = F.gelu(y @ self.P[f"{t}.mlp.fc1.weight"].t()) @ self.P[f"{t}.mlp.fc2.weight"].t()
            h = h + m * self.P[f"{t}.mlp_layer_scale.scale"]
        return h

    def _codebooks(self, bank: str, n: int):
        q = f"encoder.quantizer.{bank}_residual_vector_quantizer.layers"
        return self.d(("cb", bank, n), lambda: [self.P[f"{q}.{i}.codebook.embed_sum"] / self.P[f"{q}.{i}.codebook.cluster_usage"].clamp_min(1e-5)[:, None]
                                               for i in range(n)])

    @torch.no_grad()
    def encode(self, samples) -> torch.Tensor:
        c, p = self.cfg, "encoder.encoder.layers"
        x = torch.as_tensor(samples, dtype=torch.float32, device=self.dev).reshape(-1, 1)
        n_samples = x.shape[0]
        if n_samples == 0:
            raise ValueError("empty waveform")
        x = self._sconv(x, f"{p}.0.conv")
        for i, r in enumerate(c.enc_ratios):
            h = self._sconv(F.elu(x), f"{p}.{3 * i + 1}.block.1.conv")
            x = x + self._sconv(F.elu(h), f"{p}.{3 * i + 1}.block.3.conv")
            x = self._sconv(F.elu(x), f"{p}.{3 * i + 3}.conv", r)
        x = self._sconv(F.elu(x), f"{p}.{self.final_index}.conv")
        x = self._transformer(x)
        emb = self._sconv(x, "encoder.downsample.conv", 2, replicate=True)
        codes = []
        for bank, n in (("semantic", 1), ("acoustic", c.num_code_groups - 1)):
            w = self.P[f"encoder.quantizer.{bank}_residual_vector_quantizer.input_proj.weight"][:, :, 0]
            codes.append(rvq_encode(emb @ w.t(), self._codebooks(bank, n)))
        codes = torch.cat(codes, 1)
        frames = min(-(-n_samples // c.samples_per_frame), codes.shape[0])
        return codes[:frames]

"""Gemma-4 vision tower: image patches -> soft tokens in the decoder's embedding space (src/models/gemma/gemma4/vision.rs and the
vision loader, weights.rs:230-386).

One image is a ragged list of ``patch x patch`` pixel patches (values in [0, 1]) with their (x, y) grid coordinates — any
aspect ratio, no padding rows here.  A patch is scaled to [-1, 1], projected by one GEMM and given the sum of two learned
position embeddings (one table per axis).  The blocks are the text decoder's block (sandwich RMSNorms, learned q / k norm,
weightless v norm, attention scale 1.0, GeGLU) with bidirectional attention and a 2-D rotary code: the first half of every
head rotates with the x coordinate, the second half with y, each over its own full frequency range.  The pooler averages every
``k x k`` patch neighbourhood into one soft token and multiplies by ``sqrt(hidden)``; the multimodal embedder applies a weightless
RMSNorm and projects to the decoder's width.  Checkpoints of the larger towers clamp the input and output of every linear
("clipped linears"); the bounds are loaded when present."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


@dataclass
class Gemma4VisionConfig:
    hidden: int = 768
    layers: int = 16
    heads: int = 12
    kv_heads: int = 12
    head_dim: int = 64
    ffn: int = 3072
    patch: int = 16
    pos_size: int = 10240
    pool: int = 3
    theta: float = 100.0
    eps: float = 1e-6
    standardize: bool = False
    text_hidden: int = 2304

    @staticmethod
    def tiny():
        return Gemma4VisionConfig(hidden=32, layers=2, heads=4, kv_heads=2, head_dim=8, ffn=48, patch=4, pos_size=32, pool=2, text_hidden=24)


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


class ClipLinear(nn.Module):
    """``clamp(clamp(x, in_lo, in_hi) W^T, out_lo, out_hi)``; the bounds default to +-inf (no clamp)."""

    def __init__(self, n_out, n_in):
        super().__init__()
        self.w = _P(n_out, n_in)
        self.register_buffer("bounds", torch.tensor([-float("inf"), float("inf"), -float("inf"), float("inf")]))
        self.clipped = False

    def forward(self, x):
        if not self.clipped:
            return ops.linear(x, self.w)
        b = self.bounds.tolist()
        return ops.linear(x.clamp(b[0], b[1]), self.w).clamp(b[2], b[3])


class VisionLayer(nn.Module):
    def __init__(self, c: Gemma4VisionConfig):
        super().__init__()
        H, D = c.hidden, c.head_dim
        self.q, self.k, self.v, self.o = ClipLinear(c.heads * D, H), ClipLinear(c.kv_heads * D, H), ClipLinear(c.kv_heads * D, H), ClipLinear(H, c.heads * D)
        self.gate, self.up, self.down = ClipLinear(c.ffn, H), ClipLinear(c.ffn, H), ClipLinear(H, c.ffn)
        self.q_norm, self.k_norm = _P(D), _P(D)
        self.ln_in, self.ln_post_attn, self.ln_pre_ffn, self.ln_post_ffn = _P(H), _P(H), _P(H), _P(H)


def rope_2d(x, pos, inv_freq):
    """``x [N, heads, D]``; the first ``D / 2`` channels rotate (split-half) with ``pos[:, 0]``, the rest with ``pos[:, 1]``."""
    half = x.shape[-1] // 2
    out = []
    for axis in range(2):
        part = x[..., axis * half:(axis + 1) * half]
        ang = pos[:, axis, None].float() * inv_freq
        cos, sin = ang.cos()[:, None, :].to(x.dtype), ang.sin()[:, None, :].to(x.dtype)
        a, b = part[..., :half // 2], part[..., half // 2:]
        out.append(torch.cat([a * cos - b * sin, b * cos + a * sin], -1))
    return torch.cat(out, -1)


class Gemma4VisionTower(nn.Module):
    def __init__(self, c: Gemma4VisionConfig):
        super().__init__()
        self.c = c
        self.input_proj, self.pos_table = _P(c.hidden, 3 * c.patch * c.patch), _P(2, c.pos_size, c.hidden)
        self.layers = nn.ModuleList([VisionLayer(c) for _ in range(c.layers)])
        if c.standardize:
            self.std_bias, self.std_scale = _P(c.hidden), _P(c.hidden)
        self.embed_proj = _P(c.text_hidden, c.hidden)
        sd = c.head_dim // 2
        self.register_buffer("inv_freq", 1.0 / (c.theta ** (torch.arange(0, sd, 2, dtype=torch.float32) / sd)), persistent=False)

    def encode(self, patches, pos):
        """``patches [N, 3 p p]`` in [0, 1], ``pos [N, 2]`` (x, y) -> ``[N, hidden]``."""
        c = self.c
        N, D = patches.shape[0], c.head_dim
        x = ops.linear((2.0 * (patches - 0.5)).to(self.input_proj.dtype), self.input_proj) + self.pos_table[0][pos[:, 0]] + self.pos_table[1][pos[:, 1]]
        for L in self.layers:
            h = ops.rmsnorm(x, L.ln_in, c.eps)
            q = ops.rmsnorm(L.q(h).view(N, c.heads, D), L.q_norm, c.eps)
            k = ops.rmsnorm(L.k(h).view(N, c.kv_heads, D), L.k_norm, c.eps)
            v = ops.rmsnorm(L.v(h).view(N, c.kv_heads, D), None, c.eps)
            q, k = rope_2d(q, pos, self.inv_freq), rope_2d(k, pos, self.inv_freq)
            a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], scale=1.0,
                                               enable_gqa=True)[0].transpose(0, 1).reshape(N, c.heads * D)
            x = x + ops.rmsnorm(L.o(a), L.ln_post_attn, c.eps)
            h = ops.rmsnorm(x, L.ln_pre_ffn, c.eps)
            m = L.down(ops.glu(torch.cat([L.gate(h), L.up(h)], -1), "geglu"))
            x = x + ops.rmsnorm(m, L.ln_post_ffn, c.eps)
        return x

    def pool(self, x, pos):
        """Average every ``pool x pool`` neighbourhood (by coordinates) and scale by ``sqrt(hidden)`` -> ``[N / pool^2, hidden]``, row-major
        over the pooled grid."""
        c = self.c
        k = c.pool
        wx = int(pos[:, 0].max()) + 1
        cell = (pos[:, 0] // k + (wx // k) * (pos[:, 1] // k)).long()
        n_out = x.shape[0] // (k * k)
        out = torch.zeros(n_out, x.shape[1], dtype=torch.float32, device=x.device).index_add_(0, cell, x.float()) / (k * k)
        y = (out * c.hidden ** 0.5).to(x.dtype)
        return (y - self.std_bias) * self.std_scale if c.standardize else y

    def forward(self, patches, pos):
        """Soft tokens of one image, already in the decoder's width (they replace the image placeholder rows of the prompt)."""
        y = self.pool(self.encode(patches, pos), pos)
        return ops.linear(ops.rmsnorm(y, None, self.c.eps), self.embed_proj)


def patchify(image, patch: int):
    """``image [3, H, W]`` (H, W multiples of ``patch``) -> ``(patches [N, 3 p p], pos [N, 2])`` in row-major order; a patch is
    flattened (row, column, channel) like the checkpoint's input projection expects."""
    C, H, W = image.shape
    gh, gw = H // patch, W // patch
    p = image.reshape(C, gh, patch, gw, patch).permute(1, 3, 2, 4, 0).reshape(gh * gw, patch * patch * C)
    ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    return p, torch.stack([xs.reshape(-1), ys.reshape(-1)], -1)


def load_into(m: Gemma4VisionTower, loader, prefix: str = "model.vision_tower.", embed_prefix: str = "model.embed_vision.") -> None:
    """Names of the Hugging Face ``Gemma4ForConditionalGeneration`` layout (``vision_tower.*`` and ``embed_vision.*``)."""
    dt = m.input_proj.dtype

    def get(n):
        return loader.load_tensor(n, dt)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    put(m.input_proj, prefix + "patch_embedder.input_proj.weight")
    put(m.pos_table, prefix + "patch_embedder.position_embedding_table")
    if m.c.standardize:
        put(m.std_bias, prefix + "std_bias")
        put(m.std_scale, prefix + "std_scale")
    put(m.embed_proj, embed_prefix + "embedding_projection.weight")
    for i, L in enumerate(m.layers):
        p = f"{prefix}encoder.layers.{i}."
        for lin, name in ((L.q, "self_attn.q_proj"), (L.k, "self_attn.k_proj"), (L.v, "self_attn.v_proj"), (L.o, "self_attn.o_proj"),
                          (L.gate, "mlp.gate_proj"), (L.up, "mlp.up_proj"), (L.down, "mlp.down_proj")):
            put(lin.w, p + name + ".linear.weight")
            if loader.has_weight(p + name + ".input_min"):
                lin.bounds.copy_(torch.stack([get(p + name + "." + b).float().reshape(()) for b in ("input_min", "input_max", "output_min", "output_max")]))
                lin.clipped = bool(torch.isfinite(lin.bounds).any())
        for ours, theirs in (("q_norm", "self_attn.q_norm"), ("k_norm", "self_attn.k_norm"), ("ln_in", "input_layernorm"),
                             ("ln_post_attn", "post_attention_layernorm"), ("ln_pre_ffn", "pre_feedforward_layernorm"),
                             ("ln_post_ffn", "post_feedforward_layernorm")):
            put(getattr(L, ours), p + theirs + ".weight")

"""FLUX.2 diffusion transformer (src/models/flux/transformer/*): double-stream blocks (image and text keep separate weights
and meet in one joint attention), single-stream blocks (attention and SwiGLU MLP computed in parallel from one fused
projection), modulation shared by all blocks of a kind.

The flow time (x 1000, sinusoid of 256, two-layer SiLU MLP, plus a guidance code in the guidance-distilled variant) is turned
ONCE per step into shift / scale / gate triples by three shared modulation layers (image double-stream x 2 sets, text
double-stream x 2 sets, single-stream x 1 set); blocks hold no modulation weights.  Every branch is
``x + gate * f(layer_norm(x) * (1 + scale) + shift)`` with an affine-free LayerNorm.  Queries and keys get a per-head RMSNorm
and a 4-axis rotary code: the head dim is split into ``axes_dims_rope`` slices and slice ``a`` rotates consecutive pairs by
``ids[:, a] * theta^(-2i / d_a)`` (ids = (t, h, w, l): text tokens differ in ``l``, image tokens in ``h, w``).  No biases anywhere.
Text tokens are concatenated in front of image tokens for attention and for the single-stream part, and dropped before the
output AdaLN + projection."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


@dataclass
class Flux2Config:
    # FLUX.2-klein-4B
    heads: int = 24
    head_dim: int = 128
    layers: int = 5
    single_layers: int = 20
    joint_dim: int = 7680
    in_channels: int = 128
    mlp_ratio: float = 3.0
    guidance_embeds: bool = False
    rope_theta: float = 2000.0
    axes_dims: tuple = (32, 32, 32, 32)
    time_channels: int = 256
    eps: float = 1e-6

    @property
    def dim(self):
        return self.heads * self.head_dim

    @property
    def mlp(self):
        return int(self.dim * self.mlp_ratio)

    @staticmethod
    def tiny(guidance=False):
        return Flux2Config(heads=2, head_dim=16, layers=2, single_layers=2, joint_dim=24, in_channels=8, mlp_ratio=2.0,
                           guidance_embeds=guidance, axes_dims=(4, 4, 4, 4), time_channels=16)


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


def sinusoid(t, dim: int):
    """``[B] -> [B, dim]`` as ``[cos, sin]`` of ``t * 10000^(-i / half)`` (the timestep projection of the checkpoint)."""
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    a = t.float()[:, None] * f
    return torch.cat([a.cos(), a.sin()], -1)


def rope_angles(ids, axes_dims, theta):
    """``ids [S, n_axes]`` -> angles ``[S, sum(axes_dims) / 2]``."""
    out = []
    for a, d in enumerate(axes_dims):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        out.append(ids[:, a].double()[:, None] * inv)
    return torch.cat(out, -1).float()


def rope_pairs(x, ang):
    """Rotate consecutive pairs of ``x [S, heads, D]`` by ``ang [S, D / 2]``."""
    cos, sin = ang.cos()[:, None, :].to(x.dtype), ang.sin()[:, None, :].to(x.dtype)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)


def _ln(x):
    return F.layer_norm(x, (x.shape[-1],), None, None, 1e-6)


def _attn(q, k, v):
    o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None])
    return o[0].transpose(0, 1).reshape(q.shape[0], -1)


class DoubleBlock(nn.Module):
    def __init__(self, c: Flux2Config):
        super().__init__()
        D, M, hd = c.dim, c.mlp, c.head_dim
        self.img_qkv, self.txt_qkv, self.img_o, self.txt_o = _P(3 * D, D), _P(3 * D, D), _P(D, D), _P(D, D)
        self.img_qn, self.img_kn, self.txt_qn, self.txt_kn = _P(hd), _P(hd), _P(hd), _P(hd)
        self.img_ff_in, self.img_ff_out, self.txt_ff_in, self.txt_ff_out = _P(2 * M, D), _P(D, M), _P(2 * M, D), _P(D, M)


class SingleBlock(nn.Module):
    def __init__(self, c: Flux2Config):
        super().__init__()
        D, M, hd = c.dim, c.mlp, c.head_dim
        self.w_in, self.w_out, self.qn, self.kn = _P(3 * D + 2 * M, D), _P(D, D + M), _P(hd), _P(hd)


class Flux2Transformer(nn.Module):
    def __init__(self, c: Flux2Config):
        super().__init__()
        self.c = c
        D = c.dim
        self.t1, self.t2 = _P(D, c.time_channels), _P(D, D)
        if c.guidance_embeds:
            self.g1, self.g2 = _P(D, c.time_channels), _P(D, D)
        self.mod_img, self.mod_txt, self.mod_single = _P(6 * D, D), _P(6 * D, D), _P(3 * D, D)
        self.x_embed, self.ctx_embed = _P(D, c.in_channels), _P(D, c.joint_dim)
        self.double_blocks = nn.ModuleList([DoubleBlock(c) for _ in range(c.layers)])
        self.single_blocks = nn.ModuleList([SingleBlock(c) for _ in range(c.single_layers)])
        self.out_mod, self.out_proj = _P(2 * D, D), _P(c.in_channels, D)

    def time_code(self, t, guidance=None):
        dt = self.t1.dtype
        e = ops.linear(F.silu(ops.linear(sinusoid(t * 1000.0, self.c.time_channels).to(dt), self.t1)), self.t2)
        if self.c.guidance_embeds:
            g = torch.full_like(t, 1.0) if guidance is None else guidance
            e = e + ops.linear(F.silu(ops.linear(sinusoid(g * 1000.0, self.c.time_channels).to(dt), self.g1)), self.g2)
        return e

    def _heads(self, x, n):
        return x.view(x.shape[0], n, self.c.heads, self.c.head_dim)

    def forward(self, latents, text, t, img_ids, txt_ids, guidance=None, blocks=None):
        """``latents [S_img, in_channels]``, ``text [S_txt, joint_dim]``, flow time ``t`` in [0, 1], ``*_ids [S, 4]`` -> velocity
        ``[S_img, in_channels]``.  ``blocks`` (an iterator of ``("double" | "single", block)``) lets a caller stream block weights in
        one at a time instead of keeping all of them resident."""
        c = self.c
        D, M, eps = c.dim, c.mlp, c.eps
        temb = self.time_code(torch.as_tensor([float(t)], device=latents.device), guidance)
        st = F.silu(temb)
        mi, mt, ms = (ops.linear(st, w)[0] for w in (self.mod_img, self.mod_txt, self.mod_single))
        (i_sa, i_ca, i_ga, i_sm, i_cm, i_gm), (t_sa, t_ca, t_ga, t_sm, t_cm, t_gm) = mi.chunk(6), mt.chunk(6)
        s_s, s_c, s_g = ms.chunk(3)
        x = ops.linear(latents.to(self.x_embed.dtype), self.x_embed)
        y = ops.linear(text.to(self.x_embed.dtype), self.ctx_embed)
        St = y.shape[0]
        ang = rope_angles(torch.cat([txt_ids, img_ids], 0).to(x.device), c.axes_dims, c.rope_theta)
        it = blocks if blocks is not None else ([("double", b) for b in self.double_blocks] + [("single", b) for b in self.single_blocks])
        joined = None
        for kind, b in it:
            if kind == "double":
                qi, ki, vi = self._heads(ops.linear((_ln(x) * (1 + i_ca) + i_sa).contiguous(), b.img_qkv), 3).unbind(1)
                qt, kt, vt = self._heads(ops.linear((_ln(y) * (1 + t_ca) + t_sa).contiguous(), b.txt_qkv), 3).unbind(1)
                q = rope_pairs(torch.cat([ops.rmsnorm(qt, b.txt_qn, eps), ops.rmsnorm(qi, b.img_qn, eps)], 0), ang)
                k = rope_pairs(torch.cat([ops.rmsnorm(kt, b.txt_kn, eps), ops.rmsnorm(ki, b.img_kn, eps)], 0), ang)
                a = _attn(q, k, torch.cat([vt, vi], 0))
                x = x + i_ga * ops.linear(a[St:].contiguous(), b.img_o)
                y = y + t_ga * ops.linear(a[:St].contiguous(), b.txt_o)
                x = x + i_gm * ops.linear(ops.linear_glu((_ln(x) * (1 + i_cm) + i_sm).contiguous(), b.img_ff_in, "swiglu"), b.img_ff_out)
                y = y + t_gm * ops.linear(ops.linear_glu((_ln(y) * (1 + t_cm) + t_sm).contiguous(), b.txt_ff_in, "swiglu"), b.txt_ff_out)
            else:
                if joined is None:
                    joined = torch.cat([y, x], 0)
                h = ops.linear((_ln(joined) * (1 + s_c) + s_s).contiguous(), b.w_in)
                q, k, v = self._heads(h[:, :3 * D].contiguous(), 3).unbind(1)
                a = _attn(rope_pairs(ops.rmsnorm(q, b.qn, eps), ang), rope_pairs(ops.rmsnorm(k, b.kn, eps), ang), v)
                m = ops.glu(h[:, 3 * D:].contiguous(), "swiglu")
                joined = joined + s_g * ops.linear(torch.cat([a, m.to(a.dtype)], -1), b.w_out)
        x = joined[St:] if joined is not None else x
        sc, sh = ops.linear(st, self.out_mod)[0].chunk(2)
        return ops.linear((_ln(x) * (1 + sc) + sh).contiguous(), self.out_proj)


def load_into(m: Flux2Transformer, loader) -> None:
    """Names of the ``Flux2Transformer2DModel`` checkpoint layout; q / k / v of a stream are stored fused here."""
    dt = m.x_embed.dtype

    def get(n):
        return loader.load_tensor(n, dt)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    put(m.t1, "time_guidance_embed.timestep_embedder.linear_1.weight")
    put(m.t2, "time_guidance_embed.timestep_embedder.linear_2.weight")
    if m.c.guidance_embeds:
        put(m.g1, "time_guidance_embed.guidance_embedder.linear_1.weight")
        put(m.g2, "time_guidance_embed.guidance_embedder.linear_2.weight")
    for p, n in ((m.mod_img, "double_stream_modulation_img.linear.weight"), (m.mod_txt, "double_stream_modulation_txt.linear.weight"),
                 (m.mod_single, "single_stream_modulation.linear.weight"), (m.x_embed, "x_embedder.weight"),
                 (m.ctx_embed, "context_embedder.weight"), (m.out_mod, "norm_out.linear.weight"), (m.out_proj, "proj_out.weight")):
        put(p, n)
    for i, b in enumerate(m.double_blocks):
        a = f"transformer_blocks.{i}.attn."
        b.img_qkv.data.copy_(torch.cat([get(a + f"to_{n}.weight") for n in "qkv"], 0))
        b.txt_qkv.data.copy_(torch.cat([get(a + f"add_{n}_proj.weight") for n in "qkv"], 0))
        for p, n in ((b.img_o, a + "to_out.0.weight"), (b.txt_o, a + "to_add_out.weight"), (b.img_qn, a + "norm_q.weight"),
                     (b.img_kn, a + "norm_k.weight"), (b.txt_qn, a + "norm_added_q.weight"), (b.txt_kn, a + "norm_added_k.weight"),
                     (b.img_ff_in, f"transformer_blocks.{i}.ff.linear_in.weight"), (b.img_ff_out, f"transformer_blocks.{i}.ff.linear_out.weight"),
                     (b.txt_ff_in, f"transformer_blocks.{i}.ff_context.linear_in.weight"),
                     (b.txt_ff_out, f"transformer_blocks.{i}.ff_context.linear_out.weight")):
            put(p, n)
    for i, b in enumerate(m.single_blocks):
        a = f"single_transformer_blocks.{i}.attn."
        for p, n in ((b.w_in, a + "to_qkv_mlp_proj.weight"), (b.w_out, a + "to_out.weight"), (b.qn, a + "norm_q.weight"), (b.kn, a + "norm_k.weight")):
            put(p, n)

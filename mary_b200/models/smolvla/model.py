"""SmolVLA: a vision-language-action policy (src/models/smolvla/*: SigLIP + SmolLM2 backbone, flow-matching action expert,
``smolvla_infer``).

``observe -> reason -> act``: camera frames, a language instruction and the robot's proprioceptive state form the PREFIX; the
backbone (SigLIP tower, pixel-shuffle connector, SmolLM2 decoder truncated to 16 layers) runs once over it and keeps every
layer's keys and values.  The SUFFIX is a chunk of ``chunk_size`` noised actions fused with the flow time; the action expert
(narrower residual, same head geometry as the backbone so its heads can read the backbone's cache) alternates

* even layers: self-attention over ``[prefix K/V of that backbone layer ; the suffix's own K/V]``,
* odd layers: cross-attention whose keys / values are the backbone layer's cached K/V pushed through the expert's own
  ``k_proj`` / ``v_proj`` (``kv_dim -> kv_dim``), with query positions restarting at 0,

and predicts the flow velocity.  Sampling integrates ``x <- x + dt v(x, t)`` from pure noise at ``t = 1`` back to ``t = 0`` in
``num_steps`` Euler steps; the prefix is computed once per observation, every step re-runs only the expert.

Attention visibility follows block ids: images and language see each other (block 0), the state token sees them and itself
(block 1), the action chunk sees everything and itself (block 2).  All GEMMs go through ``ops.linear``; with parameters that
require gradients the same code trains the expert (the reference's SGD overfit probe is ``tests/test_smolvla_cpu.py``)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ..embed.clip import Block, gelu_tanh


@dataclass
class TowerConfig:
    width: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_dim: int
    eps: float = 1e-5
    rope_theta: float = 1e4


@dataclass
class SmolVLAConfig:
    vlm: TowerConfig = field(default_factory=lambda: TowerConfig(960, 16, 15, 5, 64, 2560))
    expert: TowerConfig = field(default_factory=lambda: TowerConfig(720, 16, 15, 5, 64, 2048))
    vocab: int = 49280
    image_size: int = 512
    patch: int = 16
    v_hidden: int = 768
    v_layers: int = 12
    v_heads: int = 12
    v_ffn: int = 3072
    shuffle: int = 4
    action_dim: int = 32
    state_dim: int = 32
    expressive_dim: int = 9
    chunk_size: int = 50
    num_steps: int = 10
    min_period: float = 4e-3
    max_period: float = 4.0
    self_attn_every: int = 2

    @staticmethod
    def tiny():
        return SmolVLAConfig(vlm=TowerConfig(48, 4, 3, 1, 16, 96), expert=TowerConfig(32, 4, 3, 1, 16, 64), vocab=64, image_size=32, patch=8,
                             v_hidden=32, v_layers=2, v_heads=4, v_ffn=64, shuffle=2, action_dim=8, state_dim=8, expressive_dim=3,
                             chunk_size=6, num_steps=4)


def time_embedding(t, dim: int, min_period: float, max_period: float):
    """``[B] -> [B, dim]``: periods spaced geometrically from ``min_period`` to ``max_period``; ``[sin(2 pi t / p), cos(2 pi t / p)]``."""
    half = dim // 2
    frac = torch.arange(half, dtype=torch.float64, device=t.device) / max(half - 1, 1)
    period = min_period * (max_period / min_period) ** frac
    ang = (2.0 * math.pi / period)[None, :] * t.double()[:, None]
    return torch.cat([ang.sin(), ang.cos()], -1).float()


def euler_sample(denoise, noise, num_steps: int):
    """Integrate the flow backwards: ``dt = -1 / num_steps``; ``t = 1 + step dt``; ``x <- x + dt * denoise(x, t)``."""
    x, dt = noise, -1.0 / num_steps
    for step in range(num_steps):
        t = torch.full((x.shape[0],), 1.0 + step * dt, dtype=torch.float32, device=x.device)
        x = x + dt * denoise(x, t)
    return x


def _P(*s):
    return nn.Parameter(torch.empty(*s))


def _rope(x, pos, theta):
    """Split-half rotation of ``x [L, heads, D]`` at integer positions ``pos [L]``."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32, device=x.device) / D))
    ang = pos.float()[:, None] * inv
    cos, sin = ang.cos()[:, None, :].to(x.dtype), ang.sin()[:, None, :].to(x.dtype)
    a, b = x[..., :D // 2], x[..., D // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


def _attend(q, k, v, mask):
    """``q [Lq, Hq, D]``, ``k, v [Lk, Hkv, D]``, ``mask [Lq, Lk]`` (True = visible) -> ``[Lq, Hq * D]``."""
    o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], attn_mask=mask[None, None],
                                       enable_gqa=True)
    return o[0].transpose(0, 1).reshape(q.shape[0], -1)


class DecoderLayer(nn.Module):
    """Pre-RMSNorm GQA + SwiGLU layer whose residual width (``width``) may differ from its attention width (``heads * head_dim``);
    ``kv_in`` is the width its key / value projections read (the residual, or the backbone's kv width on cross-attention layers)."""

    def __init__(self, t: TowerConfig, kv_in: int | None = None):
        super().__init__()
        self.t = t
        W, D = t.width, t.head_dim
        kv_in = W if kv_in is None else kv_in
        self.ln1, self.ln2 = _P(W), _P(W)
        self.wq, self.wk, self.wv, self.wo = _P(t.n_heads * D, W), _P(t.n_kv_heads * D, kv_in), _P(t.n_kv_heads * D, kv_in), _P(W, t.n_heads * D)
        self.w_gu, self.w_down = _P(2 * t.ffn_dim, W), _P(W, t.ffn_dim)

    def mlp(self, x):
        return x + ops.linear(ops.linear_glu(ops.rmsnorm(x, self.ln2, self.t.eps), self.w_gu, "swiglu"), self.w_down)


class SmolVLA(nn.Module):
    def __init__(self, c: SmolVLAConfig):
        super().__init__()
        self.c = c
        v, e = c.vlm, c.expert
        n = (c.image_size // c.patch) ** 2
        self.patch_w, self.patch_b, self.v_pos = _P(c.v_hidden, 3, c.patch, c.patch), _P(c.v_hidden), _P(n, c.v_hidden)
        self.v_blocks = nn.ModuleList([Block(c.v_hidden, c.v_heads, c.v_ffn, gelu_tanh) for _ in range(c.v_layers)])
        self.v_post_w, self.v_post_b = _P(c.v_hidden), _P(c.v_hidden)
        self.connector = _P(v.width, c.v_hidden * c.shuffle ** 2)
        self.embed = _P(c.vocab, v.width)
        self.vlm_layers = nn.ModuleList([DecoderLayer(v) for _ in range(v.n_layers)])
        kv = v.n_kv_heads * v.head_dim
        self.expert_layers = nn.ModuleList([DecoderLayer(e, None if i % c.self_attn_every == 0 else kv) for i in range(e.n_layers)])
        self.expert_norm = _P(e.width)
        self.state_proj_w, self.state_proj_b = _P(v.width, c.state_dim), _P(v.width)
        self.act_in_w, self.act_in_b = _P(e.width, c.action_dim), _P(e.width)
        self.act_out_w, self.act_out_b = _P(c.action_dim, e.width), _P(c.action_dim)
        self.at_in_w, self.at_in_b, self.at_out_w, self.at_out_b = _P(e.width, 2 * e.width), _P(e.width), _P(e.width, e.width), _P(e.width)
        for p in self.parameters():
            p.requires_grad_(False)

    # ------------------------------------------------------------------ backbone
    def image_tokens(self, pixels):
        """``pixels [3, S, S]`` in [-1, 1] -> ``[(S / patch / shuffle)^2, vlm.width]`` scaled by ``sqrt(width)``."""
        c = self.c
        x = F.conv2d(pixels[None].to(self.patch_w.dtype), self.patch_w, self.patch_b, stride=c.patch).flatten(2).transpose(1, 2) + self.v_pos
        for b in self.v_blocks:
            x = b(x, 1e-6, causal=False)
        x = F.layer_norm(x, (c.v_hidden,), self.v_post_w, self.v_post_b, 1e-6)[0]
        g, r = c.image_size // c.patch, c.shuffle
        # pixel shuffle: every r x r patch neighbourhood becomes one token with r^2 times the channels
        x = x.view(g // r, r, g // r, r, c.v_hidden).permute(0, 2, 1, 3, 4).reshape((g // r) ** 2, r * r * c.v_hidden)
        return ops.linear(x.contiguous(), self.connector) * math.sqrt(self.c.vlm.width)

    def embed_prefix(self, images, lang_ids, state):
        """``[image tokens..., language tokens, state token]`` and their visibility block ids."""
        v = self.c.vlm
        toks = [self.image_tokens(im) for im in images]
        lang = self.embed[torch.as_tensor(lang_ids, device=self.embed.device).long()] * math.sqrt(v.width)
        st = ops.linear(state.to(self.embed.dtype)[None], self.state_proj_w, self.state_proj_b)
        x = torch.cat(toks + [lang, st], 0)
        blocks = torch.cat([torch.zeros(x.shape[0] - 1, dtype=torch.long), torch.ones(1, dtype=torch.long)]).to(x.device)
        return x, blocks

    def prefix_cache(self, x, blocks):
        """Run the backbone over the prefix; returns per layer the (rotated) keys and the values ``[Lp, Hkv, D]``."""
        v = self.c.vlm
        Lp = x.shape[0]
        pos = torch.arange(Lp, device=x.device)
        mask = blocks[None, :] <= blocks[:, None]
        cache = []
        for L in self.vlm_layers:
            h = ops.rmsnorm(x, L.ln1, v.eps)
            q = _rope(ops.linear(h, L.wq).view(Lp, v.n_heads, v.head_dim), pos, v.rope_theta)
            k = _rope(ops.linear(h, L.wk).view(Lp, v.n_kv_heads, v.head_dim), pos, v.rope_theta)
            val = ops.linear(h, L.wv).view(Lp, v.n_kv_heads, v.head_dim)
            cache.append((k, val))
            x = L.mlp(x + ops.linear(_attend(q, k, val, mask), L.wo))
        return cache

    # ------------------------------------------------------------------ expert
    def embed_suffix(self, noisy, t):
        """``noisy [chunk, action_dim]``, scalar flow time ``t`` -> ``[chunk, expert.width]``: ``mlp(cat(action_in(noisy), time_code))``."""
        c, e = self.c, self.c.expert
        a = ops.linear(noisy.to(self.act_in_w.dtype), self.act_in_w, self.act_in_b)
        te = time_embedding(t.reshape(1), e.width, c.min_period, c.max_period).to(a.dtype).expand(a.shape[0], -1)
        h = F.silu(ops.linear(torch.cat([a, te], -1), self.at_in_w, self.at_in_b))
        return ops.linear(h, self.at_out_w, self.at_out_b)

    def cross_kv(self, cache):
        """The cross-attention layers' key / value projections of the prefix: they do not depend on the flow time, so one
        inference computes them once instead of once per Euler step."""
        c, e = self.c, self.c.expert
        out = {}
        for i, L in enumerate(self.expert_layers):
            if i % c.self_attn_every:
                pk, pv = cache[i]
                Lp = pk.shape[0]
                out[i] = (ops.linear(pk.reshape(Lp, -1), L.wk).view(Lp, e.n_kv_heads, e.head_dim),
                          ops.linear(pv.reshape(Lp, -1), L.wv).view(Lp, e.n_kv_heads, e.head_dim))
        return out

    def denoise(self, cache, noisy, t, cross=None):
        """Flow velocity ``[chunk, action_dim]`` of the noised chunk at time ``t`` given the backbone's prefix cache (``cross``:
        the result of :meth:`cross_kv` when the caller holds it)."""
        c, e = self.c, self.c.expert
        x = self.embed_suffix(noisy, t)
        Ls, Lp = x.shape[0], cache[0][0].shape[0]
        pos_self = torch.arange(Lp, Lp + Ls, device=x.device)                   # the suffix continues the prefix
        pos_cross = torch.arange(Ls, device=x.device)                           # cross-attention queries restart at 0
        see_all = torch.ones(Ls, Lp + Ls, dtype=torch.bool, device=x.device)
        for i, L in enumerate(self.expert_layers):
            h = ops.rmsnorm(x, L.ln1, e.eps)
            pk, pv = cache[i]
            if i % c.self_attn_every == 0:
                q = _rope(ops.linear(h, L.wq).view(Ls, e.n_heads, e.head_dim), pos_self, e.rope_theta)
                k = _rope(ops.linear(h, L.wk).view(Ls, e.n_kv_heads, e.head_dim), pos_self, e.rope_theta)
                val = ops.linear(h, L.wv).view(Ls, e.n_kv_heads, e.head_dim)
                a = _attend(q, torch.cat([pk, k], 0), torch.cat([pv, val], 0), see_all)
            else:
                q = _rope(ops.linear(h, L.wq).view(Ls, e.n_heads, e.head_dim), pos_cross, e.rope_theta)
                if cross is not None:
                    k, val = cross[i]
                else:
                    k = ops.linear(pk.reshape(Lp, -1), L.wk).view(Lp, e.n_kv_heads, e.head_dim)
                    val = ops.linear(pv.reshape(Lp, -1), L.wv).view(Lp, e.n_kv_heads, e.head_dim)
                a = _attend(q, k, val, see_all[:, :Lp])
            x = L.mlp(x + ops.linear(a, L.wo))
        return ops.linear(ops.rmsnorm(x, self.expert_norm, e.eps), self.act_out_w, self.act_out_b)

    # ------------------------------------------------------------------ policy
    @torch.no_grad()
    def act(self, images, lang_ids, state, noise=None, generator=None):
        """One inference: a chunk of ``chunk_size`` future actions; only the first ``expressive_dim`` columns drive the robot."""
        c = self.c
        cache = self.prefix_cache(*self.embed_prefix(images, lang_ids, state))
        if noise is None:
            noise = torch.randn(c.chunk_size, c.action_dim, generator=generator, device=self.embed.device)
        noise = noise.to(self.embed.dtype)
        if noise.is_cuda and self.use_graph:
            out = self._sample_graphed(cache, noise)
        else:
            cross = self.cross_kv(cache)
            out = euler_sample(lambda x, t: self.denoise(cache, x[0], t[0], cross)[None], noise[None], c.num_steps)[0]
        return out[:, :c.expressive_dim]

    use_graph = True

    def _sample_graphed(self, cache, noise):
        """The whole flow sampler (cross-attention projections of the prefix once, then ``num_steps`` Euler steps through all expert
        layers) as one CUDA graph per prefix length: the prefix cache and the noise are copied into static buffers, the graph is
        replayed, the chunk is read back.  The sampler is thousands of small dependent kernels, so its cost is launch submission."""
        c = self.c
        Lp = cache[0][0].shape[0]
        graphs = self.__dict__.setdefault("_graphs", {})
        if Lp not in graphs:
            st = {"cache": [(k.clone(), v.clone()) for k, v in cache], "noise": noise.clone()}

            def run():
                cross = self.cross_kv(st["cache"])
                return euler_sample(lambda x, t: self.denoise(st["cache"], x[0], t[0], cross)[None], st["noise"][None], c.num_steps)[0]
            side = torch.cuda.Stream(device=noise.device)
            side.wait_stream(torch.cuda.current_stream(noise.device))
            with torch.cuda.stream(side):
                run()
            torch.cuda.current_stream(noise.device).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                st["out"] = run()
            st["graph"] = g
            graphs[Lp] = st
        st = graphs[Lp]
        for (sk, sv), (k, v) in zip(st["cache"], cache):
            sk.copy_(k), sv.copy_(v)
        st["noise"].copy_(noise)
        st["graph"].replay()
        return st["out"].clone()

    def flow_loss(self, cache, actions, noise, t):
        """Training objective of the expert: ``x_t = t noise + (1 - t) actions``; target velocity ``noise - actions``; mean squared error."""
        x_t = t * noise + (1.0 - t) * actions
        return F.mse_loss(self.denoise(cache, x_t, torch.as_tensor(t, dtype=torch.float32)).float(), (noise - actions).float())


def init_random_(m: SmolVLA, seed: int = 0, std: float = 0.05) -> None:
    g = torch.Generator().manual_seed(seed)
    for n, p in m.named_parameters():
        if p.dim() == 1:
            p.data.fill_(0.0 if (n.endswith("_b") or "b_" in n.split(".")[-1]) else 1.0)
        else:
            p.data.normal_(0.0, std, generator=g)


def load_into(m: SmolVLA, loader, prefix: str = "model.") -> None:
    """Fill the policy from the released checkpoint's names (src/models/smolvla/{vision,vlm,denoiser,projections}.rs): the SmolVLM
    backbone under ``vlm_with_expert.vlm.model`` (``vision_model.*``, ``connector.modality_projection.proj``, ``text_model.*`` — only
    the first ``vlm.n_layers`` text layers exist in the policy), the action expert under ``vlm_with_expert.lm_expert`` (cross-attention
    layers carry k / v projections that read the backbone's kv width) and five biased projections beside them."""
    from ..embed.clip import load_blocks
    dt = m.embed.dtype

    def get(n):
        return loader.load_tensor(prefix + n, dt)

    def put(p, n):
        t = get(n)
        if t.numel() != p.numel():
            raise ValueError(f"{prefix}{n}: stored {tuple(t.shape)}, expected {tuple(p.shape)}")
        p.data.copy_(t.reshape(p.shape))
    vlm = "vlm_with_expert.vlm.model."
    v = vlm + "vision_model"
    put(m.patch_w, v + ".embeddings.patch_embedding.weight"), put(m.patch_b, v + ".embeddings.patch_embedding.bias")
    put(m.v_pos, v + ".embeddings.position_embedding.weight")
    put(m.v_post_w, v + ".post_layernorm.weight"), put(m.v_post_b, v + ".post_layernorm.bias")
    load_blocks(m.v_blocks, v, get)
    put(m.connector, vlm + "connector.modality_projection.proj.weight")
    put(m.embed, vlm + "text_model.embed_tokens.weight")

    def layer(L, p):
        put(L.ln1, p + "input_layernorm.weight"), put(L.ln2, p + "post_attention_layernorm.weight")
        for ours, theirs in (("wq", "q_proj"), ("wk", "k_proj"), ("wv", "v_proj"), ("wo", "o_proj")):
            put(getattr(L, ours), p + f"self_attn.{theirs}.weight")
        L.w_gu.data.copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
        put(L.w_down, p + "mlp.down_proj.weight")
    for i, L in enumerate(m.vlm_layers):
        layer(L, vlm + f"text_model.layers.{i}.")
    for i, L in enumerate(m.expert_layers):
        layer(L, f"vlm_with_expert.lm_expert.layers.{i}.")
    put(m.expert_norm, "vlm_with_expert.lm_expert.norm.weight")
    for ours, theirs in (("state_proj", "state_proj"), ("act_in", "action_in_proj"), ("act_out", "action_out_proj"),
                         ("at_in", "action_time_mlp_in"), ("at_out", "action_time_mlp_out")):
        put(getattr(m, ours + "_w"), theirs + ".weight"), put(getattr(m, ours + "_b"), theirs + ".bias")

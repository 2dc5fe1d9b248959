"""Qwen2.5-VL as a multimodal embedder (BiQwen2.5 / nomic-embed-multimodal): vision tower + decoder run as an encoder
(src/models/qwen2_5_vl/*: vision tower, text model, ``BiQwen`` pooling).

Vision tower: every image (or video) arrives as a list of ``temporal x patch x patch`` pixel patches ordered so that four
consecutive patches form one 2 x 2 merge block.  A patch is embedded by one GEMM (the stride-equals-kernel 3-D convolution),
rotated with a 2-D rotary code (half of each head's frequencies follow the row, half the column), and runs through pre-RMSNorm
blocks with biased fused qkv and biased SwiGLU.  Most blocks attend inside ``window x window`` pixel windows, the listed ones over
the whole frame; both are block-diagonal masks built from per-patch segment ids, so patches are never reordered.  The merger
norms every patch, concatenates each 2 x 2 block and maps it to the decoder's width with a two-layer GELU MLP.

Text model: Qwen2 decoder (biased q/k/v, RMSNorm, SwiGLU) with multimodal rotary positions: the rotary frequencies are split
into three sections that read the temporal, row and column coordinate of a token (all three equal for text).  An embedder needs
only one causal pass over the whole sequence, so there is no cache here; the sentence vector is the final hidden state of the
LAST token, L2-normalised."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


@dataclass
class Qwen25VLConfig:
    # vision (Qwen2.5-VL-7B)
    v_depth: int = 32
    v_hidden: int = 1280
    v_heads: int = 16
    v_ffn: int = 3420
    patch: int = 14
    temporal_patch: int = 2
    merge: int = 2
    window: int = 112
    fullatt_blocks: tuple = (7, 15, 23, 31)
    in_channels: int = 3
    tokens_per_second: int = 2
    # text
    vocab: int = 152064
    hidden: int = 3584
    layers: int = 28
    heads: int = 28
    kv_heads: int = 4
    ffn: int = 18944
    rope_theta: float = 1e6
    mrope_section: tuple = (16, 24, 24)
    eps: float = 1e-6
    image_token: int = 151655

    @staticmethod
    def tiny():
        return Qwen25VLConfig(v_depth=3, v_hidden=32, v_heads=2, v_ffn=48, patch=4, temporal_patch=2, merge=2, window=16,
                              fullatt_blocks=(1,), vocab=120, hidden=48, layers=2, heads=4, kv_heads=2, ffn=80, rope_theta=1e4,
                              mrope_section=(2, 2, 2), image_token=119)


def _P(*s):
    return nn.Parameter(torch.empty(*s), requires_grad=False)


def _lin(x, w, b=None):
    y = ops.linear(x, w)
    return y if b is None else (y.float() + b.float()).to(x.dtype)


def _rot(x, ang):
    """Split-half rotation of ``x [T, heads, D]`` by ``ang [T, D/2]``."""
    d = x.shape[-1] // 2
    cos, sin = ang.cos()[:, None, :].to(x.dtype), ang.sin()[:, None, :].to(x.dtype)
    a, b = x[..., :d], x[..., d:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


class VisionBlock(nn.Module):
    def __init__(self, c: Qwen25VLConfig):
        super().__init__()
        H, Fv = c.v_hidden, c.v_ffn
        self.n1, self.n2 = _P(H), _P(H)
        self.w_qkv, self.b_qkv, self.w_o, self.b_o = _P(3 * H, H), _P(3 * H), _P(H, H), _P(H)
        self.w_g, self.b_g, self.w_u, self.b_u, self.w_d, self.b_d = _P(Fv, H), _P(Fv), _P(Fv, H), _P(Fv), _P(H, Fv), _P(H)


class VisionTower(nn.Module):
    def __init__(self, c: Qwen25VLConfig):
        super().__init__()
        self.c = c
        H = c.v_hidden
        self.patch_w = _P(H, c.in_channels * c.temporal_patch * c.patch * c.patch)
        self.blocks = nn.ModuleList([VisionBlock(c) for _ in range(c.v_depth)])
        self.ln_q = _P(H)
        m = c.merge * c.merge
        self.m1_w, self.m1_b, self.m2_w, self.m2_b = _P(H * m, H * m), _P(H * m), _P(c.hidden, H * m), _P(c.hidden)
        hd = H // c.v_heads
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2))), persistent=False)

    def layout(self, grids, device):
        """Per patch: (row, column) for the rotary code, the id of its frame (full attention) and of its window."""
        c = self.c
        rows, cols, frame, win = [], [], [], []
        ws = c.window // c.merge // c.patch                      # window edge in merge blocks
        f0 = w0 = 0
        for t, h, w in grids:
            hb, wb = h // c.merge, w // c.merge
            bi = torch.arange(hb).view(hb, 1, 1, 1).expand(hb, wb, c.merge, c.merge)
            bj = torch.arange(wb).view(1, wb, 1, 1).expand(hb, wb, c.merge, c.merge)
            di = torch.arange(c.merge).view(1, 1, c.merge, 1).expand(hb, wb, c.merge, c.merge)
            dj = torch.arange(c.merge).view(1, 1, 1, c.merge).expand(hb, wb, c.merge, c.merge)
            r, cc = (bi * c.merge + di).reshape(-1), (bj * c.merge + dj).reshape(-1)
            nww = -(-wb // ws)
            wid = ((bi // ws) * nww + bj // ws).reshape(-1)
            nwin = (-(-hb // ws)) * nww
            for f in range(t):
                rows.append(r), cols.append(cc)
                frame.append(torch.full_like(r, f0 + f))
                win.append(wid + w0 + f * nwin)
            f0 += t
            w0 += t * nwin
        cat = lambda xs: torch.cat(xs).to(device)  # noqa: E731
        return cat(rows), cat(cols), cat(frame), cat(win)

    def forward(self, patches, grids):
        """``patches [N, C * temporal * patch * patch]``, ``grids`` = ``(t, h, w)`` per image in patches -> ``[N / merge^2, hidden]``."""
        c = self.c
        H, nh = c.v_hidden, c.v_heads
        x = ops.linear(patches.to(self.patch_w.dtype), self.patch_w)
        N = x.shape[0]
        r, cc, frame, win = self.layout(grids, x.device)
        ang = torch.cat([r[:, None].float() * self.inv_freq, cc[:, None].float() * self.inv_freq], -1)       # [N, hd/2]
        masks = {True: frame[:, None] == frame[None, :], False: win[:, None] == win[None, :]}
        for i, b in enumerate(self.blocks):
            h = ops.rmsnorm(x, b.n1, c.eps)
            qkv = _lin(h, b.w_qkv, b.b_qkv).view(N, 3, nh, H // nh)
            q, k, v = _rot(qkv[:, 0], ang), _rot(qkv[:, 1], ang), qkv[:, 2]
            a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                               attn_mask=masks[i in c.fullatt_blocks][None, None])[0].transpose(0, 1).reshape(N, H)
            x = x + _lin(a, b.w_o, b.b_o)
            h = ops.rmsnorm(x, b.n2, c.eps)
            g = F.silu(_lin(h, b.w_g, b.b_g).float()).to(x.dtype) * _lin(h, b.w_u, b.b_u)
            x = x + _lin(g, b.w_d, b.b_d)
        m = c.merge * c.merge
        y = ops.rmsnorm(x, self.ln_q, 1e-6).reshape(N // m, H * m)
        return _lin(F.gelu(_lin(y, self.m1_w, self.m1_b).float()).to(x.dtype), self.m2_w, self.m2_b)


def mrope_positions(token_types, grids, merge: int = 2, time_interval=1):
    """``[3, T]`` (temporal, row, column) positions of one sequence.  ``token_types``: 0 = text, 1 = image / video token; runs of
    vision tokens consume ``grids`` in order.  Text counts up by one on all three axes; a vision run starting at position ``p``
    gets temporal ``p * interval`` and rows / columns ``p + i`` / ``p + j`` of the merged grid; the text after it resumes at
    ``p + max(h, w) / merge``."""
    out, pos, it = [], 0, iter(grids)
    i, T = 0, len(token_types)
    while i < T:
        j = i
        while j < T and token_types[j] == token_types[i]:
            j += 1
        if token_types[i] == 0:
            out.append(torch.arange(pos, pos + j - i).expand(3, -1))
            pos += j - i
        else:
            t, h, w = next(it)
            hb, wb = h // merge, w // merge
            if t * hb * wb != j - i:
                raise ValueError(f"a run of {j - i} vision tokens does not match its grid {(t, h, w)}")
            pw = torch.arange(pos, pos + wb).repeat(hb * t)
            ph = torch.arange(pos, pos + hb).repeat_interleave(wb * t)
            out.append(torch.stack([torch.full((j - i,), pos * time_interval), ph, pw]))
            pos += max(h, w) // merge
        i = j
    return torch.cat(out, 1)


class TextLayer(nn.Module):
    def __init__(self, c: Qwen25VLConfig):
        super().__init__()
        H, D = c.hidden, c.hidden // c.heads
        n = (c.heads + 2 * c.kv_heads) * D
        self.ln1, self.ln2 = _P(H), _P(H)
        self.w_qkv, self.b_qkv, self.w_o = _P(n, H), _P(n), _P(H, c.heads * D)
        self.w_gu, self.w_down = _P(2 * c.ffn, H), _P(H, c.ffn)


class TextModel(nn.Module):
    def __init__(self, c: Qwen25VLConfig):
        super().__init__()
        self.c = c
        self.embed, self.norm = _P(c.vocab, c.hidden), _P(c.hidden)
        self.layers = nn.ModuleList([TextLayer(c) for _ in range(c.layers)])
        D = c.hidden // c.heads
        self.register_buffer("inv_freq", 1.0 / (c.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D)), persistent=False)
        sec = torch.cat([torch.full((n,), i % 3) for i, n in enumerate(c.mrope_section)])
        self.register_buffer("section", sec, persistent=False)                # which axis each rotary frequency reads

    def hidden(self, x, pos3):
        """One causal pass: ``x [T, H]`` input embeddings, ``pos3 [3, T]`` -> final-normed hidden states ``[T, H]``."""
        c = self.c
        T, D = x.shape[0], c.hidden // c.heads
        ang = pos3.to(x.device).float()[self.section].T * self.inv_freq                  # [T, D/2]
        for L in self.layers:
            h = ops.rmsnorm(x, L.ln1, c.eps)
            qkv = _lin(h, L.w_qkv, L.b_qkv)
            q, k, v = qkv.split([c.heads * D, c.kv_heads * D, c.kv_heads * D], -1)
            q, k = _rot(q.view(T, c.heads, D), ang), _rot(k.view(T, c.kv_heads, D), ang)
            a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.view(T, c.kv_heads, D).transpose(0, 1)[None],
                                               is_causal=True, enable_gqa=True)[0].transpose(0, 1).reshape(T, c.heads * D)
            x = x + ops.linear(a, L.w_o)
            h = ops.rmsnorm(x, L.ln2, c.eps)
            x = x + ops.linear(ops.linear_glu(h, L.w_gu, "swiglu"), L.w_down)
        return ops.rmsnorm(x, self.norm, c.eps)


class BiQwenEmbedder(nn.Module):
    """One vector per (text, images) input: image features replace the image-token rows, the decoder runs once, the last token's
    state is the embedding."""

    def __init__(self, c: Qwen25VLConfig):
        super().__init__()
        self.c, self.visual, self.text = c, VisionTower(c), TextModel(c)

    def embed(self, ids, patches=None, grids=()):
        c = self.c
        ids = torch.as_tensor(ids, device=self.text.embed.device).long()
        x = self.text.embed[ids]
        is_img = ids == c.image_token
        if patches is not None:
            feats = self.visual(patches, grids)
            if int(is_img.sum()) != feats.shape[0]:
                raise ValueError(f"{int(is_img.sum())} image tokens for {feats.shape[0]} image features")
            x = x.clone()
            x[is_img] = feats.to(x.dtype)
        pos3 = mrope_positions(is_img.int().tolist(), grids, c.merge)
        return F.normalize(self.text.hidden(x, pos3)[-1].float(), dim=-1)


def load_into(m: BiQwenEmbedder, loader, prefix: str = "") -> None:
    """Names of the Hugging Face ``Qwen2_5_VLModel`` layout (``visual.*`` and ``language_model.*``)."""
    def get(n):
        return loader.load_tensor(prefix + n, m.text.embed.dtype)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    v = m.visual
    put(v.patch_w, "visual.patch_embed.proj.weight")
    for i, b in enumerate(v.blocks):
        p = f"visual.blocks.{i}."
        for ours, theirs in (("n1", "norm1.weight"), ("n2", "norm2.weight"), ("w_qkv", "attn.qkv.weight"), ("b_qkv", "attn.qkv.bias"),
                             ("w_o", "attn.proj.weight"), ("b_o", "attn.proj.bias"), ("w_g", "mlp.gate_proj.weight"), ("b_g", "mlp.gate_proj.bias"),
                             ("w_u", "mlp.up_proj.weight"), ("b_u", "mlp.up_proj.bias"), ("w_d", "mlp.down_proj.weight"), ("b_d", "mlp.down_proj.bias")):
            put(getattr(b, ours), p + theirs)
    for ours, theirs in (("ln_q", "ln_q.weight"), ("m1_w", "mlp.0.weight"), ("m1_b", "mlp.0.bias"), ("m2_w", "mlp.2.weight"), ("m2_b", "mlp.2.bias")):
        put(getattr(v, ours), "visual.merger." + theirs)
    t = m.text
    put(t.embed, "language_model.embed_tokens.weight")
    put(t.norm, "language_model.norm.weight")
    for i, L in enumerate(t.layers):
        p = f"language_model.layers.{i}."
        L.w_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
        L.b_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.bias") for n in "qkv"], 0))
        put(L.w_o, p + "self_attn.o_proj.weight")
        L.w_gu.data.copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
        put(L.w_down, p + "mlp.down_proj.weight")
        put(L.ln1, p + "input_layernorm.weight")
        put(L.ln2, p + "post_attention_layernorm.weight")

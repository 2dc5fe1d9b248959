"""CLIP as a local embedder: images and texts in one contrastive space, L2-normalised so that cosine similarity is a dot product.

Architecture as the reference pins it (src/embed.rs:1-27): vision ViT — patch convolution without bias, learned class and
position embeddings, ``pre_layrnorm`` (the checkpoint's spelling) before the blocks, pre-LayerNorm blocks with **quick-GELU**
(``x * sigmoid(1.702 x)``), ``post_layernorm`` on the class token, ``visual_projection`` without bias; text transformer — token
+ position embeddings, causal attention, quick-GELU, final LayerNorm, the hidden state at the end-of-text position
(``argmax`` of the ids), ``text_projection`` without bias.  ``LocalEmbedder`` in the reference is the seam a file-indexing
service calls (``embed_image`` / ``embed_text`` against a warm handle, src/embed.rs:446); ``ClipEmbedder`` here is that handle.
The GEMMs go through ``ops.linear`` (the tensor-core kernels on a GPU); attention of these 50- and 77-token sequences and the
LayerNorms are plain tensor ops."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


@dataclass
class ClipConfig:
    # clip-vit-base-patch32
    image_size: int = 224
    patch: int = 32
    v_hidden: int = 768
    v_layers: int = 12
    v_heads: int = 12
    v_ffn: int = 3072
    t_vocab: int = 49408
    t_ctx: int = 77
    t_hidden: int = 512
    t_layers: int = 12
    t_heads: int = 8
    t_ffn: int = 2048
    dim: int = 512
    eps: float = 1e-5

    @staticmethod
    def tiny():
        return ClipConfig(image_size=32, patch=8, v_hidden=64, v_layers=2, v_heads=4, v_ffn=128, t_vocab=99, t_ctx=16, t_hidden=48,
                          t_layers=2, t_heads=4, t_ffn=96, dim=40)


def _P(*shape):
    return nn.Parameter(torch.empty(*shape), requires_grad=False)


def quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


class Block(nn.Module):
    """Pre-LayerNorm transformer block with biases; ``act`` is the MLP's activation (quick-GELU for CLIP)."""

    def __init__(self, H, heads, ffn, act=quick_gelu):
        super().__init__()
        self.heads, self.act = heads, act
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = _P(H), _P(H), _P(H), _P(H)
        self.w_qkv, self.b_qkv = _P(3 * H, H), _P(3 * H)
        self.w_o, self.b_o = _P(H, H), _P(H)
        self.w_fc1, self.b_fc1, self.w_fc2, self.b_fc2 = _P(ffn, H), _P(ffn), _P(H, ffn), _P(H)

    def forward(self, x, eps, causal):
        """``x [B, T, H]``."""
        B, T, H = x.shape
        h = F.layer_norm(x, (H,), self.ln1_w, self.ln1_b, eps)
        qkv = (ops.linear(h.reshape(B * T, H), self.w_qkv).float() + self.b_qkv.float()).to(x.dtype).view(B, T, 3, self.heads, H // self.heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=causal).transpose(1, 2).reshape(B * T, H)
        x = x + (ops.linear(a, self.w_o).float() + self.b_o.float()).to(x.dtype).view(B, T, H)
        h = F.layer_norm(x, (H,), self.ln2_w, self.ln2_b, eps).reshape(B * T, H)
        m = self.act((ops.linear(h, self.w_fc1).float() + self.b_fc1.float())).to(x.dtype)
        return x + (ops.linear(m, self.w_fc2).float() + self.b_fc2.float()).to(x.dtype).view(B, T, H)


class ClipEmbedder(nn.Module):
    MEAN = (0.48145466, 0.4578275, 0.40821073)
    STD = (0.26862954, 0.26130258, 0.27577711)

    def __init__(self, c: ClipConfig):
        super().__init__()
        self.c = c
        n = (c.image_size // c.patch) ** 2
        self.patch_w = _P(c.v_hidden, 3, c.patch, c.patch)
        self.cls, self.v_pos = _P(c.v_hidden), _P(n + 1, c.v_hidden)
        self.pre_w, self.pre_b, self.post_w, self.post_b = _P(c.v_hidden), _P(c.v_hidden), _P(c.v_hidden), _P(c.v_hidden)
        self.v_blocks = nn.ModuleList([Block(c.v_hidden, c.v_heads, c.v_ffn) for _ in range(c.v_layers)])
        self.v_proj = _P(c.dim, c.v_hidden)
        self.tok, self.t_pos = _P(c.t_vocab, c.t_hidden), _P(c.t_ctx, c.t_hidden)
        self.t_blocks = nn.ModuleList([Block(c.t_hidden, c.t_heads, c.t_ffn) for _ in range(c.t_layers)])
        self.fin_w, self.fin_b = _P(c.t_hidden), _P(c.t_hidden)
        self.t_proj = _P(c.dim, c.t_hidden)

    def preprocess(self, image):
        """``image [3, H, W]`` floats in [0, 1] -> normalised ``[3, S, S]``: bicubic resize of the shorter side to the model's
        size, centre crop, channel mean / std of the CLIP training set."""
        S = self.c.image_size
        _, h, w = image.shape
        scale = S / min(h, w)
        nh, nw = max(S, round(h * scale)), max(S, round(w * scale))
        img = F.interpolate(image[None].float(), size=(nh, nw), mode="bicubic", align_corners=False, antialias=True)[0]
        t, l = (nh - S) // 2, (nw - S) // 2
        img = img[:, t:t + S, l:l + S].clamp(0, 1)
        mean, std = (torch.tensor(v, device=img.device)[:, None, None] for v in (self.MEAN, self.STD))
        return (img - mean) / std

    def embed_image(self, pixels):
        """``pixels [B, 3, S, S]`` already normalised -> unit vectors ``[B, dim]``."""
        c = self.c
        x = F.conv2d(pixels.to(self.patch_w.dtype), self.patch_w, stride=c.patch).flatten(2).transpose(1, 2)      # [B, n, H]
        x = torch.cat([self.cls.expand(x.shape[0], 1, -1), x], 1) + self.v_pos
        x = F.layer_norm(x, (c.v_hidden,), self.pre_w, self.pre_b, c.eps)
        for b in self.v_blocks:
            x = b(x, c.eps, causal=False)
        pooled = F.layer_norm(x[:, 0], (c.v_hidden,), self.post_w, self.post_b, c.eps)
        return F.normalize(ops.linear(pooled, self.v_proj).float(), dim=-1)

    def embed_text(self, ids):
        """``ids [B, T]`` (padded with values below the end-of-text id) -> unit vectors ``[B, dim]``."""
        c = self.c
        ids = torch.as_tensor(ids, device=self.tok.device).long()
        x = self.tok[ids] + self.t_pos[:ids.shape[1]]
        for b in self.t_blocks:
            x = b(x, c.eps, causal=True)
        x = F.layer_norm(x, (c.t_hidden,), self.fin_w, self.fin_b, c.eps)
        pooled = x[torch.arange(ids.shape[0], device=x.device), ids.argmax(-1)]          # end-of-text holds the largest id
        return F.normalize(ops.linear(pooled, self.t_proj).float(), dim=-1)

    def similarity(self, pixels, ids):
        return self.embed_image(pixels) @ self.embed_text(ids).T


def load_into(m: ClipEmbedder, loader) -> None:
    """Checkpoint names of ``openai/clip-vit-*`` (``vision_model.*``, ``text_model.*``, ``visual_projection``, ``text_projection``)."""
    def get(n):
        return loader.load_tensor(n, m.patch_w.dtype)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    put(m.patch_w, "vision_model.embeddings.patch_embedding.weight")
    put(m.cls, "vision_model.embeddings.class_embedding")
    put(m.v_pos, "vision_model.embeddings.position_embedding.weight")
    put(m.pre_w, "vision_model.pre_layrnorm.weight")
    put(m.pre_b, "vision_model.pre_layrnorm.bias")
    put(m.post_w, "vision_model.post_layernorm.weight")
    put(m.post_b, "vision_model.post_layernorm.bias")
    put(m.v_proj, "visual_projection.weight")
    put(m.tok, "text_model.embeddings.token_embedding.weight")
    put(m.t_pos, "text_model.embeddings.position_embedding.weight")
    put(m.fin_w, "text_model.final_layer_norm.weight")
    put(m.fin_b, "text_model.final_layer_norm.bias")
    put(m.t_proj, "text_projection.weight")
    for tower, blocks in (("vision_model", m.v_blocks), ("text_model", m.t_blocks)):
        load_blocks(blocks, tower, get)


def load_blocks(blocks, tower: str, get) -> None:
    """Fill ``Block`` s from the ``<tower>.encoder.layers.<i>.*`` names that the CLIP and SigLIP checkpoints share."""
    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    if True:
        for i, b in enumerate(blocks):
            p = f"{tower}.encoder.layers.{i}."
            b.w_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
            b.b_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.bias") for n in "qkv"], 0))
            put(b.w_o, p + "self_attn.out_proj.weight")
            put(b.b_o, p + "self_attn.out_proj.bias")
            for ours, theirs in (("ln1", "layer_norm1"), ("ln2", "layer_norm2")):
                put(getattr(b, ours + "_w"), p + theirs + ".weight")
                put(getattr(b, ours + "_b"), p + theirs + ".bias")
            for ours, theirs in (("fc1", "mlp.fc1"), ("fc2", "mlp.fc2")):
                put(getattr(b, "w_" + ours), p + theirs + ".weight")
                put(getattr(b, "b_" + ours), p + theirs + ".bias")

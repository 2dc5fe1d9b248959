"""nomic-embed-text as a local embedder (src/embed.rs: the ``nomic`` text arm of ``LocalEmbedder``).

A BERT-shaped encoder with the changes nomic made: rotary positions instead of learned ones (split-half rotation over the whole
head), SwiGLU MLPs, no biases in attention or MLP, POST-LayerNorm blocks (``x = LN(x + f(x))``), token-type embedding row 0
added to every token, LayerNorm after the embeddings.  The sentence vector is the mean of the final hidden states over the real
(unpadded) tokens, optionally truncated to a Matryoshka prefix after a weightless LayerNorm, then L2-normalised.  Texts carry a
task prefix (``search_document: `` / ``search_query: ``), which is the caller's job (it is part of the text)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...ops import reference as ref
from .clip import _P


@dataclass
class NomicConfig:
    vocab_size: int = 30528
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 3072
    type_vocab: int = 2
    rope_theta: float = 1000.0
    eps: float = 1e-12

    @staticmethod
    def tiny():
        return NomicConfig(vocab_size=120, hidden=64, layers=2, heads=4, ffn=96)


class NomicLayer(nn.Module):
    def __init__(self, c: NomicConfig):
        super().__init__()
        H = c.hidden
        self.w_qkv, self.w_o, self.w_gu, self.w_down = _P(3 * H, H), _P(H, H), _P(2 * c.ffn, H), _P(H, c.ffn)
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = _P(H), _P(H), _P(H), _P(H)


class NomicTextEmbedder(nn.Module):
    def __init__(self, c: NomicConfig):
        super().__init__()
        self.c = c
        self.tok, self.typ = _P(c.vocab_size, c.hidden), _P(c.type_vocab, c.hidden)
        self.emb_ln_w, self.emb_ln_b = _P(c.hidden), _P(c.hidden)
        self.layers = nn.ModuleList([NomicLayer(c) for _ in range(c.layers)])
        self.register_buffer("inv_freq", ref.rope_inv_freq(c.hidden // c.heads, c.rope_theta), persistent=False)

    def hidden(self, ids, mask=None):
        """``ids [B, T]``, ``mask [B, T]`` (1 = real token) -> final hidden states ``[B, T, H]``."""
        c = self.c
        ids = torch.as_tensor(ids, device=self.tok.device).long()
        B, T = ids.shape
        H, nh = c.hidden, c.heads
        x = F.layer_norm(self.tok[ids] + self.typ[0], (H,), self.emb_ln_w, self.emb_ln_b, c.eps)
        pos = torch.arange(T, device=x.device).repeat(B)
        bias = None
        if mask is not None:
            bias = torch.zeros(B, 1, 1, T, dtype=x.dtype, device=x.device).masked_fill(~torch.as_tensor(mask, device=x.device).bool()[:, None, None, :], float("-inf"))
        for L in self.layers:
            qkv = ops.linear(x.reshape(B * T, H), L.w_qkv).view(B * T, 3, nh, H // nh)
            q, k = ref.rope(qkv[:, 0], pos, self.inv_freq), ref.rope(qkv[:, 1], pos, self.inv_freq)
            q, k, v = (t.reshape(B, T, nh, -1).transpose(1, 2) for t in (q, k, qkv[:, 2]))
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=bias).transpose(1, 2).reshape(B * T, H)
            x = F.layer_norm(x + ops.linear(a, L.w_o).view(B, T, H), (H,), L.ln1_w, L.ln1_b, c.eps)
            m = ops.linear(ops.linear_glu(x.reshape(B * T, H), L.w_gu, "swiglu"), L.w_down).view(B, T, H)
            x = F.layer_norm(x + m, (H,), L.ln2_w, L.ln2_b, c.eps)
        return x

    def embed_text(self, ids, mask=None, dim: int | None = None):
        """Mean over real tokens -> (optional Matryoshka prefix of ``dim`` after a weightless LayerNorm) -> unit vectors."""
        x = self.hidden(ids, mask).float()
        m = torch.ones(x.shape[:2], device=x.device) if mask is None else torch.as_tensor(mask, device=x.device).float()
        v = (x * m[..., None]).sum(1) / m.sum(1, keepdim=True).clamp_min(1e-9)
        if dim is not None:
            v = F.layer_norm(v, (v.shape[-1],))[:, :dim]
        return F.normalize(v, dim=-1)


def load_into(m: NomicTextEmbedder, loader, prefix: str = "") -> None:
    """Checkpoint names of the Hugging Face ``nomic_bert`` layout (``embeddings.*``, ``layers.<i>.*``)."""
    def get(n):
        return loader.load_tensor(prefix + n, m.tok.dtype)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    put(m.tok, "embeddings.word_embeddings.weight")
    put(m.typ, "embeddings.token_type_embeddings.weight")
    put(m.emb_ln_w, "embeddings.LayerNorm.weight")
    put(m.emb_ln_b, "embeddings.LayerNorm.bias")
    for i, L in enumerate(m.layers):
        p = f"layers.{i}."
        L.w_qkv.data.copy_(torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
        put(L.w_o, p + "self_attn.o_proj.weight")
        L.w_gu.data.copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
        put(L.w_down, p + "mlp.down_proj.weight")
        for ours, theirs in (("ln1", "post_attention_layernorm"), ("ln2", "post_mlp_layernorm")):
            put(getattr(L, ours + "_w"), p + theirs + ".weight")
            put(getattr(L, ours + "_b"), p + theirs + ".bias")


# ---- nomic-embed-vision: the image arm, aligned to the text arm's space -----------------------------------------------------

@dataclass
class NomicVisionConfig:
    image_size: int = 224
    patch: int = 16
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 2048
    eps: float = 1e-6                   # encoder and selector LayerNorms; the MLP's inner norm keeps torch's default 1e-5

    @staticmethod
    def tiny():
        return NomicVisionConfig(image_size=32, patch=8, hidden=64, layers=2, heads=4, ffn=96)

    @property
    def grid(self) -> int:
        return self.image_size // self.patch


def axial_rope_tables(grid: int, head_dim: int, temperature: float = 10000.0):
    """cos / sin ``[grid*grid, head_dim]`` of the 2-D axial rotary embedding over the patch grid (src/embed.rs:2325-2370):
    ``head_dim / 4`` bands ``temperature^(-i / bands)``; token (r, c) gets the angles ``[r * bands ; c * bands]`` and every angle
    is repeated twice, so that consecutive PAIRS of channels rotate together (the interleaved convention)."""
    nb = head_dim // 4
    bands = temperature ** (-torch.arange(nb, dtype=torch.float64) / nb)
    r, c = torch.meshgrid(torch.arange(grid, dtype=torch.float64), torch.arange(grid, dtype=torch.float64), indexing="ij")
    ang = torch.cat([r.reshape(-1, 1) * bands, c.reshape(-1, 1) * bands], 1).repeat_interleave(2, dim=1)      # [n, head_dim]
    return ang.cos().float(), ang.sin().float()


def rotate_pairs(x, cos, sin):
    """``x * cos + rot(x) * sin`` with ``rot(x) = (-x1, x0, -x3, x2, ...)``."""
    x2 = x.unflatten(-1, (-1, 2))
    rot = torch.stack([-x2[..., 1], x2[..., 0]], -1).flatten(-2)
    return x * cos + rot * sin


class NomicVisionLayer(nn.Module):
    def __init__(self, c: NomicVisionConfig):
        super().__init__()
        H, Fh = c.hidden, c.ffn
        self.w_qkv, self.b_qkv, self.w_o, self.b_o = _P(3 * H, H), _P(3 * H), _P(H, H), _P(H)
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = _P(H), _P(H), _P(H), _P(H)
        self.w_fc11, self.b_fc11, self.w_fc12, self.b_fc12 = _P(Fh, H), _P(Fh), _P(Fh, H), _P(Fh)
        self.mlp_ln_w, self.mlp_ln_b = _P(Fh), _P(Fh)
        self.w_fc2, self.b_fc2 = _P(H, Fh), _P(H)


def _lin(x, w, b):
    return ops.linear(x, w, b)


class NomicVisionEmbedder(nn.Module):
    """A 12-layer PRE-norm ViT with a learned-query attention-pooling head (src/embed.rs:2144-2560).

    * patches: a linear map over flattened ``(c, p1, p2)`` patches (run as a strided convolution with the weight reshaped), a
      learned class token in front, a learned absolute position table added to all ``1 + n`` tokens;
    * attention: full, bidirectional, with the axial rotary embedding applied to the PATCH tokens' q and k only (the class token is
      left alone);
    * blocks keep a running residual: ``res = x + res; h = attn(ln1(res)); res = h + res; h = mlp(ln2(res))`` and the block
      returns ``(h, res)``; after the last block ``hidden = h + res``; there is no final LayerNorm;
    * MLP: ``fc2(LayerNorm(fc11(x) * silu(fc12(x))))`` with biases everywhere;
    * pooling (the "selector"): one learned latent query cross-attends over all tokens, then ``out = a + mlp(ln(a))`` (same gated
      MLP without the inner norm).  That pooled vector is what the released model calls ``last_hidden_state``; class-token
      pooling is NOT the embedding.  L2-normalise for the 768-d unit vector."""
    MEAN, STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)

    def __init__(self, c: NomicVisionConfig):
        super().__init__()
        self.c = c
        H, n = c.hidden, c.grid ** 2
        self.patch_w, self.patch_b = _P(H, 3 * c.patch * c.patch), _P(H)
        self.cls, self.pos = _P(1, 1, H), _P(1, n + 1, H)
        self.layers = nn.ModuleList([NomicVisionLayer(c) for _ in range(c.layers)])
        self.latent = _P(1, 1, H)
        self.sel_wq, self.sel_bq, self.sel_wkv, self.sel_bkv, self.sel_wo, self.sel_bo = _P(H, H), _P(H), _P(2 * H, H), _P(2 * H), _P(H, H), _P(H)
        self.sel_ln_w, self.sel_ln_b = _P(H), _P(H)
        self.sel_fc11, self.sel_b11, self.sel_fc12, self.sel_b12 = _P(c.ffn, H), _P(c.ffn), _P(c.ffn, H), _P(c.ffn)
        self.sel_fc2, self.sel_b2 = _P(H, c.ffn), _P(H)
        cos, sin = axial_rope_tables(c.grid, H // c.heads)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    preprocess = None                   # assigned below: the CLIP image processor (same resize, crop and statistics)

    def tokens(self, pixels):
        """``pixels [B, 3, S, S]`` normalised -> encoder output ``[B, 1 + n, H]`` (before pooling)."""
        c = self.c
        H, nh = c.hidden, c.heads
        w = self.patch_w.view(H, 3, c.patch, c.patch)
        x = F.conv2d(pixels.to(w.dtype), w, self.patch_b, stride=c.patch).flatten(2).transpose(1, 2)
        B = x.shape[0]
        x = torch.cat([self.cls.expand(B, 1, H), x], 1) + self.pos
        T = x.shape[1]
        cos, sin = self.cos.to(x.dtype), self.sin.to(x.dtype)
        res = None
        for L in self.layers:
            res = x if res is None else x + res
            h = F.layer_norm(res, (H,), L.ln1_w, L.ln1_b, c.eps)
            qkv = _lin(h.reshape(B * T, H), L.w_qkv, L.b_qkv).view(B, T, 3, nh, H // nh)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))                        # [B, nh, T, hd]
            q = torch.cat([q[:, :, :1], rotate_pairs(q[:, :, 1:], cos, sin)], 2)
            k = torch.cat([k[:, :, :1], rotate_pairs(k[:, :, 1:], cos, sin)], 2)
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B * T, H)
            res = _lin(a, L.w_o, L.b_o).view(B, T, H) + res
            h = F.layer_norm(res, (H,), L.ln2_w, L.ln2_b, c.eps).reshape(B * T, H)
            g = _lin(h, L.w_fc11, L.b_fc11) * F.silu(_lin(h, L.w_fc12, L.b_fc12))
            g = F.layer_norm(g, (c.ffn,), L.mlp_ln_w, L.mlp_ln_b, 1e-5)
            x = _lin(g, L.w_fc2, L.b_fc2).view(B, T, H)
        return x + res

    def pool(self, x):
        """The selector: ``x [B, T, H]`` -> ``[B, H]``."""
        c = self.c
        B, T, H = x.shape
        nh = c.heads
        q = _lin(self.latent.expand(B, 1, H).reshape(B, H).to(x.dtype), self.sel_wq, self.sel_bq).view(B, 1, nh, H // nh).transpose(1, 2)
        kv = _lin(x.reshape(B * T, H), self.sel_wkv, self.sel_bkv).view(B, T, 2, nh, H // nh)
        k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, H)
        a = _lin(a, self.sel_wo, self.sel_bo)
        n = F.layer_norm(a, (H,), self.sel_ln_w, self.sel_ln_b, c.eps)
        return a + _lin(_lin(n, self.sel_fc11, self.sel_b11) * F.silu(_lin(n, self.sel_fc12, self.sel_b12)), self.sel_fc2, self.sel_b2)

    def embed_image(self, pixels):
        return F.normalize(self.pool(self.tokens(pixels)).float(), dim=-1)

    def embed_text(self, ids, mask=None, dim=None):
        raise ValueError("nomic-embed-vision is image-only; use NomicTextEmbedder for text")


def _clip_preprocess(self, image):
    from .clip import ClipEmbedder
    return ClipEmbedder.preprocess(self, image)


NomicVisionEmbedder.preprocess = _clip_preprocess


def vision_tensor_shapes(c: NomicVisionConfig | None = None) -> dict:
    """The fixed tensor inventory of the released vision checkpoint, name -> shape (``EmbeddingArchitecture::tensor_shapes``,
    src/embed.rs:310-350): what a key map must provide, checked before any weight is read."""
    c = c or NomicVisionConfig()
    H, Fh, n = c.hidden, c.ffn, c.grid ** 2
    t = {"embeddings.cls_token": (1, 1, H), "embeddings.pos_embed": (1, n + 1, H)}

    def lin(name, o, i):
        t[name + ".weight"], t[name + ".bias"] = (o, i), (o,)

    def ln(name, d):
        t[name + ".weight"], t[name + ".bias"] = (d,), (d,)

    def mlp(p, inner):
        lin(p + ".fc11", Fh, H), lin(p + ".fc12", Fh, H)
        if inner:
            ln(p + ".norm", Fh)
        lin(p + ".fc2", H, Fh)
    lin("embeddings.proj", H, 3 * c.patch * c.patch)
    for i in range(c.layers):
        p = f"layers.{i}"
        lin(p + ".attn.Wqkv", 3 * H, H), lin(p + ".attn.out_proj", H, H), ln(p + ".norm1", H), mlp(p + ".mlp", True), ln(p + ".norm2", H)
    t["selector.attn.latent"] = (1, 1, H)
    lin("selector.attn.Wq", H, H), lin("selector.attn.Wkv", 2 * H, H), lin("selector.attn.out_proj", H, H)
    ln("selector.norm1", H), mlp("selector.mlp", False)
    return t


def load_vision_into(m: NomicVisionEmbedder, loader, prefix: str = "") -> None:
    """Checkpoint names of the released ``nomic_bert`` ViT (``embeddings.*``, ``layers.<i>.*``, ``selector.*``).  The inventory is
    validated first: a missing name or a wrong shape is reported before any tensor is copied."""
    want = vision_tensor_shapes(m.c)
    if hasattr(loader, "has_weight"):
        missing = [n for n in want if not loader.has_weight(prefix + n)]
        if missing:
            raise ValueError(f"{len(missing)} of {len(want)} tensors missing, e.g. {missing[:3]}")

    def put(p, n):
        t = loader.load_tensor(prefix + n, p.dtype)
        if tuple(t.shape) != tuple(want[n]):
            raise ValueError(f"{n}: stored shape {tuple(t.shape)}, the architecture fixes {tuple(want[n])}")
        p.data.copy_(t.reshape(p.shape))
    put(m.cls, "embeddings.cls_token"), put(m.pos, "embeddings.pos_embed")
    put(m.patch_w, "embeddings.proj.weight"), put(m.patch_b, "embeddings.proj.bias")
    pairs = (("w_qkv", "b_qkv", "attn.Wqkv"), ("w_o", "b_o", "attn.out_proj"), ("ln1_w", "ln1_b", "norm1"), ("ln2_w", "ln2_b", "norm2"),
             ("w_fc11", "b_fc11", "mlp.fc11"), ("w_fc12", "b_fc12", "mlp.fc12"), ("mlp_ln_w", "mlp_ln_b", "mlp.norm"),
             ("w_fc2", "b_fc2", "mlp.fc2"))
    for i, L in enumerate(m.layers):
        for w, b, theirs in pairs:
            put(getattr(L, w), f"layers.{i}.{theirs}.weight"), put(getattr(L, b), f"layers.{i}.{theirs}.bias")
    put(m.latent, "selector.attn.latent")
    for w, b, theirs in (("sel_wq", "sel_bq", "attn.Wq"), ("sel_wkv", "sel_bkv", "attn.Wkv"), ("sel_wo", "sel_bo", "attn.out_proj"),
                         ("sel_ln_w", "sel_ln_b", "norm1"), ("sel_fc11", "sel_b11", "mlp.fc11"), ("sel_fc12", "sel_b12", "mlp.fc12"),
                         ("sel_fc2", "sel_b2", "mlp.fc2")):
        put(getattr(m, w), f"selector.{theirs}.weight"), put(getattr(m, b), f"selector.{theirs}.bias")

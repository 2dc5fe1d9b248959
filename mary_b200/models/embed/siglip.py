"""SigLIP / SigLIP2 (fixed-resolution) as a local embedder (src/embed.rs: the ``siglip2`` arm of ``LocalEmbedder``).

Differences from CLIP that matter for parity: the patch convolution has a bias and there is no class token; blocks use
tanh-GELU; the image vector is a **multi-head attention pooling** of all patch tokens (one learned probe as the only query,
then LayerNorm + MLP with a residual); the text tower is NOT causal, pools the LAST position and projects it with a biased
linear head; similarity is ``exp(logit_scale) * cos + logit_bias`` (a sigmoid loss, so scores are per-pair probabilities)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from .clip import Block, _P, gelu_tanh, load_blocks


@dataclass
class SiglipConfig:
    # siglip2-base-patch16-224
    image_size: int = 224
    patch: int = 16
    v_hidden: int = 768
    v_layers: int = 12
    v_heads: int = 12
    v_ffn: int = 3072
    t_vocab: int = 256000
    t_ctx: int = 64
    t_hidden: int = 768
    t_layers: int = 12
    t_heads: int = 12
    t_ffn: int = 3072
    eps: float = 1e-6

    @staticmethod
    def tiny():
        return SiglipConfig(image_size=32, patch=8, v_hidden=64, v_layers=2, v_heads=4, v_ffn=128, t_vocab=99, t_ctx=16, t_hidden=64,
                            t_layers=2, t_heads=4, t_ffn=96)


class SiglipEmbedder(nn.Module):
    MEAN = STD = (0.5, 0.5, 0.5)

    def __init__(self, c: SiglipConfig):
        super().__init__()
        self.c = c
        Hv, Ht = c.v_hidden, c.t_hidden
        n = (c.image_size // c.patch) ** 2
        self.patch_w, self.patch_b, self.v_pos = _P(Hv, 3, c.patch, c.patch), _P(Hv), _P(n, Hv)
        self.v_blocks = nn.ModuleList([Block(Hv, c.v_heads, c.v_ffn, gelu_tanh) for _ in range(c.v_layers)])
        self.post_w, self.post_b = _P(Hv), _P(Hv)
        # attention pooling head
        self.probe, self.pool_in_w, self.pool_in_b, self.pool_out_w, self.pool_out_b = _P(Hv), _P(3 * Hv, Hv), _P(3 * Hv), _P(Hv, Hv), _P(Hv)
        self.pool_ln_w, self.pool_ln_b = _P(Hv), _P(Hv)
        self.pool_fc1_w, self.pool_fc1_b, self.pool_fc2_w, self.pool_fc2_b = _P(c.v_ffn, Hv), _P(c.v_ffn), _P(Hv, c.v_ffn), _P(Hv)
        self.tok, self.t_pos = _P(c.t_vocab, Ht), _P(c.t_ctx, Ht)
        self.t_blocks = nn.ModuleList([Block(Ht, c.t_heads, c.t_ffn, gelu_tanh) for _ in range(c.t_layers)])
        self.fin_w, self.fin_b, self.head_w, self.head_b = _P(Ht), _P(Ht), _P(Ht, Ht), _P(Ht)
        self.logit_scale, self.logit_bias = _P(1), _P(1)

    def preprocess(self, image):
        """``image [3, H, W]`` in [0, 1] -> ``[3, S, S]``: bilinear resize straight to the square (no crop), then ``(x - 0.5) / 0.5``."""
        S = self.c.image_size
        img = F.interpolate(image[None].float(), size=(S, S), mode="bilinear", align_corners=False, antialias=True)[0]
        return (img.clamp(0, 1) - 0.5) / 0.5

    def image_features(self, pixels):
        c = self.c
        Hv, nh = c.v_hidden, c.v_heads
        x = F.conv2d(pixels.to(self.patch_w.dtype), self.patch_w, self.patch_b, stride=c.patch).flatten(2).transpose(1, 2) + self.v_pos
        for b in self.v_blocks:
            x = b(x, c.eps, causal=False)
        x = F.layer_norm(x, (Hv,), self.post_w, self.post_b, c.eps)
        B, T, _ = x.shape
        wq, wk, wv = self.pool_in_w.split(Hv, 0)
        bq, bk, bv = self.pool_in_b.split(Hv, 0)
        q = (self.probe @ wq.T + bq).view(1, nh, 1, Hv // nh).expand(B, -1, -1, -1)
        flat = x.reshape(B * T, Hv)
        k = (ops.linear(flat, wk.contiguous()).float() + bk).to(x.dtype).view(B, T, nh, -1).transpose(1, 2)
        v = (ops.linear(flat, wv.contiguous()).float() + bv).to(x.dtype).view(B, T, nh, -1).transpose(1, 2)
        a = F.scaled_dot_product_attention(q.to(x.dtype), k, v).transpose(1, 2).reshape(B, Hv)
        a = (ops.linear(a, self.pool_out_w).float() + self.pool_out_b).to(x.dtype)
        h = F.layer_norm(a, (Hv,), self.pool_ln_w, self.pool_ln_b, c.eps)
        m = gelu_tanh(ops.linear(h, self.pool_fc1_w).float() + self.pool_fc1_b).to(x.dtype)
        return a + (ops.linear(m, self.pool_fc2_w).float() + self.pool_fc2_b).to(x.dtype)

    def text_features(self, ids):
        c = self.c
        ids = torch.as_tensor(ids, device=self.tok.device).long()
        x = self.tok[ids] + self.t_pos[:ids.shape[1]]
        for b in self.t_blocks:
            x = b(x, c.eps, causal=False)
        x = F.layer_norm(x, (c.t_hidden,), self.fin_w, self.fin_b, c.eps)
        return (ops.linear(x[:, -1].contiguous(), self.head_w).float() + self.head_b).to(x.dtype)

    def embed_image(self, pixels):
        return F.normalize(self.image_features(pixels).float(), dim=-1)

    def embed_text(self, ids):
        return F.normalize(self.text_features(ids).float(), dim=-1)

    def pair_probability(self, pixels, ids):
        """``sigmoid(exp(logit_scale) * cos(image, text) + logit_bias)`` for every (image, text) pair."""
        return torch.sigmoid(self.embed_image(pixels) @ self.embed_text(ids).T * self.logit_scale.float().exp() + self.logit_bias.float())


def load_into(m: SiglipEmbedder, loader) -> None:
    """Checkpoint names of ``google/siglip-*`` / ``google/siglip2-*-patchNN-RES``."""
    def get(n):
        return loader.load_tensor(n, m.patch_w.dtype)

    def put(p, n):
        p.data.copy_(get(n).reshape(p.shape))
    v, t = "vision_model.", "text_model."
    for p, n in ((m.patch_w, v + "embeddings.patch_embedding.weight"), (m.patch_b, v + "embeddings.patch_embedding.bias"),
                 (m.v_pos, v + "embeddings.position_embedding.weight"), (m.post_w, v + "post_layernorm.weight"),
                 (m.post_b, v + "post_layernorm.bias"), (m.probe, v + "head.probe"), (m.pool_in_w, v + "head.attention.in_proj_weight"),
                 (m.pool_in_b, v + "head.attention.in_proj_bias"), (m.pool_out_w, v + "head.attention.out_proj.weight"),
                 (m.pool_out_b, v + "head.attention.out_proj.bias"), (m.pool_ln_w, v + "head.layernorm.weight"),
                 (m.pool_ln_b, v + "head.layernorm.bias"), (m.pool_fc1_w, v + "head.mlp.fc1.weight"), (m.pool_fc1_b, v + "head.mlp.fc1.bias"),
                 (m.pool_fc2_w, v + "head.mlp.fc2.weight"), (m.pool_fc2_b, v + "head.mlp.fc2.bias"),
                 (m.tok, t + "embeddings.token_embedding.weight"), (m.t_pos, t + "embeddings.position_embedding.weight"),
                 (m.fin_w, t + "final_layer_norm.weight"), (m.fin_b, t + "final_layer_norm.bias"), (m.head_w, t + "head.weight"),
                 (m.head_b, t + "head.bias"), (m.logit_scale, "logit_scale"), (m.logit_bias, "logit_bias")):
        put(p, n)
    load_blocks(m.v_blocks, "vision_model", get)
    load_blocks(m.t_blocks, "text_model", get)

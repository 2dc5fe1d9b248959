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

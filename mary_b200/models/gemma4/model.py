"""Gemma-4 text decoder over the flattened ragged batch and the paged KV cache.

Math: src/models/gemma/gemma4/{layers,decoder}.rs (restated step by step in ``mary_b200.oracle.gemma4``).
Weights are torch ``[out, in]``; q/k/v and gate/up are stored fused (``[q;k;v]``, ``[gate;up]``) so each block
issues four GEMMs.  Tensor parallelism shards q/k/v and gate/up by output rows (whole heads) and o/down by
input columns; ``tp`` supplies the reduction after the row-parallel GEMMs — an all-reduce, or, when ``tp.sp`` is set
(``parallel.sp.SequenceParallel``), a reduce-scatter from the GEMM epilogue followed by a fused sum + sandwich norms +
all-gather kernel with the residual stream sharded by token rows."""
from __future__ import annotations

import math

import torch
from torch import nn

from ... import ops
from ...ops import reference as ref
from .config import Gemma4TextConfig


class _NoTP:
    rank, size = 0, 1

    def row_linear(self, x, w, lora=None):
        y = ops.linear(x, w)
        return y if lora is None else y + lora(x)

    def reduce(self, x, residual=None):
        return x

    all_reduce = reduce


class Gemma4Layer(nn.Module):
    def __init__(self, cfg: Gemma4TextConfig, i: int, tp=None, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.cfg, self.i, self.tp = cfg, i, tp or _NoTP()
        H, D = cfg.hidden_size, cfg.layer_head_dim(i)
        self.D = D
        self.n_q = cfg.num_attention_heads // self.tp.size
        self.n_kv = max(cfg.layer_kv_heads(i) // self.tp.size, 1)
        # a KV-shared layer projects queries only and attends to the cache its source layer filled
        self.kv_source = cfg.kv_source(i)
        self.cache_layer = i if self.kv_source is None else self.kv_source
        F = cfg.layer_intermediate(i) // self.tp.size
        self.F = F
        kw = dict(dtype=dtype, device=device)
        P = lambda *s: nn.Parameter(torch.empty(*s, **kw), requires_grad=False)  # noqa: E731
        self.w_qkv = P((self.n_q + (2 * self.n_kv if self.kv_source is None else 0)) * D, H)
        self.w_o = P(H, self.n_q * D)
        self.w_gu = P(2 * F, H)
        self.w_down = P(H, F)
        self.q_norm, self.k_norm = P(D), P(D)
        self.ln_in, self.ln_post_attn, self.ln_pre_ffn, self.ln_post_ffn = P(H), P(H), P(H), P(H)
        self.layer_scalar = 1.0
        # 26B-A4B: routed experts beside the dense MLP (layers.rs:269-418).  Experts are split over the TP ranks by index.
        self.moe = bool(cfg.enable_moe_block)
        if self.moe:
            E, Fm = cfg.num_experts, cfg.moe_intermediate_size
            if E % self.tp.size:
                raise ValueError("num_experts must divide by the tensor-parallel size")
            self.e_local = E // self.tp.size
            self.router_scale, self.router_proj, self.per_expert_scale = P(H), P(E, H), P(E)
            self.ex_gate_up, self.ex_down = P(self.e_local, 2 * Fm, H), P(self.e_local, H, Fm)
            self.ln_post_ffn_1, self.ln_post_ffn_2, self.ln_pre_ffn_2 = P(H), P(H), P(H)
        # per-layer embeddings (layers.rs:476-518): a gated low-rank injection of a per-layer token signal
        self.ple = cfg.hidden_size_per_layer_input
        if self.ple:
            self.ple_gate, self.ple_proj, self.ln_post_ple = P(self.ple, H), P(H, self.ple), P(H)
        self.sliding = cfg.is_sliding(i)
        theta = cfg.rope_theta_local if self.sliding else cfg.rope_theta_global
        part = 1.0 if self.sliding else cfg.partial_rotary_factor_global
        self.register_buffer("inv_freq", ref.rope_inv_freq(D, theta, part, device), persistent=False)
        self.window = cfg.sliding_window if (self.sliding and cfg.apply_sliding_window) else 0
        self.lora = None  # {"qkv": LoraPair, ...} set by train.lora

    def _routed(self, h):
        """Routed expert sum of the MoE block, read from the residual BEFORE the dense MLP: weightless norm, learned scale and
        ``1/sqrt(H)``, softmax over all experts, top-k renormalised, then the per-expert output scale."""
        c = self.cfg
        r = ops.rmsnorm(h, self.router_scale * c.hidden_size ** -0.5, c.rms_norm_eps)     # the scale rides on the norm's gain
        idx, w = ops.router_topk(ops.linear_f32(r, self.router_proj), c.top_k_experts, "softmax", renorm=True)
        w = w * self.per_expert_scale.float()[idx.long()]
        x2 = ops.rmsnorm(h, self.ln_pre_ffn_2, c.rms_norm_eps)
        e0 = self.tp.rank * self.e_local
        y = ops.bf16_experts(x2, idx, w, self.ex_gate_up, self.ex_down, e0, "geglu")
        return self.tp.reduce(y) if self.tp.size > 1 else y

    def forward(self, x, h, meta, cache, next_norm, ple=None):
        """``x`` = normed input, ``h`` = residual stream.  Returns ``(x_next, h)`` where ``x_next`` is already
        normed by ``next_norm`` (the next layer's input norm or the final norm).  ``ple`` = this layer's ``[T, P]``
        per-layer input when the model has per-layer embeddings."""
        c, L = self.cfg, self.lora or {}
        qkv = ops.linear(x, self.w_qkv)
        if "qkv" in L:
            qkv = qkv + L["qkv"](x)
        ci = self.cache_layer
        q = ops.qk_norm_rope_append(qkv, self.n_q, self.n_kv if self.kv_source is None else 0, self.D, self.q_norm, self.k_norm, True,
                                    self.inv_freq, meta, cache.k[ci], cache.v[ci], c.rms_norm_eps)
        cp = getattr(self.tp, "cp", None)
        if cp is not None and self.kv_source is None:
            cp.share(cache.k[ci], cache.v[ci])           # context-parallel prefill: earlier chunks' K / V of this layer become local
        o = ops.paged_attention(q, cache.k[ci], cache.v[ci], meta, 1.0, self.window)
        o = o.reshape(o.shape[0], -1)
        sp = getattr(self.tp, "sp", None)
        if sp is not None and x.is_cuda and not L and not self.moe and not self.ple:
            # sequence-parallel residual: ``h`` holds this rank's token rows only.  The row-parallel GEMMs deliver their partial
            # rows to the owners from the epilogue; the owner sums, applies the sandwich norms and all-gathers the next input.
            sp.row_linear_rs(o, self.w_o)
            x = sp.reduce_add_rmsnorm(h, self.ln_pre_ffn, c.rms_norm_eps, w_post=self.ln_post_attn)
            m = ops.linear_glu(x, self.w_gu, "geglu")
            sp.row_linear_rs(m, self.w_down)
            x = sp.reduce_add_rmsnorm(h, next_norm, c.rms_norm_eps, w_post=self.ln_post_ffn, scalar=self.layer_scalar)
            return x, h
        a = self.tp.reduce(self.tp.row_linear(o, self.w_o, L.get("o")))
        x, h = ops.norm_add_norm(a, self.ln_post_attn, h, self.ln_pre_ffn, c.rms_norm_eps)
        if "gu" in L:
            m = ops.glu(ops.linear(x, self.w_gu) + L["gu"](x), "geglu")
        else:
            m = ops.linear_glu(x, self.w_gu, "geglu")
        d = self.tp.reduce(self.tp.row_linear(m, self.w_down, L.get("down")))
        if self.moe:
            d = ops.rmsnorm(d, self.ln_post_ffn_1, c.rms_norm_eps) + ops.rmsnorm(self._routed(h), self.ln_post_ffn_2, c.rms_norm_eps)
        if not self.ple:
            return ops.norm_add_norm(d, self.ln_post_ffn, h, next_norm, c.rms_norm_eps, self.layer_scalar)
        _, h = ops.norm_add_norm(d, self.ln_post_ffn, h, None, c.rms_norm_eps)
        g = ops.glu(torch.cat([ops.linear(h, self.ple_gate), ple.to(h.dtype)], -1), "geglu")
        return ops.norm_add_norm(ops.linear(g, self.ple_proj), self.ln_post_ple, h, next_norm, c.rms_norm_eps, self.layer_scalar)


class Gemma4Model(nn.Module):
    def __init__(self, cfg: Gemma4TextConfig, tp=None, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.cfg, self.tp, self.dtype = cfg, tp or _NoTP(), dtype
        kw = dict(dtype=dtype, device=device)
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw), requires_grad=False)
        self.layers = nn.ModuleList([Gemma4Layer(cfg, i, self.tp, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.empty(cfg.hidden_size, **kw), requires_grad=False)
        self.lm_head = None  # tied
        self.embed_scale = float(torch.tensor(math.sqrt(cfg.hidden_size), dtype=torch.float32))
        P = cfg.hidden_size_per_layer_input
        if P:                                          # per-layer embeddings (decoder.rs:114-175)
            n = cfg.num_hidden_layers
            self.ple_embed = nn.Parameter(torch.empty(cfg.ple_vocab, n * P, **kw), requires_grad=False)
            self.ple_model_proj = nn.Parameter(torch.empty(n * P, cfg.hidden_size, **kw), requires_grad=False)
            self.ple_proj_norm = nn.Parameter(torch.empty(P, **kw), requires_grad=False)

    def per_layer_inputs(self, ids, h0):
        """``[T, layers, P]``: (norm(proj(h0) / sqrt(H)) + embed_per_layer(ids) * sqrt(P)) / sqrt(2) — the token's own per-layer
        embedding mixed with a projection of its scaled input embedding ``h0``."""
        c = self.cfg
        P, n = c.hidden_size_per_layer_input, c.num_hidden_layers
        proj = ops.linear(h0, self.ple_model_proj) * (c.hidden_size ** -0.5)
        proj = ops.rmsnorm(proj.reshape(-1, P), self.ple_proj_norm, c.rms_norm_eps).reshape(-1, n, P)
        if ids is None:                                # rows given as embeddings (soft tokens) carry no per-layer embedding
            return proj
        tok = ops.embed(ids, self.ple_embed, float(torch.tensor(math.sqrt(P), dtype=torch.float32))).reshape(-1, n, P)
        return ((proj.float() + tok.float()) * (2.0 ** -0.5)).to(h0.dtype)

    # -- cache geometry for the runtime
    def kv_spec(self):
        c = self.cfg
        return dict(num_layers=c.num_hidden_layers,
                    kv_heads=[max(c.layer_kv_heads(i) // self.tp.size, 1) for i in range(c.num_hidden_layers)],
                    head_dim=[c.layer_head_dim(i) for i in range(c.num_hidden_layers)])

    def hidden(self, ids, meta, cache, soft=None):
        """Final-normed hidden states ``[T, H]`` of every row.  ``soft = (rows, embeds)`` replaces the embedding of the placeholder
        rows ``rows`` (a long tensor) by multimodal soft tokens ``embeds [len(rows), H]`` (unscaled, lm.rs:212-311); those rows take
        the pad token's per-layer embedding."""
        h = ops.embed(ids, self.embed, self.embed_scale)
        if soft is not None:
            rows, emb = soft
            h = h.index_copy(0, rows, emb.to(h.dtype))
            ids = ids.clone().index_fill_(0, rows, 0)
        ple = self.per_layer_inputs(ids, h) if self.cfg.hidden_size_per_layer_input else None
        x = ops.rmsnorm(h, self.layers[0].ln_in, self.cfg.rms_norm_eps)
        sp = getattr(self.tp, "sp", None)
        plain = not (self.cfg.enable_moe_block or self.cfg.hidden_size_per_layer_input)
        if sp is not None and h.is_cuda and plain and not any(l.lora for l in self.layers):
            h = sp.residual_slice(h)                 # from here on every rank carries only its own rows of the residual
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].ln_in if i + 1 < n else self.norm
            x, h = layer(x, h, meta, cache, nxt, None if ple is None else ple[:, i].contiguous())
        return x

    def head_weight(self):
        return self.embed if self.lm_head is None else self.lm_head

    def logits(self, x):
        return ref.softcap(ops.linear(x, self.head_weight()).float(), self.cfg.final_logit_softcapping)

    def forward(self, ids, meta, cache, rows=None, soft=None):
        """Logits (f32, soft-capped) of ``rows`` (all rows when ``None``)."""
        x = self.hidden(ids, meta, cache, soft)
        if rows is not None:
            x = x[rows]
        return self.logits(x)

    def greedy(self, ids, meta, cache, rows, soft=None):
        x = self.hidden(ids, meta, cache, soft)[rows]
        tok, _ = ops.lm_head_argmax(x, self.head_weight(), self.cfg.final_logit_softcapping)
        return tok

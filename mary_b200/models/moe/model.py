"""Sparse-MoE decoder (GQA or MLA attention, NVFP4 routed experts, shared expert, MTP draft layers) over the
flattened ragged batch and the paged cache.

Layer: ``h += attn(rms(h)); h += ffn(rms(h))``.  Routed experts live in :class:`NVFP4Experts`; attention, router,
shared expert, dense FFN and head are bf16.  Parallel layout (``par``): attention heads and dense/shared FFN columns are
sharded over the group (tensor parallel), routed experts are sharded by expert index (expert parallel); both produce
partial sums of the hidden state that one reduction per block combines."""
from __future__ import annotations

import os

import torch
from torch import nn

from ... import ops
from ...ops import reference as ref
from ...ops.moe import NVFP4Experts, experts_forward
from ...utils import flags
from .config import MoEConfig


class NoParallel:
    rank, size = 0, 1
    tp_rank, tp_size, ep_rank, ep_size, ep_mode = 0, 1, 0, 1, "replicated"

    def reduce(self, partial, residual=None):
        """Sum the partial hidden states over the group.  Returns a tensor every rank holds."""
        return partial

    def row_linear(self, x, w):
        return ops.linear(x, w)


def _P(*shape, dtype, device):
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device), requires_grad=False)


class GQAAttention(nn.Module):
    def __init__(self, c: MoEConfig, layer_idx: int, par, dtype, device):
        super().__init__()
        self.c, self.li, self.par = c, layer_idx, par
        self.n_q = c.num_attention_heads // par.tp_size
        self.n_kv = max(c.num_key_value_heads // par.tp_size, 1)
        D = c.head_dim
        self.w_qkv = _P((self.n_q + 2 * self.n_kv) * D, c.hidden_size, dtype=dtype, device=device)
        self.w_o = _P(c.hidden_size, self.n_q * D, dtype=dtype, device=device)
        self.register_buffer("inv_freq", ref.rope_inv_freq(D, c.rope_theta, 1.0, device), persistent=False)

    def forward(self, x, meta, cache):
        c = self.c
        qkv = ops.linear(x, self.w_qkv)
        q = ops.qk_norm_rope_append(qkv, self.n_q, self.n_kv, c.head_dim, None, None, False, self.inv_freq, meta,
                                    cache.k[self.li], cache.v[self.li], c.rms_norm_eps)
        o = ops.paged_attention(q, cache.k[self.li], cache.v[self.li], meta, c.attn_scale)
        return self.par.row_linear(o.reshape(o.shape[0], -1), self.w_o)


class MLAAttention(nn.Module):
    """Latent attention with absorbed W_UK / W_UV and a latent cache row ``[c_kv (512) | k_rope (64)]``."""

    def __init__(self, c: MoEConfig, layer_idx: int, par, dtype, device):
        super().__init__()
        assert c.kv_lora_rank == 512 and c.qk_rope_head_dim == 64 and c.qk_nope_head_dim == 128 and c.v_head_dim == 128
        self.c, self.li, self.par = c, layer_idx, par
        self.H = c.num_attention_heads // par.tp_size
        kw = dict(dtype=dtype, device=device)
        self.w_qa_kva = _P(c.q_lora_rank + 576, c.hidden_size, **kw)       # replicated
        self.qa_norm = _P(c.q_lora_rank, **kw)
        self.kv_norm = _P(512, **kw)
        self.w_qb = _P(self.H * 192, c.q_lora_rank, **kw)                  # heads sharded
        self.w_uk = _P(self.H, 512, 128, **kw)                             # q_lat = W_UK q_nope
        self.w_uv = _P(self.H, 128, 512, **kw)                             # o = W_UV o_lat
        self.w_o = _P(c.hidden_size, self.H * 128, **kw)
        inv = None if c.use_nope else ref.rope_inv_freq(64, c.rope_theta, 1.0, device)
        self.register_buffer("inv_freq", inv, persistent=False)

    PREFILL_MIN_ROWS = 48     # mean query tokens per sequence from which the expanded (non-absorbed) prefill path is used

    def _prefill_expanded(self, qb, meta, cache):
        """Prefill with the keys and values EXPANDED from the latent rows (per-head K = [W_UK^T c_kv | k_rope], V = W_UV c_kv)
        and ordinary causal attention with 192-wide keys and 128-wide values: a third of the arithmetic of attending in the
        576 / 512-wide latent space, which is what long query blocks are bound by.  The scores are identical
        (q_nope . W_UK^T c_kv = W_UK q_nope . c_kv); decode keeps the absorbed form, where the cache stream is the bound."""
        T, H = qb.shape[0], self.H
        lat = cache.k[self.li]                                              # [pages, page, 576]
        pick, meta2 = meta.repage(64)                                       # the same for every layer of this step
        rows = lat[pick].view(-1, 64, 576)                                  # context of every sequence in 64-token pages
        P, ps = rows.shape[0], 64
        if getattr(self, "_w_uk_t", None) is None:
            self._w_uk_t = self.w_uk.permute(0, 2, 1).reshape(H * 128, 512).contiguous()      # k_nope[h, n] = sum_k c_kv[k] W_UK[h, k, n]
        if qb.is_cuda:
            # the rope dims of q rotated in place, K and V written straight into their paged layout: no concatenation copies
            q = (ops.mla_q_rope_inplace(qb, self.inv_freq, meta, H) if self.inv_freq is not None else qb).view(T, H, 192)
            k, v = ops.mla_expand_kv(rows.view(P * ps, 576), self._w_uk_t, self.w_uv.reshape(H * 128, 512), H)
            k, v = k.view(P, ps, H, 192), v.view(P, ps, H, 128)
        else:
            q = qb.view(T, H, 192)
            if self.inv_freq is not None:
                q = torch.cat([q[..., :128], ref.rope(q[..., 128:], meta.positions, self.inv_freq).to(q.dtype)], -1)
            ckv = rows[..., :512].reshape(P * ps, 512)
            k_nope = ops.linear(ckv, self._w_uk_t).view(P, ps, H, 128)
            v = ops.linear(ckv, self.w_uv.reshape(H * 128, 512)).view(P, ps, H, 128)
            k = torch.cat([k_nope, rows[..., 512:].unsqueeze(2).expand(P, ps, H, 64)], -1).contiguous()
        o = ops.paged_attention(q.contiguous(), k, v, meta2, self.c.attn_scale)
        return self.par.row_linear(o.reshape(T, H * 128), self.w_o)

    def forward(self, x, meta, cache):
        c = self.c
        qakv = ops.linear(x, self.w_qa_kva)
        qa = ops.mla_prep(qakv, c.q_lora_rank, self.qa_norm, self.kv_norm, self.inv_freq, meta, cache.k[self.li], 1e-6)
        cp = getattr(self.par, "cp", None)
        if cp is not None:
            cp.share(cache.k[self.li], None)       # context-parallel prefill: the earlier chunks' latent rows become local
        qb = ops.linear(qa, self.w_qb)
        if meta.kv_lens_host is not None and meta.num_tokens >= self.PREFILL_MIN_ROWS * meta.num_seqs:
            return self._prefill_expanded(qb, meta, cache)
        q_full = ops.mla_absorb_q(qb, self.w_uk, self.inv_freq, meta, self.H)
        o_lat = ops.mla_attention(q_full, cache.k[self.li], meta, c.attn_scale)
        o = ops.mla_unabsorb_o(o_lat, self.w_uv, self.H)
        return self.par.row_linear(o, self.w_o)


class DenseFFN(nn.Module):
    def __init__(self, H, F, par, act, dtype, device):
        super().__init__()
        self.par, self.act = par, act
        Fl = F // par.tp_size
        self.w_gu = _P(2 * Fl, H, dtype=dtype, device=device)
        self.w_down = _P(H, Fl, dtype=dtype, device=device)

    def forward(self, x):
        return self.par.row_linear(ops.linear_glu(x, self.w_gu, self.act), self.w_down)


class MoEFFN(nn.Module):
    def __init__(self, c: MoEConfig, par, dtype, device):
        super().__init__()
        self.c, self.par = c, par
        E = c.n_routed_experts
        self.e_local = E // par.ep_size
        self.e0 = par.ep_rank * self.e_local
        self.ep_layer = None                             # parallel.ep.EPLayer in all-to-all mode
        self.w_router = _P(E, c.hidden_size, dtype=dtype, device=device)
        self.router_bias = nn.Parameter(torch.zeros(E, dtype=torch.float32, device=device), requires_grad=False) \
            if c.router == "sigmoid" else None
        # the shared expert is either a bf16 dense FFN (tensor parallel) or, with `shared_expert_nvfp4`, one more NVFP4
        # expert appended behind the local routed ones (index e_local) that every token visits with weight 1
        self.shared_in_experts = bool(c.shared_expert_nvfp4 and c.n_shared_experts == 1)
        self.shared = DenseFFN(c.hidden_size, c.moe_intermediate_size * c.n_shared_experts, par, c.act, dtype, device) \
            if (c.n_shared_experts and not self.shared_in_experts) else None
        self.experts: NVFP4Experts | None = None        # set by the loader / random init
        self._tail = {}

    def route(self, x):
        c = self.c
        logits = ops.linear_f32(x, self.w_router)
        return ops.router_topk(logits, c.num_experts_per_tok, c.router, self.router_bias, c.n_group, c.topk_group,
                               c.routed_scaling_factor, c.norm_topk_prob)

    FUSED_MAX_ROWS = 512      # decode-sized batches take the four-launch pipeline; larger ones the planned path with 128-row tiles

    def fused_ctx(self, x):
        """The four-launch expert pipeline (``parallel.ep_fused``) for this batch, or ``None`` when the batch is not decode-sized,
        lives on the CPU, or ``MARY_MOE_FUSED=0`` asks for the planned path."""
        if not x.is_cuda or self.experts is None or not flags.get("MARY_MOE_FUSED"):
            return None
        from ...parallel import ep_fused
        c, par, T = self.c, self.par, x.shape[0]
        E, k = c.n_routed_experts, c.num_experts_per_tok
        if E > 512 or k * 8 > 256 or c.hidden_size * 4 > 48 * 1024:
            return None
        store = par.__dict__.setdefault("_fused_moe", {})
        a2a = par.ep_mode == "a2a" and par.ep_size > 1
        if a2a:
            cap = getattr(par, "ep_decode_cap", None)
            if cap is None or T > cap or (par.ep_size * cap * (k + 1) + 31) // 32 + self.e_local + 1 > ep_fused.MAX_TILES:
                return None
            if ("a2a", cap) not in store:        # collective: every rank reaches its first MoE layer with the same shapes
                store[("a2a", cap)] = ep_fused.distributed(par.ep_rank, par.ep_size, E, c.hidden_size, c.moe_intermediate_size, cap, k,
                                                           self.shared_in_experts, x.device)
            return store[("a2a", cap)]
        if T > self.FUSED_MAX_ROWS:
            return None
        fits = [v for (kind, cap), v in store.items() if kind == "local" and cap >= T]
        if fits:
            return min(fits, key=lambda v: v.t_cap)
        cap = (T + 31) // 32 * 32
        # worst case of token tiles: every entry's tile plus one ragged tile per expert
        if (T * (k + 1) + 31) // 32 + self.e_local + 1 > ep_fused.MAX_TILES:
            return None
        store[("local", cap)] = ep_fused.FusedMoE(par.ep_rank, par.ep_size, E, c.hidden_size, c.moe_intermediate_size, cap, k,
                                                  self.shared_in_experts, x.device, True)
        return store[("local", cap)]

    def forward_fused(self, fm, x, h, next_norm):
        """``h += ffn(x)`` and the next block's normed input through the four-launch pipeline.  Returns ``(x_next | None, h)``."""
        c, par = self.c, self.par
        logits = ops.linear_f32(x, self.w_router)
        router = dict(mode=c.router, bias=self.router_bias, n_group=c.n_group, topk_group=c.topk_group, scale=c.routed_scaling_factor,
                      renorm=c.norm_topk_prob)
        add = ops.linear(ops.linear_glu(x, self.shared.w_gu, c.act), self.shared.w_down) if self.shared is not None else None
        if fm.local_only and par.ep_size > 1:
            # replicated tokens: this rank's experts give a partial sum that the group reduces before it joins the residual
            f = par.reduce(fm.forward(x, logits, router, self.experts, add=add))
            if next_norm is None:
                return None, (h.float() + f.float()).to(h.dtype)
            return ops.add_rmsnorm(f, h, next_norm, c.rms_norm_eps)
        return fm.forward(x, logits, router, self.experts, add=add, res=h, w_norm=next_norm, eps=c.rms_norm_eps)

    def forward(self, x):
        idx, w = self.route(x)
        if self.par.ep_mode == "a2a" and self.par.ep_size > 1:
            # tokens are local: routed experts through the all-to-all (global expert ids), shared expert computed at home
            cap = getattr(self.par, "ep_decode_cap", None)
            if cap is None:
                raise RuntimeError("all-to-all expert parallelism needs par.ep_decode_cap (rows per rank of the decode-sized slabs)")
            big = x.shape[0] > cap
            if big:
                # prefill-sized batches get slabs of their own (and 128-row token tiles) next to the decode-sized ones
                if getattr(self, "ep_layer_big", None) is None:
                    self.ep_layer_big = self.par.ep_factory(self.experts, self.c, self.par.ep_prefill_cap, 128)
            elif self.ep_layer is None:
                self.ep_layer = self.par.ep_factory(self.experts, self.c)
            shared = ops.linear(ops.linear_glu(x, self.shared.w_gu, self.c.act), self.shared.w_down) if self.shared is not None else None
            # an NVFP4 shared expert sits behind the local routed ones on every rank; the EP layer serves it in the same launches
            return (self.ep_layer_big if big else self.ep_layer).forward(x, idx, w, shared)
        if self.par.ep_size > 1:              # keep the entries of the local experts, renumbered from zero
            local = (idx >= self.e0) & (idx < self.e0 + self.e_local)
            idx = torch.where(local, idx - self.e0, torch.full_like(idx, -1))
        if self.shared_in_experts:
            T = x.shape[0]
            tail = self._tail.get((T, x.device))
            if tail is None:
                # with replicated tokens every rank holds the shared expert; rank r serves the tokens t = r (mod size)
                mine = (torch.arange(T, device=x.device) % self.par.ep_size) == self.par.ep_rank
                sh = torch.where(mine, self.e_local, -1).to(torch.int32)[:, None]
                tail = (sh, torch.ones(T, 1, dtype=torch.float32, device=x.device))
                self._tail[(T, x.device)] = tail
            idx = torch.cat([idx.to(torch.int32), tail[0]], 1)
            w = torch.cat([w.float(), tail[1]], 1)
            return experts_forward(x, idx, w, self.experts, None)
        # the shared expert's partial sum rides along in the un-permute (one pass over the hidden state)
        shared = ops.linear(ops.linear_glu(x, self.shared.w_gu, self.c.act), self.shared.w_down) if self.shared is not None else None
        return experts_forward(x, idx, w, self.experts, shared)


class MoELayer(nn.Module):
    def __init__(self, c: MoEConfig, i: int, par, dtype, device, cache_index: int | None = None):
        super().__init__()
        self.c, self.par = c, par
        li = i if cache_index is None else cache_index
        self.attn = (MLAAttention if c.attention == "mla" else GQAAttention)(c, li, par, dtype, device)
        self.dense = c.is_dense(i) and cache_index is None
        self.ffn = DenseFFN(c.hidden_size, c.dense_intermediate_size, par, c.act, dtype, device) if self.dense \
            else MoEFFN(c, par, dtype, device)
        self.ln_attn = _P(c.hidden_size, dtype=dtype, device=device)
        self.ln_ffn = _P(c.hidden_size, dtype=dtype, device=device)

    def forward(self, x, h, meta, cache, next_norm):
        """``x`` normed input, ``h`` residual.  Returns ``(next normed x, h)``."""
        a = self.par.reduce(self.attn(x, meta, cache))
        x, h = ops.add_rmsnorm(a, h, self.ln_ffn, self.c.rms_norm_eps)
        if not self.dense:
            fm = self.ffn.fused_ctx(x)
            if fm is not None:
                return self.ffn.forward_fused(fm, x, h, next_norm)
        f = self.par.reduce(self.ffn(x))
        if next_norm is None:
            return None, (h.float() + f.float()).to(h.dtype)
        return ops.add_rmsnorm(f, h, next_norm, self.c.rms_norm_eps)


class MTPLayer(nn.Module):
    """Multi-token-prediction draft layer: ``x = proj([rms(h_prev) ; rms(embed(next token))])`` (hidden first, as in
    src/models/inkling/mtp.rs:108-244), one decoder block with its own cache rows, then the shared head."""

    def __init__(self, c: MoEConfig, d: int, par, dtype, device):
        super().__init__()
        self.c = c
        H = c.hidden_size
        self.h_norm = _P(H, dtype=dtype, device=device)
        self.e_norm = _P(H, dtype=dtype, device=device)
        self.proj = _P(H, 2 * H, dtype=dtype, device=device)
        self.block = MoELayer(c, c.num_hidden_layers + d, par, dtype, device, cache_index=c.num_hidden_layers + d)
        self.out_norm = _P(H, dtype=dtype, device=device)

    def forward(self, h_prev, tok_emb, meta, cache):
        c = self.c
        x = torch.cat([ops.rmsnorm(h_prev, self.h_norm, c.rms_norm_eps), ops.rmsnorm(tok_emb, self.e_norm, c.rms_norm_eps)], -1)
        h = ops.linear(x, self.proj)
        x = ops.rmsnorm(h, self.block.ln_attn, c.rms_norm_eps)
        _, h = self.block(x, h, meta, cache, None)
        return h


class MoEDecoder(nn.Module):
    def __init__(self, c: MoEConfig, par=None, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg, self.par, self.dtype = c, par or NoParallel(), dtype
        kw = dict(dtype=dtype, device=device)
        self.embed = _P(c.vocab_size, c.hidden_size, **kw)
        self.layers = nn.ModuleList([MoELayer(c, i, self.par, dtype, device) for i in range(c.num_hidden_layers)])
        self.norm = _P(c.hidden_size, **kw)
        # vocabulary-parallel head: every rank keeps V / tp rows of the head and the ranks merge (value, index) candidates
        self.vocab_parallel = bool(getattr(self.par, "vocab_parallel", False)) and self.par.tp_size > 1 \
            and c.vocab_size % self.par.tp_size == 0
        head_rows = c.vocab_size // self.par.tp_size if self.vocab_parallel else c.vocab_size
        self.lm_head = None if c.tie_word_embeddings else _P(head_rows, c.hidden_size, **kw)
        self._vhead = None
        self.mtp = nn.ModuleList([MTPLayer(c, d, self.par, dtype, device) for d in range(c.num_mtp_layers)])

    def kv_spec(self):
        c = self.cfg
        n = c.num_hidden_layers + c.num_mtp_layers
        if c.attention == "mla":
            return dict(num_layers=n, kv_heads=1, head_dim=576, latent_dim=576)
        return dict(num_layers=n, kv_heads=max(c.num_key_value_heads // self.par.tp_size, 1), head_dim=c.head_dim)

    def head_weight(self):
        return self.embed if self.lm_head is None else self.lm_head

    def head_argmax(self, x):
        """Greedy token of every row of ``x`` (normed hidden states)."""
        if not self.vocab_parallel:
            return ops.lm_head_argmax(x, self.head_weight())[0]
        if self._vhead is None:
            from ...parallel.vocab import VocabParallelHead
            par = self.par
            w = self.lm_head if self.lm_head is not None else VocabParallelHead.shard(self.embed, par.tp_rank, par.tp_size)
            fused = getattr(par, "mode", "") == "fused" and getattr(par, "symm", None) is not None and w.is_cuda
            self._vhead = VocabParallelHead(w, par.tp_rank, par.tp_size, symm=par.symm if fused else None, group=getattr(par, "group", None))
        return self._vhead.argmax(x)[0]

    def trunk(self, ids, meta, cache):
        """Residual stream after the last layer (before the final norm), every row."""
        c = self.cfg
        h = ops.embed(ids, self.embed)
        x = ops.rmsnorm(h, self.layers[0].ln_attn, c.rms_norm_eps)
        n = len(self.layers)
        from ...utils.trace import nvtx_range
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].ln_attn if i + 1 < n else None
            with nvtx_range(f"layer {i}"):
                x, h = layer(x, h, meta, cache, nxt)
        return h

    def trunk_range(self, ids_or_h, lo: int, hi: int, meta, cache):
        """Layers ``[lo, hi)`` only (a pipeline stage): the first stage takes token ids, later stages take the residual
        stream that the previous stage produced.  Returns the residual stream after layer ``hi - 1``."""
        c = self.cfg
        h = ops.embed(ids_or_h, self.embed) if lo == 0 else ids_or_h
        x = ops.rmsnorm(h, self.layers[lo].ln_attn, c.rms_norm_eps)
        for i in range(lo, hi):
            nxt = self.layers[i + 1].ln_attn if i + 1 < hi else None
            x, h = self.layers[i](x, h, meta, cache, nxt)
        return h

    def hidden(self, ids, meta, cache):
        return ops.rmsnorm(self.trunk(ids, meta, cache), self.norm, self.cfg.rms_norm_eps)

    def forward(self, ids, meta, cache, rows=None):
        x = self.hidden(ids, meta, cache)
        if rows is not None:
            x = x[rows]
        if self.vocab_parallel:                       # full logits are a debugging aid here: gather the shards
            import torch.distributed as dist
            w = self.lm_head if self.lm_head is not None else self.embed.chunk(self.par.tp_size, 0)[self.par.tp_rank]
            loc = ops.linear(x, w).float().contiguous()
            parts = [torch.empty_like(loc) for _ in range(self.par.tp_size)]
            dist.all_gather(parts, loc, group=getattr(self.par, "group", None))
            return torch.cat(parts, -1)
        return ops.linear(x, self.head_weight()).float()

    def greedy(self, ids, meta, cache, rows):
        return self.head_argmax(self.hidden(ids, meta, cache)[rows])

    # -- speculative decoding -------------------------------------------------
    def _head_rows(self, h, norm, rows):
        """Arg-max token of the rows ``rows`` of ``h`` (None: every row; an empty index: no head at all).  A prompt chunk of
        thousands of rows needs the vocabulary projection for its last row only."""
        if rows is not None:
            if rows.numel() == 0:
                return torch.empty(0, dtype=torch.int64, device=h.device)
            h = h[rows]
        return self.head_argmax(ops.rmsnorm(h, norm, self.cfg.rms_norm_eps))

    def verify(self, ids, meta, cache, rows=None):
        """One forward over the fed rows.  Returns ``(arg-max token of the rows ``rows`` (default all), trunk hidden of every row)``."""
        h = self.trunk(ids, meta, cache)
        return self._head_rows(h, self.norm, rows), h

    def draft(self, d: int, h_prev, next_ids, meta, cache, rows=None):
        """Draft head ``d``: hidden of the rows + the token that follows each row -> ``(draft token of ``rows``, hidden of every row)``."""
        emb = ops.embed(next_ids, self.embed)
        h = self.mtp[min(d, len(self.mtp) - 1)](h_prev, emb, meta, cache)
        return self._head_rows(h, self.mtp[min(d, len(self.mtp) - 1)].out_norm, rows), h


def init_random_(model: MoEDecoder, seed: int = 0, std: float = 0.02, expert_slabs: int | None = None) -> None:
    """Random-init in place on the model's device: ``normal(0, std)`` matrices, unit gains, NVFP4 experts quantised from
    ``normal(0, std)``.  ``expert_slabs`` < number of MoE layers makes layers share physical expert storage cyclically
    (a memory-fitting device for benchmarks on fewer GPUs than the model needs; every layer still streams a full slab)."""
    c = model.cfg
    dev = model.embed.device
    g = torch.Generator(device=dev).manual_seed(seed)
    for n, p in model.named_parameters():
        if p.dim() == 1:
            p.data.fill_(0.0 if "router_bias" in n else 1.0)
        else:
            p.data.normal_(0.0, std, generator=g)
    moes = [m for m in model.modules() if isinstance(m, MoEFFN)]
    slabs: list[NVFP4Experts] = []
    n_slabs = len(moes) if expert_slabs is None else max(1, min(expert_slabs, len(moes)))
    for i, m in enumerate(moes):
        if i < n_slabs:
            slabs.append(NVFP4Experts.random(m.e_local + (1 if m.shared_in_experts else 0), c.hidden_size, c.moe_intermediate_size,
                                             dev, std, seed + 1 + i, c.act))
        m.experts = slabs[i % n_slabs]

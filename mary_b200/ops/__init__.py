"""Op entry points.  A CUDA tensor runs the hand-written sm_100a kernel (``ops.cuda``; a missing kernel
library is an error, never a silent fallback); a CPU tensor runs the PyTorch reference (``ops.reference``),
which is also the oracle the kernels are tested against."""
from __future__ import annotations

import torch

from . import reference as ref


def _cuda(x) -> bool:
    return isinstance(x, torch.Tensor) and x.is_cuda


def _k():
    from . import cuda
    return cuda


def rmsnorm(x, weight=None, eps=1e-6):
    return _k().rmsnorm(x, weight, eps) if _cuda(x) else ref.rmsnorm(x, weight, eps)


def add_rmsnorm(x, residual, weight, eps=1e-6):
    return _k().add_rmsnorm(x, residual, weight, eps) if _cuda(x) else ref.add_rmsnorm(x, residual, weight, eps)


def norm_add_norm(a, w_post, h, w_next, eps=1e-6, scalar: float = 1.0):
    """Gemma sandwich step: ``h' = (h + rms(a, w_post)) * scalar``; ``x = rms(h', w_next)``.  Returns ``(x, h')``;
    ``w_next=None`` skips the second norm and returns ``(None, h')``."""
    if _cuda(a):
        return _k().norm_add_norm(a, w_post, h, w_next, eps, scalar)
    hn = (h.float() + ref.rmsnorm(a, w_post, eps).float()) * scalar
    hn = hn.to(h.dtype)
    return (ref.rmsnorm(hn, w_next, eps) if w_next is not None else None), hn


def linear(x, w, bias=None):
    return _k().linear(x, w, bias) if _cuda(x) else ref.linear(x, w, bias)


def linear_f32(x, w):
    """``x @ w^T`` with an f32 result (router logits, row-parallel partial sums)."""
    if _cuda(x):
        return _k().linear_f32(x, w)
    return ref.linear(x.float(), w.float())


def qk_norm_rope_append(qkv, n_q, n_kv, head_dim, q_norm, k_norm, v_norm: bool, inv_freq, meta, kcache, vcache, eps):
    """Split ``qkv[T, (n_q+2 n_kv) D]``; per-head RMSNorm on q and k (learned gains) and optionally a weightless
    norm on v; split-half RoPE on q and k at ``meta.positions``; append k, v to the paged cache.
    Returns ``q[T, n_q, D]``."""
    if _is_q8(kcache):
        # 8-bit cache: norm and rotate into a bf16 staging row per token (the same kernel, slots 0..T-1), then quantise the rows
        # into their pages
        from types import SimpleNamespace
        T = qkv.shape[0]
        stage_k = torch.empty(T, 1, n_kv, head_dim, dtype=qkv.dtype, device=qkv.device)
        stage_v = torch.empty_like(stage_k)
        flat = SimpleNamespace(positions=meta.positions, slot_mapping=torch.arange(T, dtype=torch.int64, device=qkv.device))
        q = qk_norm_rope_append(qkv, n_q, n_kv, head_dim, q_norm, k_norm, v_norm, inv_freq, flat, stage_k, stage_v, eps)
        kv_quant_append(stage_k[:, 0], meta.slot_mapping, kcache)
        kv_quant_append(stage_v[:, 0], meta.slot_mapping, vcache)
        return q
    if _cuda(qkv):
        return _k().qk_norm_rope_append(qkv, n_q, n_kv, head_dim, q_norm, k_norm, v_norm, inv_freq, meta, kcache, vcache, eps)
    T = qkv.shape[0]
    q, k, v = qkv.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
    q, k, v = q.reshape(T, n_q, head_dim), k.reshape(T, n_kv, head_dim), v.reshape(T, n_kv, head_dim)
    if n_kv == 0:                                  # queries only (a layer that reads another layer's cache)
        q = ref.rmsnorm(q, q_norm, eps) if q_norm is not None else q
        return ref.rope(q, meta.positions, inv_freq) if inv_freq is not None else q
    if q_norm is not None:
        q = ref.rmsnorm(q, q_norm, eps)
    if k_norm is not None:
        k = ref.rmsnorm(k, k_norm, eps)
    if v_norm:
        v = ref.rmsnorm(v, None, eps)
    if inv_freq is not None:
        q, k = ref.rope(q, meta.positions, inv_freq), ref.rope(k, meta.positions, inv_freq)
    ref.kv_append(k, v, kcache, vcache, meta.slot_mapping)
    return q


def _is_q8(cache) -> bool:
    from ..runtime.kv_cache import Q8Pages
    return isinstance(cache, Q8Pages)


def kv_quant_append(rows, slots, pages) -> None:
    """Quantise ``rows [T, Hkv, D]`` to 8-bit codes with a (scale, zero) pair per (token, head) and store them at the flat cache
    slots ``slots [T]`` of ``pages`` (a ``runtime.kv_cache.Q8Pages``)."""
    if _cuda(rows):
        return _k().kv_quant_append(rows, slots, pages)
    pages.append(rows, slots)


def paged_attention(q, kcache, vcache, meta, scale, window=0, softcap=0.0, rel_bias=None):
    """``rel_bias [T, Hq, extent]`` (f32): an additive bias on the scaled score of the key ``dist`` positions back, for ``dist < extent``.
    With an 8-bit cache, decode-shaped batches run the dequantising kernel; everything else dequantises the pages of the batch."""
    if _is_q8(kcache):
        if _cuda(q) and rel_bias is None and _k().decode_q8_supported(q, kcache, meta):
            return _k().paged_attention_decode_q8(q, kcache, vcache, meta, scale, window, softcap)
        import dataclasses
        need = (meta.kv_len.long() + meta.page_size - 1) // meta.page_size
        cols = torch.arange(meta.page_table.shape[1], device=need.device)[None]
        used = (cols < need[:, None])
        pages = torch.unique(meta.page_table[used].long())
        remap = torch.zeros(kcache.shape[0], dtype=torch.int32, device=pages.device)
        remap[pages] = torch.arange(pages.numel(), dtype=torch.int32, device=pages.device)
        m2 = dataclasses.replace(meta, page_table=torch.where(used, remap[meta.page_table.long()], 0).to(torch.int32).contiguous())
        return paged_attention(q, kcache.dequantize(pages, q.dtype), vcache.dequantize(pages, q.dtype), m2, scale, window, softcap, rel_bias)
    if _cuda(q):
        return _k().paged_attention(q, kcache, vcache, meta, scale, window, softcap, rel_bias=rel_bias)
    return ref.paged_attention(q, kcache, vcache, meta, scale, window, softcap, rel_bias=rel_bias)


def mla_attention(q, cache, meta, scale):
    """Latent attention: ``q[T, Hq, 576]`` against the latent cache ``[pages, page, 576]`` (keys = all 576 dims,
    values = the first 512).  Returns ``[T, Hq, 512]``."""
    if _cuda(q):
        return _k().mla_attention(q, cache, meta, scale)
    return ref.paged_attention(q, cache, cache, meta, scale, dv=512)


def mla_expand_kv(rows, w_uk_t, w_uv, H):
    """GPU only (the host path concatenates): see ``ops.cuda.mla_expand_kv``."""
    return _k().mla_expand_kv(rows, w_uk_t, w_uv, H)


def mla_q_rope_inplace(qb, inv_freq, meta, H):
    return _k().mla_q_rope_inplace(qb, inv_freq, meta, H)


def mla_prep(qakv, q_lora, w_qa, w_kv, inv_freq, meta, cache, eps):
    """Norm the q_a part, norm the latent, rotate the carried rope dims and append ``[c_kv | k_rope]`` to the cache."""
    if _cuda(qakv):
        return _k().mla_prep(qakv, q_lora, w_qa, w_kv, inv_freq, meta, cache, eps)
    qa = ref.rmsnorm(qakv[:, :q_lora], w_qa, eps)
    ckv = ref.rmsnorm(qakv[:, q_lora:q_lora + 512], w_kv, eps)
    kr = qakv[:, q_lora + 512:q_lora + 576]
    if inv_freq is not None:
        kr = ref.rope(kr[:, None, :], meta.positions, inv_freq)[:, 0]
    cache.view(-1, 576)[meta.slot_mapping] = torch.cat([ckv, kr], -1).to(cache.dtype)
    return qa


def mla_absorb_q(qb, w_uk, inv_freq, meta, H):
    if _cuda(qb):
        return _k().mla_absorb_q(qb, w_uk, inv_freq, meta, H)
    T = qb.shape[0]
    q = qb.view(T, H, 192)
    lat = torch.einsum("thd,hnd->thn", q[..., :128].float(), w_uk.float()).to(qb.dtype)
    qr = q[..., 128:]
    if inv_freq is not None:
        qr = ref.rope(qr, meta.positions, inv_freq)
    return torch.cat([lat, qr], -1)


def mla_unabsorb_o(o_lat, w_uv, H):
    if _cuda(o_lat):
        return _k().mla_unabsorb_o(o_lat, w_uv, H)
    return torch.einsum("thk,hnk->thn", o_lat.float(), w_uv.float()).to(o_lat.dtype).reshape(o_lat.shape[0], H * 128)


def glu(gate_up, act: str = "geglu"):
    """``act(gate) * up`` over ``gate_up[T, 2F] = [gate | up]``."""
    if _cuda(gate_up):
        return _k().glu(gate_up, act)
    F = gate_up.shape[-1] // 2
    return {"geglu": ref.geglu, "swiglu": ref.swiglu, "situ": ref.situ}[act](gate_up[..., :F], gate_up[..., F:])


def linear_glu(x, w_gu, act: str = "geglu"):
    """``act(x @ gate^T) * (x @ up^T)`` with ``w_gu = [gate; up]``; fused into the GEMM epilogue on the GPU."""
    if _cuda(x):
        return _k().linear_glu(x, w_gu, act)
    return glu(ref.linear(x, w_gu), act)


def embed(ids, table, scale=1.0):
    return _k().embed(ids, table, scale) if _cuda(table) else ref.embed(ids, table, scale)


def lm_head_argmax(h, table, softcap=0.0, vocab_limit: int | None = None):
    """``argmax(softcap(h @ table^T))`` per row (first maximum wins) and the max logit.  Returns ``(ids, logit)``."""
    if _cuda(h):
        return _k().lm_head_argmax(h, table, softcap, vocab_limit)
    logits = ref.softcap(ref.linear(h, table).float(), softcap)
    if vocab_limit:
        logits = logits[:, :vocab_limit]
    ids = ref.argmax_first(logits)
    return ids, logits.gather(-1, ids[:, None])[:, 0]


def router_topk(logits, k, mode="softmax", bias=None, n_group=1, topk_group=1, scale=1.0, renorm=True):
    if _cuda(logits):
        return _k().router_topk(logits, k, mode, bias, n_group, topk_group, scale, renorm)
    if mode == "softmax":
        return ref.router_softmax_topk(logits, k, renorm)
    return ref.router_sigmoid_topk(logits, bias, k, n_group, topk_group, scale, renorm)


def bf16_experts(x, idx, w, gate_up, down, e0: int = 0, act: str = "geglu"):
    """``sum_k w[t,k] * down[e] (act(gate[e] x_t) * up[e] x_t)`` over the experts ``e0 .. e0 + len(gate_up)`` held here, with
    unquantised expert weights ``gate_up[E, 2F, H]`` / ``down[E, H, F]`` (src/models/inkling/moegroup.rs:556-719, the grouped bf16
    lane; src/models/gemma/gemma4/layers.rs:328-418).  GPU: routing plan + grouped tensor-core GEMMs.  CPU: entries grouped by
    expert, one GLU MLP per expert on its rows, weighted rows summed per token in f32."""
    if _cuda(x):
        from . import cuda_moe
        return cuda_moe.experts_forward_bf16(x, idx, w, gate_up, down, act, e0)
    T, k = idx.shape
    out = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device)
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=e0 + gate_up.shape[0]).tolist()
    start = sum(counts[:e0])
    for e in range(gate_up.shape[0]):
        n = counts[e0 + e]
        if n == 0:
            continue
        ent = order[start:start + n]
        start += n
        tok = ent // k
        y = linear(linear_glu(x[tok].contiguous(), gate_up[e], act), down[e])
        out.index_add_(0, tok, y.float() * w.reshape(-1)[ent].float()[:, None])
    return out.to(x.dtype)


def quantize_nvfp4(x):
    return _k().quantize_nvfp4(x) if _cuda(x) else ref.quantize_nvfp4(x)


def short_conv(x, w, history=None):
    return _k().short_conv(x, w, history) if _cuda(x) else ref.short_conv(x, w, history)

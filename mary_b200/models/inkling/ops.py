"""Inkling operators as the reference defines them (fidelity targets beyond the abstract "Inkling-style" workload).

* decoder layer: ``x += sconv_attn(attn(rms(x)))``; ``x += sconv_mlp(mlp(rms(x)))`` with ``sconv(y) = y + depthwise causal
  conv_k4(y)`` (src/models/inkling/layer.rs:8-174, block.rs:48-127);
* attention: K and V (not Q) pass through their own short conv; per-head RMSNorm on q and k; ``score = (q.k)/head_dim +
  rel[q,h,dist] * tau + mask`` with ``rel = (x W_r)[h, :d_rel] @ rel_proj[d_rel, extent]`` (zero outside ``[0, extent)``),
  ``tau(pos) = 1 + alpha ln(max(1, (pos+1)/n_floor))`` multiplying q and the bias on GLOBAL layers only; local layers mask
  ``dist >= window`` (attn.rs:53-68,217-335);
* router: pick top-k by ``sigmoid(l) + bias`` (ties to the lower index); weights = softmax over ``log_sigmoid(l)`` of the
  chosen UNION the shared experts, times ``route_scale * global_scale``; the shared experts' gammas come from the same
  softmax; a non-finite logit is an error (block.rs:140-250, routetopk.rs:112-260);
* dense MLP ``down(silu(g) * u) * global_scale`` (mlp.rs:69-87); stack: embed -> embed_norm ... final norm, DIVIDE by the
  muP width multiplier, un-embed, truncate to the real vocabulary (stack.rs:1-121).
Pure PyTorch (any device); these are oracles and the CPU path, the serving kernels live in ``csrc/kernels``."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ...ops import reference as ref


def short_conv_seq(x, w, history=None):
    """``y = x + conv``; returns ``(y, new_history)`` — see :func:`mary_b200.ops.reference.short_conv`."""
    return ref.short_conv(x, w, history)


def log_scale_tau(pos, alpha: float, n_floor: float):
    return 1.0 + alpha * torch.log(torch.clamp((pos.float() + 1.0) / n_floor, min=1.0))


def relative_bias(x, w_r, rel_proj, n_heads: int, d_rel: int):
    """``rel[t, h, dist]`` for dist in ``[0, extent)``: ``(x W_r^T)[t, h, :d_rel] @ rel_proj[d_rel, extent]``."""
    r = (x.float() @ w_r.float().t()).view(x.shape[0], n_heads, d_rel)
    return r @ rel_proj.float()


def attention(x, p: dict, cfg: dict, positions=None, cache: dict | None = None, is_global: bool = True):
    """Whole-sequence (or cached incremental) Inkling attention for one sequence ``x[T, H]``.
    ``p``: wq, wk, wv, wo, wr, rel_proj, q_norm, k_norm, k_conv, v_conv.  ``cache`` keeps post-conv/post-norm K, post-conv V
    and the pre-conv histories."""
    T = x.shape[0]
    Hq, Hkv, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    base = 0 if cache is None or "k" not in cache else cache["k"].shape[0]
    pos = positions if positions is not None else torch.arange(base, base + T)
    q = (x.float() @ p["wq"].float().t()).view(T, Hq, D)
    k = x.float() @ p["wk"].float().t()
    v = x.float() @ p["wv"].float().t()
    hk = cache.get("hist_k") if cache is not None else None
    hv = cache.get("hist_v") if cache is not None else None
    k, hk = ref.short_conv(k, p["k_conv"], hk)
    v, hv = ref.short_conv(v, p["v_conv"], hv)
    k, v = k.view(T, Hkv, D), v.view(T, Hkv, D)
    q = ref.rmsnorm(q, p["q_norm"], cfg.get("eps", 1e-6))
    k = ref.rmsnorm(k, p["k_norm"], cfg.get("eps", 1e-6))
    if cache is not None:
        k = torch.cat([cache["k"], k], 0) if "k" in cache else k
        v = torch.cat([cache["v"], v], 0) if "v" in cache else v
        cache.update(k=k, v=v, hist_k=hk, hist_v=hv)
    L = k.shape[0]
    kpos = torch.arange(L)
    g = Hq // Hkv
    kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    tau = log_scale_tau(pos, cfg["log_alpha"], cfg["log_n_floor"]) if is_global else torch.ones(T)
    s = torch.einsum("thd,lhd->htl", q.float() * tau[:, None, None], kk.float()) / D
    dist = pos[:, None] - kpos[None, :]
    rel = relative_bias(x, p["wr"], p["rel_proj"], Hq, cfg["d_rel"])            # [T, Hq, extent]
    ext = rel.shape[-1]
    inside = (dist >= 0) & (dist < ext)
    bias = torch.gather(rel.permute(1, 0, 2), 2, dist.clamp(0, ext - 1)[None].expand(Hq, -1, -1)) * inside[None]
    s = s + bias * tau[None, :, None]
    mask = dist >= 0
    if not is_global:
        mask = mask & (dist < cfg["window"])
    s = s.masked_fill(~mask[None], float("-inf"))
    o = torch.einsum("htl,lhd->thd", torch.softmax(s, -1), vv.float()).reshape(T, Hq * D)
    return (o @ p["wo"].float().t()).to(x.dtype)


def router(logits, bias, k: int, n_shared: int, route_scale: float, global_scale: float = 1.0):
    """``logits[T, n_routed + n_shared]``.  Returns ``(idx[T, k], w_routed[T, k], gammas[T, n_shared])``."""
    if not torch.isfinite(logits).all():
        raise FloatingPointError("non-finite router logit")
    n_routed = logits.shape[-1] - n_shared
    lr = logits[:, :n_routed].float()
    sel = torch.sigmoid(lr) + bias.float()
    _, idx = ref.topk_first(sel, k)
    chosen = lr.gather(-1, idx)
    pool = torch.cat([F.logsigmoid(chosen), F.logsigmoid(logits[:, n_routed:].float())], -1)
    w = torch.softmax(pool, -1) * (route_scale * global_scale)
    return idx.int(), w[:, :k], w[:, k:]


def dense_mlp(x, w_gate, w_up, w_down, global_scale: float = 1.0):
    h = F.silu(x.float() @ w_gate.float().t()) * (x.float() @ w_up.float().t())
    return ((h @ w_down.float().t()) * global_scale).to(x.dtype)


def unembed(h, final_norm, w_unembed, mup_width_multiplier: float, real_vocab: int, eps: float = 1e-6):
    x = ref.rmsnorm(h, final_norm, eps).float() / mup_width_multiplier
    return (x @ w_unembed.float().t())[:, :real_vocab]


# --------------------------------------------------------------------------------------------------------------------------
# whole layer, stack ends and multi-token-prediction heads (src/models/inkling/{layer,stack,mtp}.rs)

def decoder_layer(x, p: dict, cfg: dict, cache: dict | None = None, is_global: bool = True, mlp=None):
    """One decoder layer on one sequence ``x[T, H]``:

        x = x + sconv_attn(attn(rms(x, attn_norm)));   x = x + sconv_mlp(mlp(rms(x, mlp_norm)))

    Both layer-level short convolutions FOLLOW their block and carry their own inner residual (``sconv(y) = y + conv(y)``), so the
    layer has four additive paths.  Three of them keep state across steps: attention's K / V (with the K / V conv histories) and
    the two layer-level conv histories; ``cache`` holds all of it (``attn`` sub-dict, ``hist_attn``, ``hist_mlp``).
    ``mlp``: callable for a routed layer; default is the dense MLP from ``p`` (``w_gate, w_up, w_down``)."""
    eps = cfg.get("eps", 1e-6)
    if cache is not None:
        cache.setdefault("attn", {})
    h = attention(ref.rmsnorm(x, p["attn_norm"], eps), p, cfg, cache=None if cache is None else cache["attn"], is_global=is_global)
    h, ha = ref.short_conv(h, p["attn_sconv"], None if cache is None else cache.get("hist_attn"))
    x = x + h
    y = ref.rmsnorm(x, p["mlp_norm"], eps)
    m = mlp(y) if mlp is not None else dense_mlp(y, p["w_gate"], p["w_up"], p["w_down"], cfg.get("global_scale", 1.0))
    m, hm = ref.short_conv(m, p["mlp_sconv"], None if cache is None else cache.get("hist_mlp"))
    if cache is not None:
        cache.update(hist_attn=ha, hist_mlp=hm)
    return x + m


def embed_in(ids, embed, embed_norm, eps: float = 1e-6):
    """``embed_norm(embed[ids])``: the norm belongs to the embedding output, before any layer."""
    return ref.rmsnorm(embed[torch.as_tensor(ids).long()], embed_norm, eps)


def mtp_input(hidden, tok_embed, p: dict, hidden_first: bool = True, eps: float = 1e-6):
    """Input of an MTP head at position ``j``: ``input_proj(cat(hidden_norm(main_hidden[j]), embed_norm(embed(token[j + 1]))))`` with
    ``input_proj [H, 2H]``.  Upstream defines no reference for the order of the two operands; ``hidden_first`` keeps both orders
    reachable (the acceptance rate of the drafts is the measurement that picks one: a wrong order cannot change the text,
    only how many drafts survive verification)."""
    a, b = ref.rmsnorm(hidden, p["hidden_norm"], eps), ref.rmsnorm(tok_embed, p["embed_norm"], eps)
    cat = torch.cat([a, b] if hidden_first else [b, a], -1)
    return (cat.float() @ p["input_proj"].float().t()).to(hidden.dtype)


def mtp_block(main_hidden, next_tok_embed, p: dict, cfg: dict, cache: dict | None = None, hidden_first: bool = True):
    """One MTP head over rows ``(main_hidden[j], embed(token[j + 1]))``: wrapper + one DENSE decoder layer.  With ``cache`` the rows
    extend the head's own K / V and conv state (``main_hidden[j]`` never changes once produced, so its K / V are stable)."""
    return decoder_layer(mtp_input(main_hidden, next_tok_embed, p, hidden_first, cfg.get("eps", 1e-6)), p, cfg, cache, is_global=True)


def clone_cache(cache: dict) -> dict:
    """Deep copy of a layer cache: drafts run on the clone, which is then dropped — rollback is the default, commitment the exception."""
    return {k: (clone_cache(v) if isinstance(v, dict) else (v.clone() if torch.is_tensor(v) else v)) for k, v in cache.items()}


def mtp_draft(heads: list, caches: list, main_hidden_last, embed, embed_norm_w, unembed_fn, first_token: int, cfg: dict, hidden_first=True):
    """Chain the heads to draft ``len(heads)`` tokens after ``first_token`` (the main model's own next token): head ``d`` reads the
    previous head's output row and the embedding of the token drafted before it.  Runs on CLONES of the heads' caches and returns
    ``(tokens, logits_rows)``; the caller commits nothing until the main model has verified the drafts."""
    toks, rows = [], []
    h, tok = main_hidden_last[None], first_token
    for p, c in zip(heads, caches):
        e = embed[torch.tensor([tok])]
        h = mtp_block(h, e, p, cfg, clone_cache(c) if c is not None else None, hidden_first)
        logits = unembed_fn(h)
        tok = int(ref.argmax_first(logits)[0])
        toks.append(tok)
        rows.append(logits[0])
    return toks, rows

"""Kimi-K3 operators as the reference defines them (fidelity targets beyond the abstract "K3-class" workload).

* RMSNorm: ``x / sqrt(mean(x^2) + eps)`` (division), cast to the activation dtype BEFORE the gain multiply (two roundings in
  bf16); eps 1e-5 for layer norms, 1e-6 inside MLA (src/models/k3/ops.rs:24-127, mla.rs:102-111);
* MLA (NoPE): q 7168->1536->norm->H x (128+64); kv_a 7168->512+64; latent->norm->kv_b->H x (128 k_pass + 128 v);
  ``k = cat(k_pass, carried broadcast)``; scale ``192^-0.5``; mask value = bf16 min (finite); softmax in f32; output gated by
  ``sigmoid(g_proj(x))`` before ``o_proj`` (mla.rs:49-63,281-293);
* router ``noaux_tc``: ``scores = sigmoid(h W^T)`` in f32; select top-k of ``scores + bias``; weights = unbiased scores
  renormalised by ``sum + 1e-20`` times the factor (router.rs:9-15) — :func:`mary_b200.ops.reference.router_sigmoid_topk`;
* latent MoE: ``down_proj 7168->3584``; ``sum_k w * w2(situ(w1 x, w3 x))``; ``routed_expert_norm`` AFTER the sum; ``up_proj``;
  plus a shared MLP on the original hidden (moe.rs:4-39); SiTU ``beta tanh(g/beta) sigmoid(g) * lb tanh(u/lb)`` (situ.rs:54-145);
* KDA: gated delta rule with bounded gate ``-5 sigmoid(exp(A_log)(g + dt_bias))``, L2-normalised q/k, O(1) state
  (kda.rs:1-120);
* AttnRes: depth-axis softmax mixture over a bank of layer checkpoints plus an accumulator (attn_res.rs:1-120).
Pure PyTorch; these are oracles and the CPU path."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import reference as ref


def rms_norm(x, gain, eps: float = 1e-5):
    xf = x.float()
    y = (xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)      # first rounding
    return (y * gain.to(x.dtype)) if gain is not None else y                      # second rounding


def mla_nope(x, p: dict, n_heads: int, cache: dict | None = None):
    """NoPE MLA for one sequence ``x[T, H]``; the cache holds EXPANDED k and v as in the reference."""
    T = x.shape[0]
    qa = rms_norm(F.linear(x, p["q_a"]), p["q_a_norm"], 1e-6)
    q = F.linear(qa, p["q_b"]).view(T, n_heads, 192)
    kva = F.linear(x, p["kv_a"])
    latent, carried = kva[:, :512], kva[:, 512:]
    kvb = F.linear(rms_norm(latent, p["kv_a_norm"], 1e-6), p["kv_b"]).view(T, n_heads, 256)
    k = torch.cat([kvb[..., :128], carried[:, None, :].expand(T, n_heads, 64)], -1)
    v = kvb[..., 128:]
    base = 0
    if cache is not None:
        if "k" in cache:
            base = cache["k"].shape[0]
            k, v = torch.cat([cache["k"], k], 0), torch.cat([cache["v"], v], 0)
        cache.update(k=k, v=v)
    L = k.shape[0]
    s = torch.einsum("thd,lhd->htl", q.float(), k.float()) * (192 ** -0.5)
    qpos, kpos = torch.arange(base, base + T), torch.arange(L)
    s = torch.where((kpos[None, :] <= qpos[:, None])[None], s, torch.full_like(s, torch.finfo(torch.bfloat16).min))
    o = torch.einsum("htl,lhd->thd", torch.softmax(s, -1), v.float()).reshape(T, n_heads * 128).to(x.dtype)
    gate = torch.sigmoid(F.linear(x, p["g_proj"]).float()).to(x.dtype)
    return F.linear(o * gate, p["o_proj"])


def latent_moe(x, p: dict, k: int, factor: float, bias=None):
    """``p``: router, down_proj, up_proj, expert_norm, w1/w3/w2 ``[E, ...]`` (dense tensors), shared_gate/up/down."""
    idx, w = ref.router_sigmoid_topk(F.linear(x.float(), p["router"].float()), bias, k, scale=factor)
    z = F.linear(x, p["down_proj"])
    acc = torch.zeros(z.shape, dtype=torch.float32)
    for e in idx.unique().tolist():
        t, j = (idx == e).nonzero(as_tuple=True)
        h = ref.situ(F.linear(z[t], p["w1"][e]), F.linear(z[t], p["w3"][e]))
        acc.index_add_(0, t, F.linear(h, p["w2"][e]).float() * w[t, j][:, None])
    routed = F.linear(rms_norm(acc.to(x.dtype), p["expert_norm"]), p["up_proj"])
    shared = F.linear(ref.situ(F.linear(x, p["shared_gate"]), F.linear(x, p["shared_up"])), p["shared_down"])
    return routed + shared


def kda_recurrent(q, k, v, g, beta, A_log, dt_bias, state=None):
    """Gated delta rule, one head: ``q,k [T, dk]`` (L2-normalised here), ``v [T, dv]``, gate input ``g [T, dk]``, write
    strength ``beta [T]``.  ``S_t = S_{t-1} * exp(a_t) + beta_t k_t (v_t - (S_{t-1} exp(a_t))^T k_t)^T`` with the bounded
    log-decay ``a_t = -5 sigmoid(exp(A_log) (g_t + dt_bias))``; ``o_t = S_t^T q_t``.  Returns ``(o [T, dv], S [dk, dv])``."""
    T, dk = q.shape
    dv = v.shape[1]
    q = F.normalize(q.double(), dim=-1)
    k = F.normalize(k.double(), dim=-1)
    S = torch.zeros(dk, dv, dtype=torch.float64) if state is None else state.double().clone()
    a = -5.0 * torch.sigmoid(torch.exp(A_log.double()) * (g.double() + dt_bias.double()))
    out = []
    for t in range(T):
        S = S * torch.exp(a[t])[:, None]
        pred = S.t() @ k[t]
        S = S + beta[t].double() * torch.outer(k[t], v[t].double() - pred)
        out.append(S.t() @ q[t])
    return torch.stack(out).to(v.dtype), S


def attn_res_mix(bank, accumulator, query, keys_proj, eps: float = 1e-5):
    """Depth-axis mixture: softmax over ``[bank checkpoints..., accumulator]`` of ``<rms(source), query>`` scores, returning
    the mixed hidden state (attn_res.rs:1-120).  ``bank [n, T, H]``, ``accumulator [T, H]``, ``query [H]``."""
    src = torch.cat([bank, accumulator[None]], 0)
    normed = rms_norm(src, None, eps).float()
    scores = (normed @ (keys_proj.float() @ query.float())) if keys_proj is not None else (normed @ query.float())
    wgt = torch.softmax(scores, 0)
    return (wgt[..., None] * src.float()).sum(0).to(accumulator.dtype)

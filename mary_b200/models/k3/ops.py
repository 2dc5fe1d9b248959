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


# --------------------------------------------------------------------------------------------------------------------------
# configuration, the KDA sublayer with its projections, and the whole decoder layer (src/models/k3/{config,kda_attn,layer}.rs)

class K3Config:
    """The attention lists are ONE-based (layer 3 of a list means the third layer, index 2); the dense-layer index is zero-based
    (config.rs:153-370).  ``validate`` checks that the two lists partition ``1 .. n_layers``."""

    def __init__(self, n_layers: int, kda_layers, full_attn_layers, first_k_dense: int = 1, snapshot_every: int = 12, n_heads: int = 4,
                 kda_head_dim: int = 16, conv_kernel: int = 4):
        self.n_layers, self.kda_layers, self.full_attn_layers = n_layers, list(kda_layers), list(full_attn_layers)
        self.first_k_dense, self.snapshot_every = first_k_dense, snapshot_every
        self.n_heads, self.kda_head_dim, self.conv_kernel = n_heads, kda_head_dim, conv_kernel
        self.validate()

    def validate(self) -> None:
        both = self.kda_layers + self.full_attn_layers
        if sorted(both) != list(range(1, self.n_layers + 1)):
            dup = sorted({x for x in both if both.count(x) > 1})
            missing = sorted(set(range(1, self.n_layers + 1)) - set(both))
            raise ValueError(f"attention lists must partition layers 1..{self.n_layers}: duplicated {dup}, missing {missing}, "
                             f"out of range {sorted(x for x in both if not 1 <= x <= self.n_layers)}")

    def attn_kind(self, layer_index: int) -> str:
        """``"mla"`` or ``"kda"`` for the ZERO-based layer index."""
        return "mla" if layer_index + 1 in self.full_attn_layers else "kda"

    def is_dense(self, layer_index: int) -> bool:
        return layer_index < self.first_k_dense

    def is_boundary(self, layer_index: int) -> bool:
        """Layers at which the depth accumulator is pushed to the bank and reset."""
        return layer_index > 0 and layer_index % self.snapshot_every == 0


def _bf(x, like):
    return x.to(like.dtype)


def kda_attention(x, p: dict, cfg: K3Config, cache: dict | None = None):
    """The whole KDA sublayer for one sequence ``x[T, H]`` (kda_attn.rs): q / k / v projections, each followed by a depthwise causal
    short convolution (kernel 4) with SiLU; the decay-gate input from a low-rank pair ``f_b(f_a(x))``; the write strength
    ``beta = sigmoid(b_proj(x))`` per head; the gated delta-rule recurrence per head (f32 / f64 inside, state O(1) in the sequence
    length); a gated RMSNorm of the output, ``o_norm(o) * sigmoid(g_b(g_a(x)))``; ``o_proj``.  ``A_log``, ``dt_bias``, the
    convolution taps and ``o_norm`` stay f32; every projection / convolution / recurrence output is rounded to the activation
    dtype.  ``cache``: per-head recurrent state and the three convolution histories."""
    T = x.shape[0]
    nh, dk = cfg.n_heads, cfg.kda_head_dim
    K = cfg.conv_kernel

    def conv(name, y):
        hist = None if cache is None else cache.get("hist_" + name)
        if hist is None:
            hist = torch.zeros(K - 1, y.shape[1], dtype=torch.float32)
        ext = torch.cat([hist, y.float()], 0)
        w = p[name + "_conv"].float()                                   # [C, K]; tap K-1 multiplies the current row
        out = sum(ext[j:j + T] * w[:, j] for j in range(K))
        if cache is not None:
            cache["hist_" + name] = ext[-(K - 1):]
        return _bf(F.silu(out), x)
    q = conv("q", F.linear(x, p["q_proj"])).view(T, nh, dk)
    k = conv("k", F.linear(x, p["k_proj"])).view(T, nh, dk)
    v = conv("v", F.linear(x, p["v_proj"])).view(T, nh, dk)
    g = F.linear(F.linear(x, p["f_a_proj"]), p["f_b_proj"]).view(T, nh, dk)
    beta = torch.sigmoid(F.linear(x, p["b_proj"]).float())             # [T, nh]
    outs, states = [], []
    for h in range(nh):
        st = None if cache is None or "state" not in cache else cache["state"][h]
        o, S = kda_recurrent(q[:, h], k[:, h], v[:, h], g[:, h], beta[:, h], p["A_log"][h], p["dt_bias"].view(nh, dk)[h], st)
        outs.append(o * dk ** -0.5 if p.get("scale_output") else o)
        states.append(S)
    if cache is not None:
        cache["state"] = states
    o = _bf(torch.stack(outs, 1), x)                                    # [T, nh, dk]
    glin = F.linear(x, p["g_proj"]) if "g_proj" in p else F.linear(F.linear(x, p["g_a_proj"]), p["g_b_proj"])   # full-rank gate in K3
    gate = torch.sigmoid(glin.float()).view(T, nh, dk)
    of = o.float()
    normed = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + 1e-5) * p["o_norm"].float()
    return F.linear(_bf(normed * gate, x).reshape(T, nh * dk), p["o_proj"])


class DepthMixer:
    """The bank of depth checkpoints shared by ALL layers of one forward pass (a layer that owned its own copy would start every
    layer with an empty bank).  ``mix`` is the depth-axis softmax mixture of the bank and the running accumulator; with an empty
    bank it is the identity."""

    def __init__(self):
        self.bank: list = []

    def mix(self, prefix_sum, query, keys_proj=None):
        if not self.bank:
            return prefix_sum
        return attn_res_mix(torch.stack(self.bank), prefix_sum, query, keys_proj)

    def push(self, layer_in):
        self.bank.append(layer_in)


def decoder_layer(layer_in, layer_index: int, cfg: K3Config, mixer: DepthMixer, attn, ffn, p: dict):
    """``KimiDecoderLayer`` (layer.rs): NOT a residual stream.

        prefix = layer_in;  hidden = mix(prefix)                       (identity while the bank is empty)
        if boundary: bank.push(layer_in); prefix = None
        hidden = attn(input_layernorm(hidden));     prefix = hidden if prefix is None else prefix + hidden
        hidden = mix(prefix);  hidden = ffn(post_attention_layernorm(hidden))
        return prefix + hidden

    ``attn`` / ``ffn`` are callables (MLA or KDA; dense MLP or latent MoE); ``p`` holds the two norms' gains and the two mixture
    queries (``attn_res_q1``, ``attn_res_q2``)."""
    prefix = layer_in
    hidden = mixer.mix(prefix, p["attn_res_q1"])
    if cfg.is_boundary(layer_index):
        mixer.push(layer_in)
        prefix = None
    hidden = attn(rms_norm(hidden, p["input_layernorm"]))
    prefix = hidden if prefix is None else prefix + hidden
    hidden = mixer.mix(prefix, p["attn_res_q2"])
    hidden = ffn(rms_norm(hidden, p["post_attention_layernorm"]))
    return prefix + hidden

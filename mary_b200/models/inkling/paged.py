"""Inkling attention over the paged cache on the package ops: what the serving lane runs (src/models/inkling/burn.rs attention lanes,
banded.rs, scorebias.rs), with the model's own score rule instead of the abstract workload's plain GQA.

One sequence at a time (the short convolutions on K and V carry a per-sequence history): q / k / v / r projections as one GEMM,
depthwise causal short convolution on K and V with carried history, per-head RMSNorm of q and k and the cache append in the fused
norm-append kernel (no rotary code: positions enter only through the relative bias), the rank-``d_rel`` relative bias
``(x W_r)[h] @ rel_proj`` as a small GEMM, log scaling ``tau(pos)`` multiplied into q and the bias on global layers, and the general
split-KV attention kernel with the additive bias hook, score scale ``1 / head_dim`` and the window of local layers."""
from __future__ import annotations

import torch

from ... import ops
from ...ops import reference as ref
from .ops import log_scale_tau


class InklingPagedAttention:
    def __init__(self, p: dict, cfg: dict, is_global: bool = True):
        """``p``: wq, wk, wv, wo, wr, rel_proj, q_norm, k_norm, k_conv, v_conv (as in ``inkling.ops.attention``)."""
        self.p, self.cfg, self.is_global = p, cfg, is_global
        self.w_qkvr = torch.cat([p["wq"], p["wk"], p["wv"], p["wr"]], 0).contiguous()
        # rel_proj [d_rel, extent] used as the GEMM weight [extent, d_rel]
        self.rel_w = p["rel_proj"].t().contiguous()
        self.hist_k = self.hist_v = None

    def reset(self):
        self.hist_k = self.hist_v = None

    def __call__(self, x, meta, kcache, vcache):
        """``x [T, H]`` rows of ONE sequence (a prefill chunk or decode rows), ``meta`` describing them; returns ``[T, H]``."""
        c, p = self.cfg, self.p
        Hq, Hkv, D, dr = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["d_rel"]
        T = x.shape[0]
        y = ops.linear(x, self.w_qkvr)
        q, k, v, r = y.split([Hq * D, Hkv * D, Hkv * D, Hq * dr], -1)
        k, self.hist_k = ops.short_conv(k.contiguous(), p["k_conv"], self.hist_k)
        v, self.hist_v = ops.short_conv(v.contiguous(), p["v_conv"], self.hist_v)
        qkv = torch.cat([q, k, v], -1).contiguous()
        qn = ops.qk_norm_rope_append(qkv, Hq, Hkv, D, p["q_norm"], p["k_norm"], False, None, meta, kcache, vcache, c.get("eps", 1e-6))
        rel = ops.linear(r.reshape(T * Hq, dr).contiguous(), self.rel_w).float().view(T, Hq, -1)
        if self.is_global:
            tau = log_scale_tau(meta.positions, c["log_alpha"], c["log_n_floor"]).to(x.device)
            qn = (qn.float() * tau[:, None, None]).to(qn.dtype)
            rel = rel * tau[:, None, None]
        o = ops.paged_attention(qn, kcache, vcache, meta, 1.0 / D, 0 if self.is_global else c["window"], rel_bias=rel.contiguous())
        return ops.linear(o.reshape(T, Hq * D), p["wo"])

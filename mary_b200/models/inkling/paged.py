"""Inkling attention over the paged cache on the package ops: what the serving lane runs (src/models/inkling/burn.rs attention lanes,
banded.rs, scorebias.rs), with the model's own score rule instead of the abstract workload's plain GQA.

Any flattened batch: the short convolutions on K and V carry one history PER SEQUENCE (the reference's "slots"); a batch of decode
rows (one row per sequence) runs them as one vectorised step over all slots, prefill chunks run sequence by sequence.  Per call: q / k / v / r projections as one GEMM,
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
        self.hist: dict = {}            # slot (sequence id) -> (k history, v history), each [taps - 1, Hkv * D]

    def reset(self, slot=None):
        self.hist.clear() if slot is None else self.hist.pop(slot, None)

    def _conv_slots(self, x, w, which: int, slots, meta):
        """``x [T, C]`` rows of the flattened batch -> ``x + conv(x)`` with every sequence's own history."""
        taps = w.shape[1]
        S = meta.num_seqs
        starts = meta.q_start.tolist()
        zero = lambda: torch.zeros(taps - 1, x.shape[1], dtype=x.dtype, device=x.device)  # noqa: E731
        if meta.max_q_len == 1 and x.shape[0] == S:
            # decode: one row per slot, all slots in one step
            h = torch.stack([self.hist.get(s, (None, None))[which] if self.hist.get(s, (None, None))[which] is not None else zero() for s in slots])
            wf = w.float()
            y = x.float() * (1.0 + wf[:, taps - 1]) + (h.float() * wf[:, :taps - 1].T[None]).sum(1)
            new = torch.cat([h[:, 1:], x[:, None]], 1)
            for i, s in enumerate(slots):
                pair = list(self.hist.get(s, (None, None)))
                pair[which] = new[i]
                self.hist[s] = tuple(pair)
            return y.to(x.dtype)
        out = torch.empty_like(x)
        for i, s in enumerate(slots):
            a, b = starts[i], starts[i + 1]
            if a == b:
                continue
            pair = list(self.hist.get(s, (None, None)))
            out[a:b], pair[which] = ops.short_conv(x[a:b].contiguous(), w, pair[which])
            self.hist[s] = tuple(pair)
        return out

    def __call__(self, x, meta, kcache, vcache, slots=None):
        """``x [T, H]`` rows of the flattened batch described by ``meta``; ``slots`` names the sequence (conv history) of every entry of
        the batch (default ``0 .. num_seqs - 1``).  Returns ``[T, H]``."""
        c, p = self.cfg, self.p
        Hq, Hkv, D, dr = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["d_rel"]
        T = x.shape[0]
        slots = list(range(meta.num_seqs)) if slots is None else list(slots)
        y = ops.linear(x, self.w_qkvr)
        q, k, v, r = y.split([Hq * D, Hkv * D, Hkv * D, Hq * dr], -1)
        k = self._conv_slots(k.contiguous(), p["k_conv"], 0, slots, meta)
        v = self._conv_slots(v.contiguous(), p["v_conv"], 1, slots, meta)
        qkv = torch.cat([q, k, v], -1).contiguous()
        qn = ops.qk_norm_rope_append(qkv, Hq, Hkv, D, p["q_norm"], p["k_norm"], False, None, meta, kcache, vcache, c.get("eps", 1e-6))
        rel = ops.linear(r.reshape(T * Hq, dr).contiguous(), self.rel_w).float().view(T, Hq, -1)
        if self.is_global:
            tau = log_scale_tau(meta.positions, c["log_alpha"], c["log_n_floor"]).to(x.device)
            qn = (qn.float() * tau[:, None, None]).to(qn.dtype)
            rel = rel * tau[:, None, None]
        o = ops.paged_attention(qn, kcache, vcache, meta, 1.0 / D, 0 if self.is_global else c["window"], rel_bias=rel.contiguous())
        return ops.linear(o.reshape(T, Hq * D), p["wo"])

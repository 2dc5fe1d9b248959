"""Cut a full (single-rank) ``MoEDecoder`` into the shard of one rank of a tensor/expert-parallel group.

Attention heads, dense-FFN and shared-expert columns are split by rank (column-parallel weights by output rows, the
following row-parallel weights by input columns); routed experts are split by expert index; everything else is replicated."""
from __future__ import annotations

import torch

from ...ops.moe import NVFP4Experts
from .model import DenseFFN, GQAAttention, MLAAttention, MoEDecoder, MoEFFN


def _rows(t, r, n):
    k = t.shape[0] // n
    return t[r * k:(r + 1) * k]


def _cols(t, r, n):
    k = t.shape[1] // n
    return t[:, r * k:(r + 1) * k]


def _gu(t, r, n):
    F = t.shape[0] // 2
    k = F // n
    return torch.cat([t[r * k:(r + 1) * k], t[F + r * k:F + (r + 1) * k]], 0)


def slice_experts(ex: NVFP4Experts, r: int, n: int, tail: int = 0) -> NVFP4Experts:
    """Experts ``[r*e, (r+1)*e)`` of the routed ones, followed by the ``tail`` shared experts that every rank keeps."""
    e = (ex.E - tail) // n
    a, b = r * e, (r + 1) * e
    r13, r2 = 2 * ex.F, ex.H

    def cut(t, per):
        parts = [t[a * per:b * per]]
        if tail:
            parts.append(t[(ex.E - tail) * per:ex.E * per])
        return torch.cat(parts, 0) if tail else parts[0]
    return NVFP4Experts(e + tail, ex.H, ex.F, cut(ex.w13_q, r13), cut(ex.w13_sf, r13 // 128), cut(ex.w13_s2, 1),
                        cut(ex.w2_q, r2), cut(ex.w2_sf, r2 // 128), cut(ex.w2_s2, 1), ex.act)


def cut_parameter(cfg, mod, name: str, src, r: int, n: int, vocab_parallel: bool):
    """The slice of the full parameter ``name`` (owned by module ``mod``) that tensor-parallel rank ``r`` of ``n`` holds: the one rule
    for cutting a model in memory (``shard_from_full``) and for loading a rank's shard from a pile (``weights.load_from_pile``)."""
    if n == 1:
        return src
    leaf = name.rpartition(".")[2]
    if isinstance(mod, GQAAttention):
        D = cfg.head_dim
        if leaf == "w_qkv":
            q, k, v = src.split([cfg.num_attention_heads * D, cfg.num_key_value_heads * D, cfg.num_key_value_heads * D], 0)
            return torch.cat([_rows(q, r, n), _rows(k, r, n), _rows(v, r, n)], 0)
        if leaf == "w_o":
            return _cols(src, r, n)
    elif isinstance(mod, MLAAttention):
        if leaf in ("w_qb", "w_uk", "w_uv"):
            return _rows(src, r, n)
        if leaf == "w_o":
            return _cols(src, r, n)
    elif isinstance(mod, DenseFFN):
        return _gu(src, r, n) if leaf == "w_gu" else _cols(src, r, n)
    elif name == "lm_head" and vocab_parallel:
        return _rows(src, r, n)
    return src


def shard_from_full(full: MoEDecoder, par, device=None) -> MoEDecoder:
    r, n = par.tp_rank, par.tp_size        # attention / dense split; experts split by the expert-parallel coordinates
    er, en = par.ep_rank, par.ep_size
    dev = device or full.embed.device
    m = MoEDecoder(full.cfg, par=par, dtype=full.dtype, device=dev)
    fm = dict(full.named_modules())
    full_params = dict(full.named_parameters())
    with torch.no_grad():
        for name, p in m.named_parameters():
            src = cut_parameter(full.cfg, fm.get(name.rpartition(".")[0]), name, full_params[name], r, n, m.vocab_parallel)
            p.copy_(src.to(dev))
    for (_, a), (_, b) in zip(m.named_modules(), full.named_modules()):
        if isinstance(a, MoEFFN):
            ex = slice_experts(b.experts, er, en, 1 if b.shared_in_experts else 0)
            for f in ("w13_q", "w13_sf", "w13_s2", "w2_q", "w2_sf", "w2_s2"):
                setattr(ex, f, getattr(ex, f).to(dev))
            a.experts = ex
    return m

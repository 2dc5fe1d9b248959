"""Inkling's vision (HMLP) and audio (dMel) towers (src/models/inkling/vision.rs).  Neither is an encoder stack: vision is a
hierarchy of MLPs over folded patches, audio a sum of per-bin codebook lookups; both embed straight into the text model.

HMLP plan.  A patch of ``temporal x patch x patch`` pixels is folded into the channel axis in ``n_layers`` steps.  The candidate
grids come from the prime factors of the patch sizes (largest factor first, cumulative products): ``(1, h, h)`` with
``ceil(h^2 C / 64) * 64`` channels for every spatial step, then ``(t, h_last, h_last)`` with ``64 h_last^2 C t`` channels for every
temporal step.  ``n_layers + 1`` of them are picked so that the log of their fold sizes sits closest to an even spacing between
0 and ``log(total)`` (minimum-cost assignment); the first and last picks are pinned to the first and last candidate.  The layer
widths are therefore DERIVED from the patch geometry (the released 40-pixel patch gives 128, 320, 4800), never tabulated.

A stage folds ``(T, H, W, C) -> (T / t, H / s, W / s, t s s C)`` with the folded axes OUTSIDE the channel axis
(``(t', h', w', t_fold, h_fold, w_fold, C)`` flattened), projects, and — except the last stage, which targets the text width —
applies RMSNorm and exact (erf) GELU.  The projections run on ``ops.linear`` (tensor cores on a GPU)."""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from ... import ops
from ...ops import reference as ref


def _factors_desc(n: int) -> list[int]:
    out, p = [], 2
    while p * p <= n:
        while n % p == 0:
            out.append(p)
            n //= p
        p += 1
    if n > 1:
        out.append(n)
    return out[::-1]


def plan_scales(temporal_patch: int, patch: int, n_layers: int, channels: int) -> list[tuple[int, int, int, int]]:
    """The ``n_layers + 1`` grids ``(t, h, w, c)`` the pyramid passes through."""
    from scipy.optimize import linear_sum_assignment
    hs = np.cumprod(_factors_desc(patch)).tolist()
    ts = np.cumprod(_factors_desc(temporal_patch)).tolist() if temporal_patch > 1 else []
    scales = [(1, 1, 1, channels)] + [(1, h, h, -(-(h * h * channels) // 64) * 64) for h in hs]
    scales += [(t, hs[-1], hs[-1], hs[-1] * hs[-1] * channels * t * 64) for t in ts]
    size = np.log([s[0] * s[1] * s[2] for s in scales])
    want = n_layers + 1
    ideal = math.log(patch * patch * temporal_patch * channels) * np.arange(want) / (want - 1)
    cost = np.abs(ideal[:, None] - size[None, :])
    if n_layers >= len(scales):
        pick = cost.argmin(1).tolist()
    else:
        rows, cols = linear_sum_assignment(cost)
        pick = [int(c) for _, c in sorted(zip(rows.tolist(), cols.tolist()))]
    pick[0], pick[-1] = 0, len(scales) - 1
    return [scales[i] for i in pick]


def stages(scales, text_hidden: int) -> list[dict]:
    out, n = [], len(scales) - 1
    for i, (s, e) in enumerate(zip(scales[:-1], scales[1:])):
        tf, hf = e[0] // s[0], e[1] // s[1]
        out.append(dict(t_fold=tf, hw_fold=hf, input_dim=s[3] * tf * hf * hf, output_dim=text_hidden if i == n - 1 else e[3], norm=i != n - 1))
    return out


def fold(x, t_fold: int, hw_fold: int):
    """``[T, H, W, C] -> [T / t, H / s, W / s, t s s C]``; inside the new channel axis the order is ``(t_fold, h_fold, w_fold, C)``."""
    T, H, W, C = x.shape
    x = x.view(T // t_fold, t_fold, H // hw_fold, hw_fold, W // hw_fold, hw_fold, C).permute(0, 2, 4, 1, 3, 5, 6)
    return x.reshape(T // t_fold, H // hw_fold, W // hw_fold, t_fold * hw_fold * hw_fold * C)


class HMLP:
    """``proj[i] [output_dim, input_dim]`` and ``norm[i] [output_dim]`` (all stages but the last) for the stages of a plan."""

    def __init__(self, temporal_patch: int, patch: int, n_layers: int, channels: int, text_hidden: int, eps: float = 1e-6):
        self.scales = plan_scales(temporal_patch, patch, n_layers, channels)
        self.stages = stages(self.scales, text_hidden)
        self.temporal_patch, self.patch, self.channels, self.eps = temporal_patch, patch, channels, eps
        self.proj: list = [None] * len(self.stages)
        self.norm: list = [None] * len(self.stages)

    def __call__(self, pixels):
        """``pixels [T, H, W, C]`` (``T, H, W`` multiples of the patch sizes) -> ``[T / tp * H / p * W / p, text_hidden]`` soft tokens."""
        x = pixels
        for st, w, g in zip(self.stages, self.proj, self.norm):
            if st["t_fold"] > 1 or st["hw_fold"] > 1:
                x = fold(x, st["t_fold"], st["hw_fold"])
            shp = x.shape
            y = ops.linear(x.reshape(-1, shp[-1]).contiguous().to(w.dtype), w)
            if st["norm"]:
                y = F.gelu(ops.rmsnorm(y, g, self.eps).float()).to(y.dtype)
            x = y.view(*shp[:-1], y.shape[-1])
        return x.reshape(-1, x.shape[-1])


def dmel_embed(ids, table, norm_gain, levels: int, eps: float = 1e-6):
    """dMel audio: ``ids [frames, n_bins]`` with levels in ``0 .. levels``; bin ``b``'s codebook is rows ``b levels .. (b + 1) levels`` of
    ``table``; the looked-up rows are SUMMED over the bins, then RMS-normed."""
    ids = torch.as_tensor(ids, device=table.device).long()
    if int(ids.max()) >= levels or int(ids.min()) < 0:
        raise ValueError(f"mel level outside 0..{levels}")
    rows = ids + torch.arange(ids.shape[1], device=ids.device) * levels
    return ref.rmsnorm(table[rows].float().sum(1).to(table.dtype), norm_gain, eps) if not table.is_cuda \
        else ops.rmsnorm(table[rows].float().sum(1).to(table.dtype), norm_gain, eps)

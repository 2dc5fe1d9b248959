"""Vocabulary-parallel LM head and sampler: every rank holds ``V / world`` rows of the head, computes the logits of its
shard, reduces them locally to one ``(value, index)`` candidate per token, and the ranks merge the candidates — 8 bytes per
token per rank instead of a ``[tokens, V]`` logits gather.

Greedy: the merge keeps the larger value and, on equal values, the lower global index, so the result is the arg-max of the
whole vocabulary (first maximum wins, the rule of the reference's host arg-max, src/models/gemma/gemma4/lm.rs:22-32).
Tempered sampling uses the Gumbel-max identity: ``argmax_i(logit_i / T + g_i)`` with independent Gumbel noise is a sample of
``softmax(logits / T)``, and an arg-max decomposes over shards, so every rank perturbs its own shard (with its own noise
stream) and the same merge finishes the draw.  Top-k restricts the draw to the k best of the whole vocabulary: each rank
offers its local top-k, the ``k * world`` candidates are gathered, and the k-th best overall becomes the threshold.

On GPUs the merge is one kernel over peer memory (``mary_argmax_merge``: peer stores of the pairs, a flag barrier, a local
pick); the library arm and CPU ranks use ``all_gather``."""
from __future__ import annotations

import torch

from .. import ops


def merge_candidates(vals, idxs):
    """``vals``/``idxs``: ``[world, T]`` candidates (global indices).  Larger value wins; ties go to the lower index."""
    best = vals.max(dim=0).values
    cand = torch.where(vals == best[None, :], idxs, torch.full_like(idxs, torch.iinfo(idxs.dtype).max))
    return cand.min(dim=0).values, best


class VocabParallelHead:
    def __init__(self, weight_shard, rank: int, world: int, softcap: float = 0.0, symm=None, group=None):
        self.w, self.rank, self.world, self.softcap = weight_shard, rank, world, softcap
        self.rows = weight_shard.shape[0]
        self.offset = rank * self.rows
        self.symm, self.group = symm, group

    @staticmethod
    def shard(full_weight, rank: int, world: int):
        V = full_weight.shape[0]
        assert V % world == 0, "vocabulary rows must divide evenly over the ranks"
        n = V // world
        return full_weight[rank * n:(rank + 1) * n].contiguous()

    def _merge(self, val, idx_local):
        if self.world == 1:
            return idx_local, val
        if self.symm is not None and val.is_cuda:
            return self.symm.argmax_merge(val, idx_local, self.offset)
        import torch.distributed as dist
        v = [torch.empty_like(val) for _ in range(self.world)]
        i = [torch.empty_like(idx_local) for _ in range(self.world)]
        dist.all_gather(v, val.contiguous(), group=self.group)
        dist.all_gather(i, (idx_local + self.offset).contiguous(), group=self.group)
        return merge_candidates(torch.stack(v), torch.stack(i))

    def argmax(self, x):
        """Greedy token per row of ``x [T, H]`` -> ``(ids int64, max logit)``; identical on every rank."""
        idx, val = ops.lm_head_argmax(x, self.w, self.softcap)
        return self._merge(val.float(), idx.to(torch.int64))

    def local_logits(self, x):
        lg = ops.linear_f32(x, self.w) if hasattr(ops, "linear_f32") else ops.linear(x, self.w).float()
        if self.softcap:
            lg = self.softcap * torch.tanh(lg / self.softcap)
        return lg

    def sample(self, x, temperature: float, top_k: int = 0, seed: int = 0, step: int = 0):
        """One draw per row from ``softmax(logits / temperature)`` (restricted to the ``top_k`` best of the whole
        vocabulary when ``top_k > 0``)."""
        if temperature <= 0:
            return self.argmax(x)[0]
        lg = self.local_logits(x)
        if top_k:
            k = min(top_k, self.rows)
            loc = torch.topk(lg, k, dim=-1).values                                  # [T, k]
            if self.world > 1:
                import torch.distributed as dist
                parts = [torch.empty_like(loc) for _ in range(self.world)]
                dist.all_gather(parts, loc.contiguous(), group=self.group)
                loc = torch.cat(parts, -1)
            kth = torch.topk(loc, min(top_k, loc.shape[-1]), dim=-1).values[:, -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        g = torch.Generator(device=lg.device).manual_seed((seed * 1000003 + step) * 8 + self.rank)
        u = torch.rand(lg.shape, generator=g, device=lg.device).clamp_min(1e-20)
        pert = lg / temperature - torch.log(-torch.log(u))
        val, idx = pert.max(dim=-1)
        return self._merge(val, idx.to(torch.int64))[0]

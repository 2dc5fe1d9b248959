"""Context parallelism for long prefills: the rows of ONE sequence are cut into contiguous chunks, one per rank; every rank runs all
layers on its own rows only, and after each layer's cache append the ranks exchange that layer's new K / V rows so that a rank's
local paged cache holds every position its (causal) queries can see.  Attention itself stays a purely local kernel over local
pages — remote K / V are copied into this GPU's memory first and read from there (no kernel ever loads a peer's memory, no TMA
touches a peer), which is the form the build plan asks for (the reference has no sequence parallelism at all, it scales length
on one device by banding and query blocking).

The exchange is an all-gather of equal-size row blocks through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo on CPU ranks);
a rank copies in only the chunks BEFORE its own, since later positions are masked anyway.  All ranks build the same page table
(the allocators are deterministic), so a position's slot is the same everywhere.  Memory and attention FLOPs per rank shrink by
the number of ranks for the projections / MLPs and by about half of that for attention (rank ``r`` attends to ``r + 1`` chunks).

``zigzag=True`` balances the causal attention work: the prompt is cut into ``2 * world`` chunks and rank ``r`` takes chunks ``r`` and
``2 * world - 1 - r`` (an early and a late one), so every rank attends to ``2 * world + 1`` half-chunks instead of ``r + 1`` whole ones.
The two chunks are two entries of the rank's batch that share one page-table row."""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..runtime.batch import BatchMeta


class ContextParallel:
    def __init__(self, rank: int, world: int, group=None, zigzag: bool = False):
        self.rank, self.world, self.group, self.zigzag = rank, world, group, zigzag
        self.chunks = None           # zigzag plan: bounds of the 2 * world chunks (None in the contiguous layout)
        self.bounds = None
        self.slots = None
        self.active = False          # layers exchange K / V rows only between begin() and end()

    def begin(self, n_tokens: int, page_table: np.ndarray, page_size: int, device="cpu") -> BatchMeta:
        """Plan one prefill of ``n_tokens`` rows (sequence 0 of ``page_table``): returns the meta of THIS rank's rows."""
        pos = np.arange(n_tokens)
        slots = page_table[0, pos // page_size].astype(np.int64) * page_size + pos % page_size
        self.slots = torch.from_numpy(slots).to(device)
        self.active = True
        if self.zigzag and n_tokens >= 2 * self.world:
            W2 = 2 * self.world
            per = -(-n_tokens // W2)
            self.per = per
            self.chunks = [(min(c * per, n_tokens), min((c + 1) * per, n_tokens)) for c in range(W2)]
            self.bounds = None
            mine = [self.chunks[c] for c in self.my_chunks() if self.chunks[c][1] > self.chunks[c][0]]
            table = np.repeat(page_table[:1], len(mine), 0)
            return BatchMeta.build([b - a for a, b in mine], [b for _, b in mine], table, page_size, device=device)
        self.chunks = None
        per = -(-n_tokens // self.world)
        self.bounds = [(min(r * per, n_tokens), min((r + 1) * per, n_tokens)) for r in range(self.world)]
        self.per = per
        lo, hi = self.bounds[self.rank]
        return BatchMeta.build([hi - lo], [hi], page_table, page_size, device=device)

    def my_chunks(self, rank: int | None = None):
        r = self.rank if rank is None else rank
        return (r, 2 * self.world - 1 - r)

    def end(self) -> None:
        self.active = False

    def rows(self, x):
        """This rank's slice of a per-row tensor of the whole prompt."""
        if self.chunks is not None:
            return torch.cat([x[a:b] for a, b in (self.chunks[c] for c in self.my_chunks())], 0)
        lo, hi = self.bounds[self.rank]
        return x[lo:hi]

    def share(self, kcache, vcache) -> None:
        """After this rank appended its rows of one layer: fetch the rows of all earlier chunks into the local cache."""
        if self.world == 1 or not self.active:
            return
        if self.chunks is not None:
            return self._share_zigzag(kcache, vcache)
        lo, hi = self.bounds[self.rank]
        for cache in ((kcache,) if vcache is kcache or vcache is None else (kcache, vcache)):
            flat = cache.view(-1, *cache.shape[2:])
            mine = torch.zeros(self.per, *flat.shape[1:], dtype=flat.dtype, device=flat.device)
            if hi > lo:
                mine[:hi - lo] = flat[self.slots[lo:hi]]
            got = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(got, mine, group=self.group)
            for r in range(self.rank):                        # later chunks are never visible to this rank's queries
                a, b = self.bounds[r]
                if b > a:
                    flat[self.slots[a:b]] = got[r][:b - a]

    def _halves(self, x, per):
        """A rank's rows ``[early chunk ; late chunk]`` placed at offsets 0 and ``per`` of a ``[2 * per]`` block."""
        (a0, b0), (a1, b1) = (self.chunks[c] for c in self.my_chunks())
        pad = torch.zeros(2 * per, *x.shape[1:], dtype=x.dtype, device=x.device)
        pad[:b0 - a0] = x[:b0 - a0]
        pad[per:per + b1 - a1] = x[b0 - a0:b0 - a0 + b1 - a1]
        return pad

    def _share_zigzag(self, kcache, vcache) -> None:
        per, last = self.per, self.my_chunks()[1]
        for cache in ((kcache,) if vcache is kcache or vcache is None else (kcache, vcache)):
            flat = cache.view(-1, *cache.shape[2:])
            own = torch.cat([flat[self.slots[a:b]] for a, b in (self.chunks[c] for c in self.my_chunks())], 0)
            got = [torch.empty(2 * per, *flat.shape[1:], dtype=flat.dtype, device=flat.device) for _ in range(self.world)]
            dist.all_gather(got, self._halves(own, per), group=self.group)
            for r in range(self.world):
                if r == self.rank:
                    continue
                for half, c in enumerate(self.my_chunks(r)):
                    a, b = self.chunks[c]
                    if c < last and b > a:                      # every chunk before this rank's late chunk is visible to its queries
                        flat[self.slots[a:b]] = got[r][half * per:half * per + b - a]

    def gather_rows(self, x):
        """Concatenate every rank's rows (e.g. logits of the whole prompt) in sequence order."""
        if self.chunks is not None:
            per = self.per
            got = [torch.empty(2 * per, *x.shape[1:], dtype=x.dtype, device=x.device) for _ in range(self.world)]
            dist.all_gather(got, self._halves(x, per), group=self.group)
            out = []
            for c, (a, b) in enumerate(self.chunks):
                owner, half = (c, 0) if c < self.world else (2 * self.world - 1 - c, 1)
                out.append(got[owner][half * per:half * per + b - a])
            return torch.cat(out, 0)
        pad = torch.zeros(self.per, *x.shape[1:], dtype=x.dtype, device=x.device)
        pad[:x.shape[0]] = x
        got = [torch.empty_like(pad) for _ in range(self.world)]
        dist.all_gather(got, pad, group=self.group)
        return torch.cat([got[r][:b - a] for r, (a, b) in enumerate(self.bounds)], 0)

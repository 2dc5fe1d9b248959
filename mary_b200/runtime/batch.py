"""``BatchMeta``: the flattened ragged batch that every model forward consumes.

Rows of all sequences are concatenated: a prefill chunk contributes ``q_len`` rows, a decode step one row
(or ``1+k`` rows with ``k`` speculative drafts).  ``kv_len[i]`` counts the tokens of sequence ``i`` in the
cache AFTER this step's rows were appended, so row ``j`` of sequence ``i`` sits at absolute position
``kv_len[i] - q_len[i] + j`` and may attend to positions ``<=`` its own."""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np

from ..utils import flags
import torch


def check_batch(q_lens, kv_lens, page_table, page_size: int, num_pages: int | None = None) -> None:
    """Host-side bounds check of everything the kernels will index with (run on every ``build`` under ``MARY_DEBUG_CHECKS=1``): the
    lengths are consistent, every page a row can reach is listed, page ids are inside the cache and no page serves two sequences."""
    q_lens, kv_lens, page_table = np.asarray(q_lens), np.asarray(kv_lens), np.asarray(page_table)
    if (q_lens < 0).any() or (kv_lens < q_lens).any():
        raise ValueError(f"inconsistent lengths: q_lens {q_lens.tolist()} kv_lens {kv_lens.tolist()}")
    need = (kv_lens + page_size - 1) // page_size
    if page_table.shape[0] != len(q_lens) or (need > page_table.shape[1]).any():
        raise ValueError(f"page table {page_table.shape} cannot hold sequences of {kv_lens.tolist()} tokens at {page_size} per page")
    used = [page_table[s, :need[s]] for s in range(len(q_lens))]
    flat = np.concatenate(used) if used else np.zeros(0, dtype=np.int64)
    if (flat < 0).any() or (num_pages is not None and (flat >= num_pages).any()):
        raise ValueError(f"page id outside the cache (0..{num_pages}): {flat[(flat < 0) | (flat >= (num_pages or flat.max() + 1))][:4].tolist()}")
    if len(np.unique(flat)) != len(flat):
        raise ValueError("one page is listed for two positions")


@dataclass
class BatchMeta:
    positions: torch.Tensor      # int32 [T] absolute position of every row
    seq_index: torch.Tensor      # int32 [T] which sequence a row belongs to
    q_start: torch.Tensor        # int32 [S+1] row offsets (cumulative)
    kv_len: torch.Tensor         # int32 [S]
    page_table: torch.Tensor     # int32 [S, max_pages]
    slot_mapping: torch.Tensor   # int64 [T] flat cache slot (page * page_size + offset) of every row
    page_size: int
    max_q_len: int
    max_kv_len: int
    num_seqs: int
    num_tokens: int
    all_decode: bool
    # host copies (no device sync needed to read them)
    q_lens_host: np.ndarray | None = None
    kv_lens_host: np.ndarray | None = None

    @staticmethod
    def build(q_lens, kv_lens, page_table: np.ndarray, page_size: int, device="cpu") -> "BatchMeta":
        q_lens = np.asarray(q_lens, dtype=np.int32)
        kv_lens = np.asarray(kv_lens, dtype=np.int32)
        S, T = len(q_lens), int(q_lens.sum())
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        seq_index = np.repeat(np.arange(S, dtype=np.int32), q_lens)
        pos = (np.arange(T, dtype=np.int32) - q_start[seq_index]) + (kv_lens - q_lens)[seq_index]
        pages = page_table[seq_index, pos // page_size].astype(np.int64)
        slots = pages * page_size + (pos % page_size)
        dev = torch.device(device)
        if flags.get("MARY_DEBUG_CHECKS"):
            check_batch(q_lens, kv_lens, page_table, page_size)

        def t(a, dt):
            x = torch.from_numpy(np.ascontiguousarray(a)).to(dt)
            return x.to(dev, non_blocking=True) if dev.type != "cpu" else x
        return BatchMeta(positions=t(pos, torch.int32), seq_index=t(seq_index, torch.int32), q_start=t(q_start, torch.int32),
                         kv_len=t(kv_lens, torch.int32), page_table=t(page_table, torch.int32),
                         slot_mapping=t(slots, torch.int64), page_size=page_size, max_q_len=int(q_lens.max()) if S else 0,
                         max_kv_len=int(kv_lens.max()) if S else 0, num_seqs=S, num_tokens=T,
                         all_decode=bool(S and q_lens.max() == 1), q_lens_host=q_lens, kv_lens_host=kv_lens)

    def repage(self, target: int = 64):
        """Regroup every sequence's pages into ``target``-token pages: returns ``(pick, meta)`` where ``cache[pick]`` viewed as
        ``[-1, target, ...]`` holds the sequences' rows in ``target``-token pages and ``meta`` addresses them (``pick`` lists each
        sequence's pages in order, padded to a multiple of ``target / page_size`` with its first page; the padding lies beyond
        ``kv_len`` and is never visible).  Needs the host copy of the lengths; memoised, since every layer asks for the same."""
        import dataclasses
        memo = self.__dict__.setdefault("_cache", {})
        key = ("repage", target)
        if key not in memo:
            ps = self.page_size
            assert target % ps == 0 and self.kv_lens_host is not None
            per = target // ps
            nbig = [(int(n) + target - 1) // target for n in self.kv_lens_host]
            dev = self.page_table.device
            table = torch.zeros(self.num_seqs, max(max(nbig), 1), dtype=torch.int32, device=dev)
            picks, off = [], 0
            for s, n in enumerate(nbig):
                have = (int(self.kv_lens_host[s]) + ps - 1) // ps
                row = self.page_table[s, :have]
                if n * per > have:
                    row = torch.cat([row, self.page_table[s, :1].expand(n * per - have)])
                picks.append(row)
                table[s, :n] = torch.arange(off, off + n, dtype=torch.int32, device=dev)
                off += n
            memo[key] = (torch.cat(picks).long(), dataclasses.replace(self, page_table=table, page_size=target))
        return memo[key]

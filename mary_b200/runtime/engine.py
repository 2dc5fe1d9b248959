"""Serving engine: native scheduler + paged cache + a model's flattened-batch forward.

One ``step`` = the scheduler packs decode rows and prefill chunks into a batch (``_core.so``), the ids go to the
device through pinned memory, the model runs once, the sampled tokens come back in one small device-to-host
copy and are committed (with rollback of rejected speculative rows).  The reference runs one prefill or one
decode pass per loop iteration with a blocking logits readback and host arg-max per row
(src/bin/inkling_forward.rs:3908-5112, src/models/gemma/gemma4/lm.rs:164-201); here only token ids cross."""
from __future__ import annotations

import ctypes
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from .batch import BatchMeta
from .kv_cache import PagedKVCache, _declare


@dataclass
class StepStats:
    tokens_in: int = 0
    tokens_out: int = 0
    seqs: int = 0
    seconds: float = 0.0


class Engine:
    def __init__(self, model, cache: PagedKVCache, max_tokens: int = 8192, max_seqs: int = 256,
                 prefill_chunk: int = 2048, device="cpu", eos_ids=(), sampler=None, draft=None, spec_k: int = 0, metrics=None):
        self.model, self.cache, self.device = model, cache, torch.device(device)
        self.lib = cache.alloc.lib
        _declare(self.lib)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.h = self.lib.sched_create(cache.alloc.h, max_tokens, max_seqs, prefill_chunk)
        self.eos = set(int(e) for e in eos_ids)
        self.sampler = sampler
        self.draft, self.spec_k = draft, spec_k
        self._next_id = 1
        self.outputs: dict[int, list[int]] = {}
        self.first_token_time: dict[int, float] = {}
        self.submit_time: dict[int, float] = {}
        pin = self.device.type == "cuda"
        i32 = lambda n: torch.empty(n, dtype=torch.int32, pin_memory=pin)  # noqa: E731
        self._tok, self._pos, self._sidx = i32(max_tokens), i32(max_tokens), i32(max_tokens)
        self._qs, self._ql, self._dec, self._srow = i32(max_seqs), i32(max_seqs), i32(max_seqs), i32(max_seqs)
        self._ids = torch.empty(max_seqs, dtype=torch.int64, pin_memory=pin)
        self._nt = ctypes.c_int32()
        self.stats: list[StepStats] = []
        self.accepted_hist: list[int] = []
        self.metrics = metrics              # utils.metrics.MetricsLog or None: one "step" row per step, one "request" row per first token

    # ------------------------------------------------------------------ requests
    def add_request(self, ids, max_new: int) -> int:
        rid = self._next_id
        self._next_id += 1
        a = np.ascontiguousarray(ids, dtype=np.int32)
        if self.lib.sched_add(self.h, rid, a.ctypes.data, len(a), max_new) != 0:
            raise ValueError(f"request refused: {len(a)} prompt tokens + {max_new} new tokens (an empty prompt, a negative budget, "
                             "or more pages than the KV pool holds)")
        self.outputs[rid] = []
        self.submit_time[rid] = time.perf_counter()
        return rid

    def pending(self) -> int:
        return self.lib.sched_num_waiting(self.h) + self.lib.sched_num_running(self.h)

    # ------------------------------------------------------------------ one step
    def step(self) -> StepStats:
        t0 = time.perf_counter()
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        ns = self.lib.sched_next(self.h, p(self._tok), p(self._pos), p(self._sidx), p(self._ids), p(self._qs),
                                 p(self._ql), p(self._dec), p(self._srow), ctypes.byref(self._nt))
        nt = self._nt.value
        if ns == 0:
            return StepStats()
        seq_ids = self._ids[:ns].numpy()
        q_lens = self._ql[:ns].numpy()
        table, kv_lens = self.cache.alloc.page_table(seq_ids)
        meta = BatchMeta.build(q_lens, kv_lens, table, self.cache.page_size, self.device)
        ids = self._tok[:nt].to(self.device, non_blocking=True)
        srow = self._srow[:ns].numpy()
        is_dec = self._dec[:ns].numpy()
        # rows whose logits are needed: every row of a decode group (for draft verification), the last prefill row
        rows, owner = [], []
        for i in range(ns):
            if srow[i] < 0:
                continue
            n = int(q_lens[i]) if is_dec[i] else 1
            for j in range(n):
                rows.append(int(srow[i]) + j)
                owner.append(i)
        out = StepStats(tokens_in=nt, seqs=ns)
        with torch.no_grad():
            if rows:
                rows_t = torch.tensor(rows, dtype=torch.long).to(self.device)
                if self.sampler is None:
                    toks = self.model.greedy(ids, meta, self.cache, rows_t)
                else:
                    toks = self.sampler(self.model(ids, meta, self.cache, rows_t))
                toks = toks.to("cpu").numpy()
            else:
                self.model.hidden(ids, meta, self.cache)
                toks = np.zeros(0, dtype=np.int64)
        now = time.perf_counter()
        # commit
        k = 0
        fed = self._tok[:nt].numpy()
        qs = self._qs[:ns].numpy()
        for i in range(ns):
            if srow[i] < 0:
                continue
            rid = int(seq_ids[i])
            n = int(q_lens[i]) if is_dec[i] else 1
            pred = toks[k:k + n]
            k += n
            if is_dec[i] and n > 1:
                drafts = fed[qs[i] + 1:qs[i] + n]
                acc = 0
                while acc < n - 1 and int(pred[acc]) == int(drafts[acc]):
                    acc += 1
                new = [int(t) for t in drafts[:acc]] + [int(pred[acc])]
                accepted, fed_rows = acc + 1, n
                self.accepted_hist.append(acc)
            else:
                new = [int(pred[0])]
                accepted, fed_rows = 1, 1
            done = False
            for j, t in enumerate(new):
                if t in self.eos:
                    new, done = new[:j + 1], True
                    break
            if rid not in self.first_token_time:
                self.first_token_time[rid] = now
                if self.metrics is not None:
                    self.metrics.emit("request", id=rid, ttft_s=now - self.submit_time[rid])
            self.outputs[rid].extend(new)
            self.lib.sched_commit(self.h, rid, accepted, fed_rows, new[-1], 1 if done else 0)
            out.tokens_out += len(new)
        out.seconds = time.perf_counter() - t0
        self.stats.append(out)
        if self.metrics is not None:
            self.metrics.emit("step", seconds=out.seconds, tokens_in=out.tokens_in, tokens_out=out.tokens_out, seqs=out.seqs)
        return out

    def run(self, max_steps: int = 1 << 30) -> None:
        n = 0
        while self.pending() and n < max_steps:
            s = self.step()
            n += 1
            if s.seqs == 0:
                raise RuntimeError("scheduler made no progress: the KV cache is too small for the waiting requests")

    def generate(self, prompts, max_new: int) -> list[list[int]]:
        rids = [self.add_request(p, max_new) for p in prompts]
        self.run()
        return [self.outputs[r][:max_new] for r in rids]

    def __del__(self):
        try:
            self.lib.sched_destroy(self.h)
        except Exception:
            pass

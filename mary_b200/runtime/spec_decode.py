"""Fixed-batch decode loop with MTP speculative decoding, device-resident state and CUDA-graph replay.

One step, for every sequence of the batch:
  1. VERIFY: feed ``[pending, draft_1 .. draft_k]`` (k+1 rows) through the model; row ``j``'s arg-max is the model's token
     for the position after row ``j``.
  2. ACCEPT: the leading run of drafts that equal the model's tokens is kept (``a`` of them); ``a + 1`` tokens are emitted
     (the accepted drafts plus the model's token after the last kept row), which becomes the next ``pending``; the cache
     length grows by ``a + 1`` — rejected rows simply fall beyond the new length and are overwritten by the next step,
     so they leave no trace (the reference's commit/rollback: src/models/inkling/burn.rs:441-461,
     acceptance rule src/bin/inkling_forward.rs:5016-5032).
  3. DRAFT: the MTP layer runs over the fed rows (filling its own cache rows) and its output at the last kept row, given
     the new pending token, predicts draft_1; further drafts re-apply the MTP layer to its own hidden state.

All of it runs on the device without host decisions, so a whole step is one CUDA graph; the host only copies the emitted
tokens out (and, in host-driven mode, the fed tokens in)."""
from __future__ import annotations

import numpy as np
import torch

from .batch import BatchMeta
from .kv_cache import PagedKVCache


class SpecDecoder:
    def __init__(self, model, cache: PagedKVCache, batch: int, spec_k: int = 0, max_len: int = 8192, device="cuda",
                 use_graph: bool = True):
        self.model, self.cache, self.B, self.k = model, cache, batch, spec_k
        self.dev = torch.device(device)
        self.use_graph = use_graph and self.dev.type == "cuda"
        self.max_len = max_len
        ps = cache.page_size
        self.max_pages = (max_len + ps - 1) // ps
        B, R = batch, 1 + spec_k
        for s in range(B):                               # all pages up front: the step never allocates
            cache.alloc.extend(s, max_len)
        table, _ = cache.alloc.page_table(list(range(B)), self.max_pages)
        self.page_table = torch.from_numpy(table).to(self.dev)
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.kv_before = torch.zeros(B, **i32)           # committed cache length per sequence
        self.fed = torch.zeros(B, R, **i32)              # [pending, drafts...]
        self.emitted = torch.zeros(B, R, **i32)          # tokens produced by the last step (first n_emitted valid)
        self.n_emitted = torch.zeros(B, **i32)
        self.j = torch.arange(R, **i32)
        # static metas (tensors are updated in place every step)
        self.meta_v = self._static_meta(R)
        self.meta_d = self._static_meta(1) if spec_k > 0 else None
        self.graph = None
        self.steps = 0
        # host-side upper bound of the longest committed length: every step may commit up to 1 + k tokens and writes rows up to
        # 1 + k positions past the committed length, so a step is refused before launch (or replay) once it could leave max_len
        self.len_bound = 0

    def _static_meta(self, q_len: int) -> BatchMeta:
        B, dev = self.B, self.dev
        i32 = dict(dtype=torch.int32, device=dev)
        m = BatchMeta(positions=torch.zeros(B * q_len, **i32), seq_index=torch.arange(B, **i32).repeat_interleave(q_len),
                      q_start=torch.arange(0, B * q_len + 1, q_len, **i32), kv_len=torch.zeros(B, **i32),
                      page_table=self.page_table, slot_mapping=torch.zeros(B * q_len, dtype=torch.int64, device=dev),
                      page_size=self.cache.page_size, max_q_len=q_len, max_kv_len=self.max_len, num_seqs=B,
                      num_tokens=B * q_len, all_decode=(q_len == 1), q_lens_host=np.full(B, q_len, dtype=np.int32),
                      kv_lens_host=None)
        return m

    def _set_meta(self, m: BatchMeta, pos0, q_len: int):
        """Rows of sequence b sit at positions pos0[b] .. pos0[b] + q_len - 1."""
        pos = (pos0[:, None] + self.j[None, :q_len]).reshape(-1)
        m.positions.copy_(pos)
        m.kv_len.copy_(pos0 + q_len)
        ps = self.cache.page_size
        page = torch.gather(self.page_table, 1, (pos.view(self.B, q_len) // ps).long()).reshape(-1)
        m.slot_mapping.copy_(page.long() * ps + (pos % ps).long())

    # ------------------------------------------------------------------ state
    def set_context(self, kv_len, pending, drafts=None):
        """Start decoding from a populated cache: committed lengths, the next token to feed and optional drafts."""
        self.kv_before.copy_(torch.as_tensor(kv_len, dtype=torch.int32).to(self.dev))
        self.len_bound = int(np.max(np.asarray(kv_len))) if np.size(kv_len) else 0
        self.fed[:, 0].copy_(torch.as_tensor(pending, dtype=torch.int32).to(self.dev))
        if self.k:
            d = drafts if drafts is not None else torch.zeros(self.B, self.k, dtype=torch.int32)
            self.fed[:, 1:].copy_(torch.as_tensor(d, dtype=torch.int32).to(self.dev))

    def prefill(self, prompts, chunk: int = 512):
        """Run equal-length prompts ``[B, L]`` through the model in chunks (filling the main and the MTP cache rows) and
        leave the decoder ready: ``pending`` = first generated token, drafts from the MTP layer.  Returns ``pending``."""
        ids = torch.as_tensor(np.asarray(prompts), dtype=torch.int32).to(self.dev)
        B, L = ids.shape
        assert B == self.B
        table = self.page_table.cpu().numpy()
        pending = None
        with torch.no_grad():
            for c0 in range(0, L, chunk):
                n = min(chunk, L - c0)
                meta = BatchMeta.build([n] * B, [c0 + n] * B, table, self.cache.page_size, self.dev)
                flat = ids[:, c0:c0 + n].reshape(-1)
                last = torch.arange(B, device=self.dev) * n + (n - 1)
                if self.k == 0:
                    if c0 + n == L:
                        pending = self.model.greedy(flat, meta, self.cache, last).to(torch.int32)
                    else:
                        self.model.trunk(flat, meta, self.cache)
                    continue
                # the vocabulary projection runs for the last row of each prompt in the last chunk only
                head = last if c0 + n == L else last[:0]
                tok, h = self.model.verify(flat, meta, self.cache, rows=head)
                nxt = torch.cat([ids[:, c0 + 1:c0 + n], ids[:, min(c0 + n, L - 1):min(c0 + n, L - 1) + 1]], 1)
                if c0 + n == L:
                    pending = tok.to(torch.int32)
                    nxt[:, -1] = pending
                d_tok, d_h = self.model.draft(0, h, nxt.reshape(-1), meta, self.cache, rows=head)
            self.kv_before.fill_(L)
            self.len_bound = L
            self.fed[:, 0].copy_(pending)
            if self.k:
                drafts = [d_tok.to(torch.int32)]
                h_last = d_h[last]
                for d in range(1, self.k):
                    self._set_meta(self.meta_d, self.kv_before + (d - 1), 1)
                    t2, h_last = self.model.draft(d, h_last, drafts[-1], self.meta_d, self.cache)
                    drafts.append(t2.to(torch.int32))
                self.fed[:, 1:].copy_(torch.stack(drafts, 1))
        return pending

    # ------------------------------------------------------------------ one step on the device
    def _step_device(self):
        B, k, R = self.B, self.k, 1 + self.k
        self._set_meta(self.meta_v, self.kv_before, R)
        ids = self.fed.reshape(-1)
        if k == 0:
            tok = self.model.greedy(ids, self.meta_v, self.cache, slice(None)).to(torch.int32)
            self.emitted[:, 0].copy_(tok)
            self.n_emitted.fill_(1)
            self.kv_before.add_(1)
            self.fed[:, 0].copy_(tok)
            return
        tok, h = self.model.verify(ids, self.meta_v, self.cache)
        pred = tok.to(torch.int32).view(B, R)
        match = (pred[:, :k] == self.fed[:, 1:]).to(torch.int32)
        acc = torch.cumprod(match, dim=1).sum(dim=1).to(torch.int32)            # accepted drafts, 0..k
        new_pending = torch.gather(pred, 1, acc[:, None].long())[:, 0]
        # emitted = accepted drafts then the model's token
        em = torch.where(self.j[None, :] < acc[:, None], torch.cat([self.fed[:, 1:], self.fed[:, :1]], 1), new_pending[:, None])
        self.emitted.copy_(em)
        self.n_emitted.copy_(acc + 1)
        # DRAFT 1: MTP over every fed row (next token of row j = fed[j+1], of the last kept row = new pending)
        nxt = torch.cat([self.fed[:, 1:], self.fed[:, :1]], 1)
        nxt = torch.where(self.j[None, :] == acc[:, None], new_pending[:, None], nxt)
        d_tok, d_h = self.model.draft(0, h, nxt.reshape(-1), self.meta_v, self.cache)
        row = (torch.arange(B, device=self.dev) * R + acc.long())
        drafts = [d_tok[row].to(torch.int32)]
        h_last = d_h[row]
        self.kv_before.add_(acc + 1)
        for d in range(1, k):
            self._set_meta(self.meta_d, self.kv_before + (d - 1), 1)
            t2, h_last = self.model.draft(d, h_last, drafts[-1], self.meta_d, self.cache)
            drafts.append(t2.to(torch.int32))
        self.fed[:, 0].copy_(new_pending)
        self.fed[:, 1:].copy_(torch.stack(drafts, 1))

    def capture(self, warmup: int = 2):
        """Warm up eagerly (allocator, lazy kernel attributes), then record the step into a CUDA graph."""
        if not self.use_graph:
            return
        saved = (self.kv_before.clone(), self.fed.clone())
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(warmup):
                self._step_device()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.kv_before.copy_(saved[0]); self.fed.copy_(saved[1])
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self._step_device()
        self.kv_before.copy_(saved[0]); self.fed.copy_(saved[1])

    def step(self):
        """Run one step; results stay on the device (``emitted``, ``n_emitted``)."""
        R = 1 + self.k
        if self.len_bound + 2 * R > self.max_len:
            # the rows of this step (and the draft rows behind them) would index past the page table: refuse on the host
            raise RuntimeError(f"decode step refused: up to {self.len_bound} committed tokens + {2 * R} rows exceed max_len {self.max_len}")
        self.len_bound += R
        if self.graph is not None:
            self.graph.replay()
        else:
            with torch.no_grad():
                self._step_device()
        self.steps += 1

    def step_host(self, fed_pinned=None, out_pinned=None):
        """Host-driven step: copy the fed tokens in from pinned memory (when given), run, copy the result out."""
        if fed_pinned is not None:
            self.fed.copy_(fed_pinned, non_blocking=True)
        self.step()
        if out_pinned is not None:
            out_pinned[0].copy_(self.emitted, non_blocking=True)
            out_pinned[1].copy_(self.n_emitted, non_blocking=True)
            out_pinned[2].copy_(self.fed, non_blocking=True)
            torch.cuda.current_stream().synchronize()

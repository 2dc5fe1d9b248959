"""Pipeline parallelism: a decoder cut into consecutive layer ranges, one per rank, with activations handed from stage to
stage by point-to-point sends (NCCL send/recv on a side stream on GPUs, gloo on CPU ranks) and several cohorts of sequences
in flight so that no stage idles.

What the reference does with two processes over TCP — a head stage owning layers ``[0, s)``, a tail owning ``[s, L)`` plus
the LM head, a wire message of a 24-byte header ``(n, pos0, cohort)`` and ``[n, hidden]`` activations, token replies, a
byte-balanced split point and ``c`` cohorts with ``c - 1`` answers in flight (src/bin/inkling_forward.rs:1192-1271,
724-760, 18-61) — is here any number of stages over ``torch.distributed``.  The message is the same: a 3-int header and the
bf16/f32 residual rows; tokens travel back from the last stage to the first."""
from __future__ import annotations

from collections import deque

import numpy as np
import torch
import torch.distributed as dist


def balanced_split(layer_bytes, n_stages: int):
    """Cut ``len(layer_bytes)`` layers into ``n_stages`` consecutive non-empty ranges whose largest byte sum is minimal
    (the reference's byte-balanced split, src/bin/inkling_forward.rs:18-61).  Returns ``[(lo, hi), ...]``."""
    w = [int(b) for b in layer_bytes]
    L = len(w)
    assert 1 <= n_stages <= L
    pre = np.concatenate([[0], np.cumsum(w)])
    INF = float("inf")
    best = [[INF] * (L + 1) for _ in range(n_stages + 1)]
    cut = [[0] * (L + 1) for _ in range(n_stages + 1)]
    best[0][0] = 0
    for s in range(1, n_stages + 1):
        for hi in range(s, L + 1):
            for lo in range(s - 1, hi):
                v = max(best[s - 1][lo], pre[hi] - pre[lo])
                if v < best[s][hi]:
                    best[s][hi], cut[s][hi] = v, lo
    out, hi = [], L
    for s in range(n_stages, 0, -1):
        lo = cut[s][hi]
        out.append((lo, hi))
        hi = lo
    return out[::-1]


class PipeChannel:
    """Typed messages between stages.  Activations travel forward on ``fwd_group``, tokens travel back on ``back_group``;
    on CUDA these must be two process groups (two NCCL communicators), because the forward transfers run on a side stream
    — so the next cohort's compute overlaps them — while the token replies run on the compute stream, and operations of one
    communicator must not be issued from two streams.  Sends never block the host: on CPU ranks they are ``isend`` handles
    that are reaped later, so a stage that is sending an answer cannot stall a stage that is sending it work."""

    def __init__(self, hidden: int, max_rows: int, dtype, device, fwd_group=None, back_group=None):
        self.fwd, self.back, self.dev = fwd_group, back_group, torch.device(device)
        self.H, self.max_rows, self.dtype = hidden, max_rows, dtype
        self.cuda = self.dev.type == "cuda"
        if self.cuda:
            assert fwd_group is not None and back_group is not None and fwd_group is not back_group, \
                "CUDA pipelines need separate process groups for activations and token replies"
        self.side = torch.cuda.Stream(self.dev) if self.cuda else None
        self._pending = []

    def _reap(self, all_: bool = False):
        keep = []
        for w, bufs in self._pending:
            if all_:
                w.wait()
            elif not w.is_completed():
                keep.append((w, bufs))
        self._pending = [] if all_ else keep

    def _send(self, t, dst, group):
        self._pending.append((dist.isend(t, dst, group=group), t))

    def _hdr(self, n=0, pos0=0, cohort=0):
        return torch.tensor([n, pos0, cohort], dtype=torch.int64, device=self.dev)

    def send_rows(self, dst: int, rows, pos0: int, cohort: int):
        n = rows.shape[0]
        assert n <= self.max_rows and rows.shape[1] == self.H
        rows = rows.contiguous()
        if self.cuda:
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                self._send(self._hdr(n, pos0, cohort), dst, self.fwd)
                self._send(rows, dst, self.fwd)
                rows.record_stream(self.side)
        else:
            self._send(self._hdr(n, pos0, cohort), dst, self.fwd)
            self._send(rows, dst, self.fwd)
        self._reap()

    def recv_rows(self, src: int):
        hdr = self._hdr()
        if self.cuda:
            with torch.cuda.stream(self.side):
                dist.recv(hdr, src, group=self.fwd)
                n, pos0, cohort = (int(v) for v in hdr.tolist())       # the row count sizes the next receive
                rows = torch.empty(n, self.H, dtype=self.dtype, device=self.dev)
                dist.recv(rows, src, group=self.fwd)
            torch.cuda.current_stream().wait_stream(self.side)
        else:
            dist.recv(hdr, src, group=self.fwd)
            n, pos0, cohort = (int(v) for v in hdr.tolist())
            rows = torch.empty(n, self.H, dtype=self.dtype, device=self.dev)
            dist.recv(rows, src, group=self.fwd)
        return rows, pos0, cohort

    def send_tokens(self, dst: int, toks, cohort: int):
        pad = torch.zeros(2 + self.max_rows, dtype=torch.int64, device=self.dev)
        pad[0], pad[1] = cohort, toks.numel()
        pad[2:2 + toks.numel()] = toks.to(torch.int64).reshape(-1)
        self._send(pad, dst, self.back)
        self._reap()

    def recv_tokens(self, src: int):
        pad = torch.zeros(2 + self.max_rows, dtype=torch.int64, device=self.dev)
        dist.recv(pad, src, group=self.back)
        cohort, n = int(pad[0]), int(pad[1])
        return pad[2:2 + n].clone(), cohort

    def drain(self):
        self._reap(all_=True)


class PipelineStage:
    """One rank of a layer pipeline over a decoder that offers ``trunk_range`` (layers ``[lo, hi)``), ``norm`` and a head.

    Every stage holds the KV cache rows of its own layers only (the cache object is indexed by absolute layer number, the
    other layers' pages are simply never touched).  ``cohorts`` independent groups of sequences circulate: the first stage
    feeds cohort ``c + 1`` while cohort ``c`` is still further down the pipe, and waits for an answer only when all
    cohorts are in flight."""

    def __init__(self, model, ranges, rank: int, channel: PipeChannel):
        self.model, self.ranges, self.rank, self.ch = model, ranges, rank, channel
        self.lo, self.hi = ranges[rank]
        self.first, self.last = rank == 0, rank == len(ranges) - 1
        self.n_stages = len(ranges)

    def forward_stage(self, inp, meta, cache):
        return self.model.trunk_range(inp, self.lo, self.hi, meta, cache)

    def tail_tokens(self, h, rows):
        from .. import ops
        x = ops.rmsnorm(h, self.model.norm, self.model.cfg.rms_norm_eps)[rows]
        tok, _ = ops.lm_head_argmax(x, self.model.head_weight())
        return tok

    # -- the generation loop ------------------------------------------------------------------------------------
    def generate(self, cohorts_prompts, n_new: int, make_meta):
        """Greedy generation of ``n_new`` tokens for every cohort (a list of equal-length prompt batches ``[B, L]``).
        ``make_meta(cohort, q_len, kv_len)`` returns ``(meta, cache)`` of that cohort for a step that feeds ``q_len``
        rows per sequence ending at cache length ``kv_len``.  Returns, on the first stage, ``[cohort][B][n_new]`` tokens."""
        C = len(cohorts_prompts)
        B, L = cohorts_prompts[0].shape
        dev = self.ch.dev
        out = [[[] for _ in range(B)] for _ in range(C)]
        # work items, in the order the first stage issues them: (cohort, step) with step 0 = prefill
        total = C * n_new
        inflight = deque()
        fed = [torch.as_tensor(p, dtype=torch.int32, device=dev) for p in cohorts_prompts]
        kv = [0] * C
        issued = done = 0
        step_of = [0] * C
        order = deque((c, 0) for c in range(C))
        with torch.no_grad():
            while done < total:
                if self.first:
                    while order and len(inflight) < C:
                        c, s = order.popleft()
                        ids = fed[c].reshape(-1)
                        q = fed[c].shape[1]
                        meta, cache = make_meta(c, q, kv[c] + q)
                        h = self.forward_stage(ids, meta, cache)
                        kv[c] += q
                        if self.last:
                            last_rows = torch.arange(B, device=dev) * q + (q - 1)
                            inflight.append((c, self.tail_tokens(h, last_rows)))
                        else:
                            self.ch.send_rows(self.rank + 1, h, kv[c] - q, c)
                            inflight.append((c, None))
                        issued += 1
                    c, tok = inflight.popleft()
                    if tok is None:
                        tok, c2 = self.ch.recv_tokens(self.n_stages - 1)
                        assert c2 == c, "answers come back in issue order"
                    for b in range(B):
                        out[c][b].append(int(tok[b]))
                    done += 1
                    step_of[c] += 1
                    if step_of[c] < n_new:
                        fed[c] = tok.to(torch.int32).view(B, 1)
                        order.append((c, step_of[c]))
                else:
                    h_in, pos0, c = self.ch.recv_rows(self.rank - 1)
                    q = h_in.shape[0] // B
                    meta, cache = make_meta(c, q, pos0 + q)
                    h = self.forward_stage(h_in, meta, cache)
                    if self.last:
                        last_rows = torch.arange(B, device=dev) * q + (q - 1)
                        self.ch.send_tokens(0, self.tail_tokens(h, last_rows), c)
                    else:
                        self.ch.send_rows(self.rank + 1, h, pos0, c)
                    done += 1
        self.ch.drain()
        return out if self.first else None

"""Library baseline of the flagship decode step: the same K3-class MLA + MoE decoder with 2-token MTP speculation, written with
library calls only — ``torch.matmul`` / ``torch.bmm`` (cuBLAS), ``torch._grouped_mm`` for the experts, ``torch.distributed``
(NCCL) ``all_reduce`` / ``all_to_all_single`` / ``all_gather`` for the collectives — and none of this package's kernels.

It is the denominator of ``vs_baseline`` in ``bench.py``: same architecture, batch, context, speculation, parallel layout and
synthetic data as the product arm, run on the same GPUs right after it.  Two differences are inherent and printed with the
result: the experts are bf16 (this torch has no block-scaled NVFP4 grouped GEMM), so every expert byte counts 3.56 times,
and the step is launched eagerly (the expert all-to-all sizes pass through the host, as in the usual library recipe).

The reference has neither arm: it serves Inkling over a two-stage TCP pipeline (src/bin/inkling_forward.rs:1192-1271) and
prices tensor parallelism without building it (:68-99)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as Fn


def _rms(x, w, eps):
    return Fn.rms_norm(x, (x.shape[-1],), w, eps)


def _rope(x, pos, inv_freq):
    """Split-half rotation of the last dimension of ``x[T, ..., d]`` at integer positions ``pos[T]``."""
    ang = pos.float()[:, None] * inv_freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (inv_freq.shape[0],)
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], -1).to(x.dtype)


class LibraryK3Decoder:
    """``layout``: ``single`` | ``replicated`` (tokens replicated, heads and experts sharded, sums by all-reduce) | ``a2a`` (tokens on
    their home rank, full attention everywhere, experts reached by all-to-all)."""

    def __init__(self, cfg, rank: int, world: int, layout: str, batch_local: int, spec_k: int, max_len: int, device, slabs: int | None = None,
                 seed: int = 0):
        import torch.distributed as dist
        self.dist = dist
        self.c, self.rank, self.world, self.layout = cfg, rank, world, layout
        self.B, self.k, self.R, self.max_len, self.dev = batch_local, spec_k, 1 + spec_k, max_len, torch.device(device)
        c = cfg
        tp = world if layout == "replicated" else 1
        ep = world if layout in ("replicated", "a2a") else 1
        self.tp, self.ep = tp, ep
        self.Hh = c.num_attention_heads // tp
        self.e_local = c.n_routed_experts // ep
        g = torch.Generator(device=self.dev).manual_seed(seed)
        bf = dict(dtype=torch.bfloat16, device=self.dev)

        def W(*shape):
            return torch.empty(*shape, **bf).normal_(0.0, 0.02, generator=g)

        def ones(n):
            return torch.ones(n, **bf)

        H, F = c.hidden_size, c.moe_intermediate_size
        self.n_layers = c.num_hidden_layers + c.num_mtp_layers
        self.embed = W(c.vocab_size, H)
        self.head = W(c.vocab_size // tp, H)
        self.norm = ones(H)
        self.layers = []
        n_moe = sum(1 for i in range(c.num_hidden_layers) if not c.is_dense(i)) + c.num_mtp_layers
        slab_bytes = (self.e_local + 2) * 3 * H * F * 2
        if slabs is None:
            free, _ = torch.cuda.mem_get_info(self.dev)
            kv = self.n_layers * self.B * max_len * 576 * 2
            attn = self.n_layers * (2112 * H + self.Hh * 192 * 1536 + 2 * self.Hh * 512 * 128 + H * self.Hh * 128) * 2
            slabs = int(max(1, min(n_moe, (free - kv - attn - 2 * c.vocab_size * H * 2 // tp - (10 << 30)) // slab_bytes)))
        self.slabs, self.n_moe = slabs, n_moe
        slab_list = []
        moe_i = 0
        for i in range(self.n_layers):
            L = dict(w_qa_kva=W(c.q_lora_rank + 576, H), qa_norm=ones(c.q_lora_rank), kv_norm=ones(512), w_qb=W(self.Hh * 192, c.q_lora_rank),
                     w_uk=W(self.Hh, 512, 128), w_uv=W(self.Hh, 128, 512), w_o=W(H, self.Hh * 128), ln_attn=ones(H), ln_ffn=ones(H))
            dense = c.is_dense(i) and i < c.num_hidden_layers
            if dense:
                L["w_gu"], L["w_down"] = W(2 * c.dense_intermediate_size // tp, H), W(H, c.dense_intermediate_size // tp)
            else:
                L["w_router"] = W(c.n_routed_experts, H)
                L["bias"] = torch.zeros(c.n_routed_experts, dtype=torch.float32, device=self.dev)
                if moe_i < slabs:
                    # routed experts of this rank followed by the shared expert, [E, K, N] for the grouped GEMM; with replicated
                    # tokens one more all-zero group takes the entries that belong to other ranks
                    G = self.e_local + 1 + (1 if layout == "replicated" and world > 1 else 0)
                    w13, w2 = W(G, H, 2 * F), W(G, F, H)
                    if G > self.e_local + 1:
                        w13[-1].zero_()
                        w2[-1].zero_()
                    slab_list.append((w13, w2))
                L["w13"], L["w2"] = slab_list[moe_i % slabs]
                moe_i += 1
            if i >= c.num_hidden_layers:
                L["h_norm"], L["e_norm"], L["proj"], L["out_norm"] = ones(H), ones(H), W(H, 2 * H), ones(H)
            self.layers.append(L)
        self.inv_freq = (c.rope_theta ** (-torch.arange(0, 32, device=self.dev, dtype=torch.float32) / 32))
        self.cache = [torch.empty(self.B, max_len, 576, **bf).normal_(0.0, 1.0, generator=g) for _ in range(self.n_layers)]
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.kv_before = torch.zeros(self.B, **i32)
        self.fed = torch.zeros(self.B, self.R, **i32)
        self.n_emitted = torch.zeros(self.B, **i32)
        self.j = torch.arange(self.R, **i32)
        self.key_pos = torch.arange(max_len, device=self.dev)
        self.grouped = hasattr(torch, "_grouped_mm")
        self.expert_bytes_per_layer = slab_bytes

    # ---------------------------------------------------------------- pieces
    def _reduce(self, x):
        if self.layout == "replicated" and self.world > 1:
            self.dist.all_reduce(x)
        return x

    def _attention(self, L, li, x, pos, b_idx):
        c = self.c
        T = x.shape[0]
        qakv = x @ L["w_qa_kva"].T
        qa = _rms(qakv[:, :c.q_lora_rank], L["qa_norm"], 1e-6)
        ckv = _rms(qakv[:, c.q_lora_rank:c.q_lora_rank + 512], L["kv_norm"], 1e-6)
        kr = _rope(qakv[:, c.q_lora_rank + 512:], pos, self.inv_freq)
        self.cache[li][b_idx, pos.long()] = torch.cat([ckv, kr], -1)
        qb = (qa @ L["w_qb"].T).view(T, self.Hh, 192)
        q_lat = torch.einsum("thd,hnd->thn", qb[..., :128], L["w_uk"])
        q_rope = _rope(qb[..., 128:], pos, self.inv_freq)
        q = torch.cat([q_lat, q_rope], -1)                                     # [T, Hh, 576]
        R = T // self.B
        qg = q.view(self.B, R * self.Hh, 576)
        keys = self.cache[li]                                                  # [B, max_len, 576]
        s = torch.bmm(qg, keys.transpose(1, 2)).float() * c.attn_scale          # [B, R * Hh, max_len]
        qpos = pos.view(self.B, R, 1).expand(self.B, R, self.Hh).reshape(self.B, R * self.Hh, 1)
        s = s.masked_fill(self.key_pos.view(1, 1, -1) > qpos, float("-inf"))
        p = torch.softmax(s, -1).to(torch.bfloat16)
        o_lat = torch.bmm(p, keys[..., :512]).view(T, self.Hh, 512)
        o = torch.einsum("thk,hnk->thn", o_lat, L["w_uv"]).reshape(T, self.Hh * 128)
        return self._reduce(o @ L["w_o"].T)

    def _route(self, L, x):
        c = self.c
        scores = torch.sigmoid((x @ L["w_router"].T).float())
        sel = scores + L["bias"]
        T = x.shape[0]
        if c.n_group > 1:
            gs = sel.view(T, c.n_group, -1).topk(2, -1).values.sum(-1)
            keep = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, gs.topk(c.topk_group, -1).indices, True)
            sel = sel.view(T, c.n_group, -1).masked_fill(~keep[:, :, None], float("-inf")).view(T, -1)
        idx = sel.topk(c.num_experts_per_tok, -1).indices
        w = scores.gather(1, idx)
        w = w / (w.sum(-1, keepdim=True) + 1e-20) * c.routed_scaling_factor
        return idx, w

    def _experts_rows(self, L, xs, counts):
        """``xs`` rows grouped by local expert (``counts[e]`` rows each, shared expert last) -> expert MLP of every row."""
        F = self.c.moe_intermediate_size
        if self.grouped:
            offs = counts.cumsum(0).to(torch.int32)
            h = torch._grouped_mm(xs, L["w13"], offs=offs)
            h = Fn.silu(h[:, :F]) * h[:, F:]
            return torch._grouped_mm(h, L["w2"], offs=offs)
        out = torch.empty(xs.shape[0], self.c.hidden_size, dtype=xs.dtype, device=xs.device)
        start = 0
        for e, n in enumerate(counts.tolist()):
            if n:
                h = xs[start:start + n] @ L["w13"][e]
                out[start:start + n] = (Fn.silu(h[:, :F]) * h[:, F:]) @ L["w2"][e]
            start += n
        return out

    def _moe(self, L, x):
        c, T, E, el = self.c, x.shape[0], self.c.n_routed_experts, self.e_local
        idx, w = self._route(L, x)
        k = idx.shape[1]
        if self.layout == "a2a" and self.world > 1:
            return self._moe_a2a(L, x, idx, w)
        # local experts (all of them on one GPU) plus the shared expert as one more group that every token visits.  With replicated
        # tokens rank r serves the shared expert for the tokens t = r (mod world), and the entries of other ranks' experts go to a
        # last group whose weights are zero: the shapes stay static, so the step needs no host round trip.
        G = L["w13"].shape[0]
        lo = self.rank * el if self.ep > 1 else 0
        tok = torch.arange(T, device=x.device)
        if self.ep > 1:
            local = (idx >= lo) & (idx < lo + el)
            flat_e = torch.where(local, idx - lo, torch.full_like(idx, el + 1)).flatten()
            sh_e = torch.where((tok % self.ep) == self.rank, el, el + 1)
        else:
            flat_e, sh_e = idx.flatten(), torch.full((T,), el, device=x.device, dtype=idx.dtype)
        all_e = torch.cat([flat_e, sh_e])
        all_t = torch.cat([tok.repeat_interleave(k), tok])
        all_w = torch.cat([w.flatten(), torch.ones(T, device=x.device)])
        order = torch.argsort(all_e, stable=True)
        counts = torch.bincount(all_e, minlength=G)
        src = all_t[order]
        y = self._experts_rows(L, x[src], counts)
        out = torch.zeros(T, c.hidden_size, dtype=torch.float32, device=x.device).index_add_(0, src, y.float() * all_w[order][:, None])
        return self._reduce(out.to(x.dtype))

    def _moe_a2a(self, L, x, idx, w):
        """Tokens at home, experts elsewhere: the usual library recipe — counts by all-to-all, sizes through the host, rows by
        ``all_to_all_single``, grouped GEMMs, rows back, weighted sum.  The shared expert runs at home as one more group."""
        dist, c, T, el, W = self.dist, self.c, x.shape[0], self.e_local, self.world
        k = idx.shape[1]
        flat = idx.flatten()
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=c.n_routed_experts)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)                           # [W, el]: rows source s sends for my expert j
        send_split = counts.view(W, el).sum(1).tolist()
        recv_split = recv_counts.view(W, el).sum(1).tolist()
        xs = x[order // k]
        recv = torch.empty(sum(recv_split), x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, xs, recv_split, send_split)
        # received rows are ordered (source, expert); the grouped GEMM wants (expert, source)
        rc = recv_counts.view(W, el)
        seg_e = torch.arange(el, device=x.device).repeat(W)
        row_e = seg_e.repeat_interleave(rc.flatten(), output_size=recv.shape[0])
        perm = torch.argsort(row_e, stable=True)
        rows = torch.cat([recv[perm], x])                                     # + the shared expert's rows (all local tokens)
        cnt = torch.cat([rc.sum(0), torch.tensor([T], device=x.device)])
        y = self._experts_rows(L, rows, cnt)
        y_r, y_sh = y[:recv.shape[0]], y[recv.shape[0]:]
        back = torch.empty_like(recv)
        back[perm] = y_r
        ret = torch.empty_like(xs)
        dist.all_to_all_single(ret, back, send_split, recv_split)
        out = torch.zeros(T, c.hidden_size, dtype=torch.float32, device=x.device)
        out.index_add_(0, order // k, ret.float() * w.flatten()[order][:, None])
        return (out + y_sh.float()).to(x.dtype)

    def _ffn(self, L, x):
        if "w_gu" in L:
            h = x @ L["w_gu"].T
            Fd = h.shape[1] // 2
            return self._reduce((Fn.silu(h[:, :Fd]) * h[:, Fd:]) @ L["w_down"].T)
        return self._moe(L, x)

    def _block(self, L, li, h, pos, b_idx):
        eps = self.c.rms_norm_eps
        h = h + self._attention(L, li, _rms(h, L["ln_attn"], eps), pos, b_idx)
        return h + self._ffn(L, _rms(h, L["ln_ffn"], eps))

    def _argmax(self, x):
        logits = (x @ self.head.T).float()
        v, i = logits.max(-1)
        if self.tp > 1:
            i = i + self.rank * self.head.shape[0]
            vs = [torch.empty_like(v) for _ in range(self.world)]
            is_ = [torch.empty_like(i) for _ in range(self.world)]
            self.dist.all_gather(vs, v)
            self.dist.all_gather(is_, i)
            vs, is_ = torch.stack(vs), torch.stack(is_)
            best = vs.argmax(0)
            i = is_.gather(0, best[None])[0]
        return i.to(torch.int32)

    def _verify(self, ids, pos, b_idx):
        h = self.embed[ids.long()]
        for li in range(self.c.num_hidden_layers):
            h = self._block(self.layers[li], li, h, pos, b_idx)
        return self._argmax(_rms(h, self.norm, self.c.rms_norm_eps)), h

    def _draft(self, h_prev, next_ids, pos, b_idx):
        li = self.c.num_hidden_layers
        L, eps = self.layers[li], self.c.rms_norm_eps
        x = torch.cat([_rms(h_prev, L["h_norm"], eps), _rms(self.embed[next_ids.long()], L["e_norm"], eps)], -1)
        h = self._block(L, li, x @ L["proj"].T, pos, b_idx)
        return self._argmax(_rms(h, L["out_norm"], eps)), h

    # ---------------------------------------------------------------- one decode step (same algorithm as runtime.spec_decode)
    def set_context(self, kv_len, pending, drafts):
        self.kv_before.copy_(torch.as_tensor(kv_len, dtype=torch.int32).to(self.dev))
        self.fed[:, 0].copy_(torch.as_tensor(pending, dtype=torch.int32).to(self.dev))
        if self.k:
            self.fed[:, 1:].copy_(torch.as_tensor(drafts, dtype=torch.int32).to(self.dev))

    @torch.no_grad()
    def step(self):
        B, k, R = self.B, self.k, self.R
        pos = (self.kv_before[:, None] + self.j[None, :]).reshape(-1)
        b_idx = torch.arange(B, device=self.dev).repeat_interleave(R)
        tok, h = self._verify(self.fed.reshape(-1), pos, b_idx)
        if k == 0:
            self.n_emitted.fill_(1)
            self.kv_before.add_(1)
            self.fed[:, 0].copy_(tok)
            return
        pred = tok.view(B, R)
        match = (pred[:, :k] == self.fed[:, 1:]).to(torch.int32)
        acc = torch.cumprod(match, dim=1).sum(dim=1).to(torch.int32)
        new_pending = torch.gather(pred, 1, acc[:, None].long())[:, 0]
        self.n_emitted.copy_(acc + 1)
        nxt = torch.cat([self.fed[:, 1:], self.fed[:, :1]], 1)
        nxt = torch.where(self.j[None, :] == acc[:, None], new_pending[:, None], nxt)
        d_tok, d_h = self._draft(h, nxt.reshape(-1), pos, b_idx)
        row = torch.arange(B, device=self.dev) * R + acc.long()
        drafts = [d_tok[row]]
        h_last = d_h[row]
        self.kv_before.add_(acc + 1)
        b1 = torch.arange(B, device=self.dev)
        for d in range(1, k):
            t2, h_last = self._draft(h_last, drafts[-1], self.kv_before + (d - 1), b1)
            drafts.append(t2)
        self.fed[:, 0].copy_(new_pending)
        self.fed[:, 1:].copy_(torch.stack(drafts, 1))


def run_library_arm(cfg, rank: int, world: int, layout: str, batch_local: int, ctx: int, spec_k: int, steps: int, warmup: int, device,
                    limit_s: float = 240.0) -> dict:
    """Build the library decoder, run ``warmup`` + ``steps`` decode steps (device-timed over the ``steps``, barrier and synchronise on
    both sides, maximum over ranks) and the same end-to-end loop as the product arm (fed tokens from pinned memory in, results
    out, every step).  Returns the figures; raises if the arm cannot run."""
    import time

    import numpy as np
    import torch.distributed as dist
    dev = torch.device(device)
    max_len = (ctx + (warmup + 2 * steps + 4) * (1 + spec_k) + 16 + 31) // 32 * 32
    dec = LibraryK3Decoder(cfg, rank, world, layout, batch_local, spec_k, max_len, dev)
    rng = np.random.default_rng(0)
    dec.set_context(np.full(batch_local, ctx), rng.integers(0, cfg.vocab_size, batch_local),
                    rng.integers(0, cfg.vocab_size, (batch_local, max(spec_k, 1)))[:, :spec_k])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    t_start = time.time()
    for _ in range(warmup):
        dec.step()
    barrier()
    emitted = torch.zeros((), dtype=torch.int64, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        dec.step()
        emitted += dec.n_emitted.sum()
        if time.time() - t_start > limit_s:
            raise TimeoutError("library arm exceeded its time limit")
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if layout == "a2a":
            dist.all_reduce(emitted)
    ms = float(ms.item())
    # end to end: H2D of the fed tokens, the step, D2H of the results
    R = 1 + spec_k
    fed_pin = torch.empty(batch_local, R, dtype=torch.int32).pin_memory()
    out_pin = (torch.empty(batch_local, R, dtype=torch.int32).pin_memory(), torch.empty(batch_local, dtype=torch.int32).pin_memory())
    fed_pin.copy_(dec.fed.cpu())
    barrier()
    t0 = time.perf_counter()
    e2e_tok = 0
    for _ in range(steps):
        dec.fed.copy_(fed_pin, non_blocking=True)
        dec.step()
        out_pin[0].copy_(dec.fed, non_blocking=True)
        out_pin[1].copy_(dec.n_emitted, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        e2e_tok += int(out_pin[1].sum())
        fed_pin.copy_(out_pin[0])
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    tt = torch.tensor([e2e_tok], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        if layout == "a2a":
            dist.all_reduce(tt)
    res = {"ms_per_step": ms / steps, "tokens_per_s": int(emitted.item()) / (ms / 1e3), "e2e_tokens_per_s": int(tt.item()) / float(e2e_s.item()),
           "steps": steps, "warmup": warmup, "expert_slabs_resident": dec.slabs, "expert_dtype": "bf16",
           "expert_bytes_per_layer": dec.expert_bytes_per_layer, "grouped_mm": dec.grouped, "launch": "eager",
           "collectives": {"single": "none", "replicated": "nccl all_reduce / all_gather", "a2a": "nccl all_to_all_single"}[layout]}
    del dec
    torch.cuda.empty_cache()
    return res

"""Attention over a sequence whose rows are sharded across ranks (rank ``r`` holds the contiguous chunk ``r`` of ``world`` equal
chunks), in the two classical forms.  The reference has no sequence parallelism (it scales length on one device by banding and
query blocking); these are the multi-GPU counterparts for the long training and prefill sequences.

* ``ulysses_attention``: two all-to-alls turn the sequence sharding into a HEAD sharding and back — every rank attends the whole
  sequence for ``Hq / world`` query heads with a plain local attention kernel.  Differentiable (an all-to-all with equal splits is
  its own adjoint), so it serves the LoRA trainer for sequences beyond one GPU's memory.  Needs ``Hq % world == 0``; key / value
  heads that do not divide are gathered whole (they are few) and the rank picks the heads its query heads use.
* ``ring_attention``: K / V chunks travel around the ring while every rank keeps its query chunk; each step attends one chunk
  (earlier chunks fully visible, the own chunk causally, later chunks skipped) and the partial results are merged by their
  log-sum-exp.  No head-count constraint, peak memory of one remote chunk.  ``ring_attention`` is the forward (prefill);
  ``ring_attention_autograd`` adds the backward pass, in which the chunks go around once more together with their gradients.

The collectives are ``torch.distributed`` (NCCL over NVLink on GPUs, gloo on CPU ranks): whole chunks are brought into local
memory and read there by local kernels — no kernel touches a peer's memory."""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    """``x [world, ...]``: slice ``j`` goes to rank ``j``; the result's slice ``i`` came from rank ``i``."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)                       # contiguous like x: slices along dim 0 are the messages
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def _local_attention(q, k, v, scale, causal, window):
    """``q [S, Hq, D]``, ``k / v [S, Hkv, D]`` -> ``[S, Hq, D]``: PyTorch's fused attention (differentiable)."""
    S, Hq, D = q.shape
    g = Hq // k.shape[1]
    qt, kt, vt = q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None]
    if g > 1:
        kt, vt = kt.repeat_interleave(g, 1), vt.repeat_interleave(g, 1)
    mask = None
    if window and window < S:
        pos = torch.arange(S, device=q.device)
        mask = (pos[None, :] <= pos[:, None]) & ((pos[:, None] - pos[None, :]) < window)
    o = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, attn_mask=mask, is_causal=causal and mask is None, scale=scale)
    return o[0].transpose(0, 1)


def ulysses_attention(q, k, v, rank: int, world: int, group=None, scale: float | None = None, causal: bool = True, window: int = 0,
                      attn_fn=None):
    """``q [S / world, Hq, D]``, ``k / v [S / world, Hkv, D]`` (this rank's rows) -> ``[S / world, Hq, D]``.
    ``attn_fn(q, k, v, scale, causal, window)`` is the local attention over the WHOLE sequence for this rank's heads."""
    Sl, Hq, D = q.shape
    Hkv = k.shape[1]
    if Hq % world:
        raise ValueError(f"{Hq} query heads cannot be split over {world} ranks")
    scale = D ** -0.5 if scale is None else scale
    attn_fn = attn_fn or _local_attention
    hq = Hq // world

    def to_heads(x, h):              # [Sl, world * h, D] -> [S, h, D]
        x = x.reshape(Sl, world, h, -1).permute(1, 0, 2, 3)
        return _AllToAll.apply(x, group).reshape(world * Sl, h, -1)

    qh = to_heads(q, hq)
    if Hkv % world == 0:
        kh, vh = to_heads(k, Hkv // world), to_heads(v, Hkv // world)
    else:
        # few key / value heads: every rank gets all of them for the whole sequence and keeps the ones its query heads read
        g = Hq // Hkv
        first, last = (rank * hq) // g, ((rank + 1) * hq - 1) // g
        if (rank * hq) % g and first != last:
            raise ValueError("this rank's query heads straddle key / value heads unevenly")
        kh = _gather_rows(k, world, group)[:, first:last + 1]
        vh = _gather_rows(v, world, group)[:, first:last + 1]
        if (last - first + 1) * g != hq:
            # the rank's query heads cover only part of one key / value group: expand so that the local kernel sees matching heads
            reps = hq // (last - first + 1)
            kh, vh = kh.repeat_interleave(reps, 1), vh.repeat_interleave(reps, 1)
            kh, vh = kh[:, :hq], vh[:, :hq]
    o = attn_fn(qh, kh, vh, scale, causal, window)                # [S, hq, D]
    o = o.reshape(world, Sl, hq, -1)
    o = _AllToAll.apply(o, group)                                  # slice i: this rank's rows, heads of rank i
    return o.permute(1, 0, 2, 3).reshape(Sl, Hq, -1)


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, world, group):
        ctx.world, ctx.group = world, group
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        n = g.shape[0] // ctx.world
        r = dist.get_rank(ctx.group)
        return g[r * n:(r + 1) * n], None, None


def _gather_rows(x, world, group):
    return _GatherRows.apply(x, world, group)


def _chunk_attention(q, k, v, scale, mode: str):
    """Scores of a query chunk against ONE key chunk in f32: returns ``(o [Sq, Hq, D] normalised, lse [Sq, Hq])``.
    ``mode``: ``full`` (every key visible) or ``causal`` (same positions in both chunks)."""
    Sq, Hq, D = q.shape
    g = Hq // k.shape[1]
    kf = k.float().repeat_interleave(g, 1) if g > 1 else k.float()
    vf = v.float().repeat_interleave(g, 1) if g > 1 else v.float()
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    if mode == "causal":
        n = s.shape[-1]
        s = s.masked_fill(torch.ones(Sq, n, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, -1)                                    # [Hq, Sq]
    o = torch.einsum("hqk,khd->qhd", torch.exp(s - lse[..., None]), vf)
    return o, lse.transpose(0, 1)


def ring_attention(q, k, v, rank: int, world: int, group=None, scale: float | None = None, chunk_fn=None):
    """Causal attention of this rank's query chunk over the whole sequence: ``world`` steps, one key / value chunk per step, the
    chunks passed on around the ring between steps.  ``q [S / world, Hq, D]``, ``k / v [S / world, Hkv, D]`` -> ``[S / world, Hq, D]``.
    ``chunk_fn(q, k, v, scale, mode)`` returns ``(o, lse)`` of one chunk pair (default: an f32 PyTorch formula)."""
    D = q.shape[-1]
    scale = D ** -0.5 if scale is None else scale
    chunk_fn = chunk_fn or _chunk_attention
    acc = None                       # running (o, lse)
    kc, vc = k.contiguous(), v.contiguous()
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for step in range(world):
        src = (rank - step) % world                               # whose chunk we hold now
        recv = None
        if step + 1 < world:
            # pass the chunk on while this step computes
            kr, vr = torch.empty_like(kc), torch.empty_like(vc)
            ops_ = [dist.P2POp(dist.isend, kc, _global(nxt, group), group), dist.P2POp(dist.isend, vc, _global(nxt, group), group),
                    dist.P2POp(dist.irecv, kr, _global(prv, group), group), dist.P2POp(dist.irecv, vr, _global(prv, group), group)]
            recv = (dist.batch_isend_irecv(ops_), kr, vr)
        if src <= rank:                                           # later chunks are masked entirely
            o, lse = chunk_fn(q, kc, vc, scale, "causal" if src == rank else "full")
            if acc is None:
                acc = (o.float(), lse.float())
            else:
                o0, l0 = acc
                l = torch.logaddexp(l0, lse.float())
                acc = (o0 * torch.exp(l0 - l)[..., None] + o.float() * torch.exp(lse.float() - l)[..., None], l)
        if recv is not None:
            for w in recv[0]:
                w.wait()
            kc, vc = recv[1], recv[2]
    return acc[0].to(q.dtype)


def _ring_pass(tensors, rank, world, group):
    """Send ``tensors`` to the next rank of the ring and receive the previous rank's (blocking)."""
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    recv = [torch.empty_like(t) for t in tensors]
    ops_ = [dist.P2POp(dist.isend, t.contiguous(), _global(nxt, group), group) for t in tensors]
    ops_ += [dist.P2POp(dist.irecv, r, _global(prv, group), group) for r in recv]
    for w in dist.batch_isend_irecv(ops_):
        w.wait()
    return recv


class _RingAttention(torch.autograd.Function):
    """The ring form with its backward pass: K / V chunks go around once more, now together with the gradients they have
    collected so far, so that after ``world`` steps every chunk is home again with its complete dK / dV; dQ stays local.  The
    per-chunk arithmetic is the f32 formula of the forward (P = exp(S - lse), dS = P (dP - rowsum(dO O)))."""

    @staticmethod
    def forward(ctx, q, k, v, rank, world, group, scale):
        out32, lse = _ring_forward(q, k, v, rank, world, group, scale)
        ctx.save_for_backward(q, k, v, out32, lse)
        ctx.cfg = (rank, world, group, scale)
        return out32.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, out32, lse = ctx.saved_tensors
        rank, world, group, scale = ctx.cfg
        g = q.shape[1] // k.shape[1]
        qf, dof = q.float(), do.float()
        delta = (dof * out32).sum(-1)                                  # [Sq, Hq]
        dq = torch.zeros_like(qf)
        kc, vc = k.contiguous(), v.contiguous()
        dk, dv = torch.zeros_like(kc, dtype=torch.float32), torch.zeros_like(vc, dtype=torch.float32)
        for step in range(world):
            src = (rank - step) % world
            if src <= rank:
                kf = kc.float().repeat_interleave(g, 1) if g > 1 else kc.float()
                vf = vc.float().repeat_interleave(g, 1) if g > 1 else vc.float()
                s = torch.einsum("qhd,khd->hqk", qf, kf) * scale
                if src == rank:
                    n = s.shape[-1]
                    s = s.masked_fill(torch.ones(qf.shape[0], n, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
                p = torch.exp(s - lse.transpose(0, 1)[..., None])      # [Hq, Sq, Sk]
                dp = torch.einsum("qhd,khd->hqk", dof, vf)
                ds = p * (dp - delta.transpose(0, 1)[..., None]) * scale
                dq += torch.einsum("hqk,khd->qhd", ds, kf)
                dkh = torch.einsum("hqk,qhd->khd", ds, qf)
                dvh = torch.einsum("hqk,qhd->khd", p, dof)
                if g > 1:                                              # the query heads of a group share their key / value head
                    dkh = dkh.view(dkh.shape[0], -1, g, dkh.shape[-1]).sum(2)
                    dvh = dvh.view(dvh.shape[0], -1, g, dvh.shape[-1]).sum(2)
                dk += dkh
                dv += dvh
            # after the last step's pass every chunk (and its gradients) is back on its own rank
            kc, vc, dk, dv = _ring_pass([kc, vc, dk, dv], rank, world, group)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None


def _ring_forward(q, k, v, rank, world, group, scale):
    acc = None
    kc, vc = k.contiguous(), v.contiguous()
    for step in range(world):
        src = (rank - step) % world
        if src <= rank:
            o, lse = _chunk_attention(q, kc, vc, scale, "causal" if src == rank else "full")
            if acc is None:
                acc = (o.float(), lse.float())
            else:
                o0, l0 = acc
                l = torch.logaddexp(l0, lse.float())
                acc = (o0 * torch.exp(l0 - l)[..., None] + o.float() * torch.exp(lse.float() - l)[..., None], l)
        if step + 1 < world:
            kc, vc = _ring_pass([kc, vc], rank, world, group)
    return acc


def ring_attention_autograd(q, k, v, rank: int, world: int, group=None, scale: float | None = None):
    """``ring_attention`` with gradients (f32 PyTorch arithmetic per chunk pair): for sequences that are too long for the
    all-to-all form's whole-sequence attention on one rank."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return _RingAttention.apply(q, k, v, rank, world, group, scale)


def _global(r: int, group) -> int:
    return dist.get_global_rank(group, r) if group is not None else r

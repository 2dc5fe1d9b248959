"""Attention over a sequence whose rows are sharded across ranks (rank ``r`` holds the contiguous chunk ``r`` of ``world`` equal
chunks), in the two classical forms.  The reference has no sequence parallelism (it scales length on one device by banding and
query blocking); these are the multi-GPU counterparts for the long training and prefill sequences.

* ``ulysses_attention``: two all-to-alls turn the sequence sharding into a HEAD sharding and back — every rank attends the whole
  sequence for ``Hq / world`` query heads with a plain local attention kernel.  Differentiable (an all-to-all with equal splits is
  its own adjoint), so it serves the LoRA trainer for sequences beyond one GPU's memory.  Needs ``Hq % world == 0``; key / value
  heads that do not divide are gathered whole (they are few) and the rank picks the heads its query heads use.
* ``ring_attention``: K / V chunks travel around the ring while every rank keeps its query chunk; each step attends one chunk
  (earlier chunks fully visible, the own chunk causally, later chunks skipped) and the partial results are merged by their
  log-sum-exp.  No head-count constraint, peak memory of one remote chunk.  Forward only (prefill).

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


def _global(r: int, group) -> int:
    return dist.get_global_rank(group, r) if group is not None else r

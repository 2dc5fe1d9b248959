"""Plain PyTorch implementations of every op.

They serve three purposes: the CPU execution path (the tiny-decoder configuration runs on CPU in f32), the fp32
oracle each CUDA kernel is tested against, and the "NCCL + library" baseline arm of the benchmarks.
All of them accept any device and dtype; reductions are done in float32."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x, weight=None, eps: float = 1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def add_rmsnorm(x, residual, weight, eps: float = 1e-6):
    """``residual += x`` (one rounding to the storage dtype, src/models/inkling/resid.rs:180-270) then norm."""
    r = (residual.float() + x.float()).to(residual.dtype)
    return rmsnorm(r, weight, eps), r


def rope_inv_freq(head_dim: int, theta: float, partial_rotary_factor: float = 1.0, device="cpu"):
    """``theta^(-2j/D)`` computed in f64 then cast to f32; a partial rotation zeroes the tail of inv_freq
    (src/models/gemma/rope.rs:68-99)."""
    j = torch.arange(head_dim // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * j / head_dim)
    rot = int(head_dim // 2 * partial_rotary_factor)
    inv[rot:] = 0.0
    return inv.to(torch.float32).to(device)


def rope(x, positions, inv_freq):
    """Split-half (NeoX) rotation of ``x[T, heads, D]`` (src/models/gemma/rope.rs:190-217)."""
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).to(x.dtype)


def kv_append(k, v, kcache, vcache, slot_mapping):
    """Write rows ``k[T, Hkv, D]`` / ``v`` into page slots ``slot_mapping[T]``."""
    kc = kcache.view(-1, *kcache.shape[2:])
    kc[slot_mapping] = k.to(kc.dtype)
    if v is not None and vcache is not None and vcache is not kcache:
        vc = vcache.view(-1, *vcache.shape[2:])
        vc[slot_mapping] = v.to(vc.dtype)


def gather_pages(cache, page_row, kv_len: int):
    """Dense ``[kv_len, ...]`` view of one sequence's pages."""
    ps = cache.shape[1]
    n = (kv_len + ps - 1) // ps
    return cache[page_row[:n].long()].reshape(n * ps, *cache.shape[2:])[:kv_len]


def paged_attention(q, kcache, vcache, meta, scale: float, window: int = 0, softcap: float = 0.0, dv: int | None = None, rel_bias=None):
    """Causal (optionally sliding-window) attention of the flattened batch over the paged cache.
    ``q[T, Hq, D]``; caches ``[pages, page, Hkv, D]``; GQA by index; softmax in f32.  A latent cache
    (``[pages, page, D]``, one shared kv head) passes ``vcache is kcache`` and ``dv`` = value width (the first ``dv`` dims)."""
    T, Hq, D = q.shape
    if kcache.dim() == 3:
        kcache = kcache.unsqueeze(2)
        vcache = vcache.unsqueeze(2)
    if dv is not None:
        vcache = vcache[..., :dv]
    Hkv = kcache.shape[2]
    g = Hq // Hkv
    out = torch.empty(T, Hq, vcache.shape[-1], dtype=q.dtype, device=q.device)
    qs = meta.q_start.tolist()
    kl = meta.kv_len.tolist()
    for s in range(meta.num_seqs):
        a, b = qs[s], qs[s + 1]
        if a == b:
            continue
        K = gather_pages(kcache, meta.page_table[s], kl[s]).float()      # [L, Hkv, D]
        V = gather_pages(vcache, meta.page_table[s], kl[s]).float()
        Q = q[a:b].float()                                               # [n, Hq, D]
        qpos = meta.positions[a:b].long()
        kpos = torch.arange(kl[s], device=q.device)
        Kh = K.repeat_interleave(g, dim=1)
        Vh = V.repeat_interleave(g, dim=1)
        sc = torch.einsum("nhd,lhd->hnl", Q, Kh) * scale
        if rel_bias is not None:                 # rel_bias[row, head, dist] for keys dist positions back, zero outside the extent
            dist = qpos[:, None] - kpos[None, :]
            ext = rel_bias.shape[-1]
            inside = (dist >= 0) & (dist < ext)
            rb = rel_bias[a:b].float().permute(1, 0, 2)                       # [Hq, n, ext]
            sc = sc + torch.gather(rb, 2, dist.clamp(0, ext - 1)[None].expand(Hq, -1, -1)) * inside[None]
        if softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        mask = kpos[None, :] <= qpos[:, None]
        if window > 0:
            mask &= (qpos[:, None] - kpos[None, :]) < window
        sc = sc.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(sc, dim=-1)
        out[a:b] = torch.einsum("hnl,lhd->nhd", p, Vh).to(q.dtype)
    return out


def linear(x, w, bias=None):
    return F.linear(x, w, bias)


def gelu_tanh(x):
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def geglu(gate, up):
    return (F.gelu(gate.float(), approximate="tanh") * up.float()).to(gate.dtype)


def swiglu(gate, up):
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def situ(gate, up, beta: float = 4.0, linear_beta: float = 25.0):
    """``beta*tanh(g/beta)*sigmoid(g) * lb*tanh(u/lb)`` (src/models/k3/situ.rs:54-145)."""
    g, u = gate.float(), up.float()
    return (beta * torch.tanh(g / beta) * torch.sigmoid(g) * (linear_beta * torch.tanh(u / linear_beta))).to(gate.dtype)


def softcap(x, cap: float):
    return (cap * torch.tanh(x.float() / cap)).to(x.dtype) if cap and cap > 0 else x


def embed(ids, table, scale: float = 1.0):
    e = table[ids.long()]
    return e if scale == 1.0 else (e.float() * scale).to(e.dtype)


def argmax_first(logits):
    """Greedy pick, first maximum wins (src/models/gemma/gemma4/lm.rs:22-32)."""
    m = logits.max(dim=-1, keepdim=True).values
    idx = torch.arange(logits.shape[-1], device=logits.device).expand_as(logits)
    return torch.where(logits == m, idx, logits.shape[-1]).min(dim=-1).values


# --------------------------------------------------------------------------- MoE
def router_softmax_topk(logits, k: int, renorm: bool = True):
    """Softmax router: probabilities over all experts, top-k (ties -> lower index), renormalised."""
    p = torch.softmax(logits.float(), dim=-1)
    w, idx = topk_first(p, k)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx.int(), w


def topk_first(scores, k: int):
    """top-k where equal scores resolve to the lower index, returned in selection order."""
    s = scores.clone()
    vals, idxs = [], []
    for _ in range(k):
        i = argmax_first(s)
        vals.append(s.gather(-1, i[:, None]))
        idxs.append(i[:, None])
        s.scatter_(-1, i[:, None], float("-inf"))
    return torch.cat(vals, -1), torch.cat(idxs, -1)


def router_sigmoid_topk(logits, bias, k: int, n_group: int = 1, topk_group: int = 1, scale: float = 1.0,
                        renorm: bool = True):
    """Sigmoid router with selection bias (``noaux_tc``, src/models/k3/router.rs:9-15): pick top-k of
    ``sigmoid(l)+bias`` — optionally restricted to the ``topk_group`` best of ``n_group`` expert groups, a group's
    score being the sum of its two best biased scores — and weight with the UNBIASED scores renormalised by
    ``sum + 1e-20`` times ``scale``."""
    s = torch.sigmoid(logits.float())
    sel = s + (bias.float() if bias is not None else 0.0)
    T, E = sel.shape
    if n_group > 1:
        gs = sel.view(T, n_group, E // n_group)
        top2, _ = topk_first(gs.reshape(T * n_group, -1), 2)
        gscore = top2.sum(-1).view(T, n_group)
        _, gi = topk_first(gscore, topk_group)
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=sel.device).scatter_(1, gi, True)
        sel = sel.masked_fill(~gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
    _, idx = topk_first(sel, k)
    w = s.gather(-1, idx)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx.int(), w * scale


def moe_experts_dense(x, idx, w, w13, w2, act="swiglu"):
    """Reference expert MLP: ``sum_j w[t,j] * w2[e] (act(w13[e] x))`` with ``w13[e] = [gate; up]`` stacked
    (halved layout).  Weights are dense float tensors ``w13[E, 2F, H]``, ``w2[E, H, F]``."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    Fdim = w2.shape[-1]
    actf = {"swiglu": swiglu, "geglu": geglu, "situ": situ}[act]
    for e in idx.unique().tolist():
        t, j = (idx == e).nonzero(as_tuple=True)
        h = x[t].float() @ w13[e].float().T
        h = actf(h[:, :Fdim], h[:, Fdim:])
        y = h @ w2[e].float().T
        out.index_add_(0, t, y * w[t, j][:, None].float())
    return out.to(x.dtype)


# --------------------------------------------------------------------------- NVFP4 (torch twins of nn/fp4.py)
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def quantize_nvfp4(x):
    """Activation quantiser, bit-exact twin of :func:`mary_b200.nn.fp4.quantize_act_nvfp4`.
    Returns ``(codes uint8[rows, k/2], scales uint8[rows, k/16])`` with E4M3 scale bytes."""
    rows, k = x.shape
    blk = x.float().reshape(rows, k // 16, 16)
    amax = blk.abs().amax(-1)
    sf = torch.clamp(amax / 6.0, max=448.0)
    sb = sf.to(torch.float8_e4m3fn)
    s = sb.float()
    y = blk / torch.where(s > 0, s, torch.ones_like(s))[..., None]
    mag = y.abs()
    code = torch.zeros_like(mag, dtype=torch.uint8)
    for t in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (mag >= t).to(torch.uint8)
    code = torch.where(torch.signbit(y), code | 8, code)
    code = torch.where((s == 0)[..., None], torch.zeros_like(code), code).reshape(rows, k)
    return (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous(), sb.view(torch.uint8).contiguous()


def dequantize_nvfp4(codes, scales, scale2: float = 1.0):
    rows = codes.shape[0]
    c = torch.stack([codes & 0xF, codes >> 4], dim=-1).reshape(rows, -1).long()
    tab = torch.cat([_E2M1, -_E2M1]).to(codes.device)
    v = tab[c]
    s = scales.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=-1)
    return v * s * scale2


def short_conv(x, w, history=None):
    """``y = x + depthwise_causal_conv(x)`` with kernel ``w[D, k]`` (tap k-1 = current); ``history`` holds the
    previous ``k-1`` pre-conv rows (zeros at sequence start).  Returns ``(y, new_history)``
    (src/models/inkling/block.rs:48-127)."""
    T, D = x.shape
    k = w.shape[1]
    h = history if history is not None else torch.zeros(k - 1, D, dtype=x.dtype, device=x.device)
    xp = torch.cat([h, x], 0).float()
    y = x.float().clone()
    for j in range(k):
        y += xp[j:j + T] * w[:, j].float()[None, :]
    return y.to(x.dtype), xp[-(k - 1):].to(x.dtype)

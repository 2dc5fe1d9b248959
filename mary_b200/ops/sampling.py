"""Token sampling: greedy, temperature, top-k, top-p (nucleus) and Gumbel-max, seeded.

Reference: host arg-max (src/models/gemma/gemma4/lm.rs:22-32), the speech models' sampler with temperature / top-k / top-p
(src/models/personaplex/sampling.rs:81-140) and device Gumbel-max over top-k (src/models/qwen3tts/predictor_gpu.rs).  Greedy and
tempered-Gumbel run in ``ops.cuda.argmax``; temperature / top-k / top-p sampling runs in ONE launch per batch of rows
(``ops.cuda.sample_top_k_top_p``: radix select by count and by probability mass, no sort, no read-back).  ``sample_reference`` is
the same rule on the host, written the way the reference writes it (stable descending sort, truncations, draw), and the two agree
token for token because the uniform of a row is a pure function of ``(seed, step, row)`` on both sides."""
from __future__ import annotations

import torch

from . import reference as ref


def filter_top_k_top_p(logits, top_k: int = 0, top_p: float = 1.0):
    lg = logits.float().clone()
    if top_k and top_k < lg.shape[-1]:
        kth = torch.topk(lg, top_k, dim=-1).values[..., -1:]
        lg = lg.masked_fill(lg < kth, float("-inf"))
    if top_p < 1.0:
        srt, idx = torch.sort(lg, dim=-1, descending=True)
        p = torch.softmax(srt, -1)
        drop = (p.cumsum(-1) - p) >= top_p                    # keep the smallest prefix whose mass reaches top_p
        srt = srt.masked_fill(drop, float("-inf"))
        lg = torch.full_like(lg, float("-inf")).scatter(-1, idx, srt)
    return lg


_M64 = (1 << 64) - 1


def _splitmix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def draw_uniform(seed: int, step: int, row: int) -> float:
    """The uniform in [0, 1) that row ``row`` draws at ``(seed, step)``: 53 bits of a splitmix64 chain, the same on the device."""
    r = _splitmix((seed & _M64) ^ _splitmix((step & _M64) ^ _splitmix(row)))
    return (r >> 11) / 9007199254740992.0


def sample_reference(row, temperature: float, top_k: int = 0, top_p: float = 1.0, u: float = 0.0) -> tuple[int, list[int]]:
    """``(token, kept indices)`` of one logit row by the reference's rule (src/models/personaplex/sampling.rs:81-140): non-finite
    logits count as -inf; stable descending order; top-k cut; softmax of ``logit / T`` over the survivors in f64; smallest prefix
    whose mass reaches ``top_p``; then the draw with the uniform ``u`` over the kept set IN INDEX ORDER (any fixed order samples the
    same distribution; index order needs no sort on the device)."""
    x = row.detach().double().cpu()
    x = torch.where(torch.isfinite(x), x, torch.full_like(x, float("-inf")))
    if not torch.isfinite(x).any():
        return int(ref.argmax_first(row.detach().float().cpu()[None])[0]), []
    order = torch.sort(x, descending=True, stable=True).indices
    if 0 < top_k < order.numel():
        order = order[:top_k]
    sc = x[order] / temperature
    e = torch.exp(sc - sc.max())
    if top_p < 1.0:
        cum = torch.cumsum(e / e.sum(), 0)
        keep = int((cum >= top_p).nonzero()[0]) + 1 if bool((cum >= top_p).any()) else order.numel()
        order, e = order[:keep], e[:keep]
    idx, perm = torch.sort(order)
    m = e[perm]
    cum = torch.cumsum(m, 0)
    target = u * float(cum[-1])
    pos = int((cum > target).nonzero()[0]) if bool((cum > target).any()) else idx.numel() - 1
    return int(idx[pos]), idx.tolist()


def sample(logits, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0, step: int = 0):
    """Per-row token ids.  ``temperature == 0`` is greedy (first maximum wins); otherwise temperature / top-k / top-p sampling,
    seeded: the same ``(seed, step)`` gives the same tokens, on the host and on the device."""
    if temperature <= 0:
        if logits.is_cuda:
            from . import cuda as K
            return K.argmax(logits.float().contiguous())[0]
        return ref.argmax_first(logits)
    if logits.is_cuda:
        from . import cuda as K
        lg = logits if logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(-1) == 1 else logits.float().contiguous()
        return K.sample_top_k_top_p(lg, temperature, top_k, top_p, seed, step).long()
    return torch.tensor([sample_reference(logits[r], temperature, top_k, top_p, draw_uniform(seed, step, r))[0] for r in range(logits.shape[0])])

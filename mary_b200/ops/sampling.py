"""Token sampling: greedy, temperature, top-k, top-p (nucleus) and Gumbel-max, seeded.

Reference: host arg-max (src/models/gemma/gemma4/lm.rs:22-32), the speech models' sampler with temperature / top-k / top-p
(src/models/personaplex/sampling.rs) and device Gumbel-max over top-k (src/models/qwen3tts/predictor_gpu.rs).  The greedy
and tempered-Gumbel paths run in one hand-written kernel on the GPU (``ops.cuda.argmax``); top-k / top-p filter the logits
first with tensor ops and then sample the same way."""
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


def sample(logits, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0, step: int = 0):
    """Per-row token ids.  ``temperature == 0`` is greedy (first maximum wins)."""
    if temperature <= 0:
        if logits.is_cuda:
            from . import cuda as K
            return K.argmax(logits.float().contiguous())[0]
        return ref.argmax_first(logits)
    lg = filter_top_k_top_p(logits, top_k, top_p)
    if logits.is_cuda:
        from . import cuda as K
        return K.argmax(lg.contiguous(), temperature=temperature, margin=1e30, seed=seed, step=step)[0]
    g = torch.Generator().manual_seed(seed * 1000003 + step)
    u = torch.rand(lg.shape, generator=g).clamp_min(1e-20)
    return (lg / temperature - torch.log(-torch.log(u))).argmax(-1)

"""Mixture-of-experts execution: NVFP4 expert weights, the device routing plan, and the expert MLP.

GPU path (all hand-written kernels, no host round trip between router and experts):
``router_topk -> moe_plan -> gather + quantise -> grouped NVFP4 GEMM (w13, GLU epilogue) -> quantise ->
grouped NVFP4 GEMM (w2) -> weighted un-permute``.  The CPU path restates the same arithmetic with the reference
quantiser and de-quantised weights (the oracle), following src/bin/inkling_forward.rs:2355-2434."""
from __future__ import annotations

import torch

from . import reference as ref


class NVFP4Experts:
    """Packed expert weights: ``w13`` = [gate; up] rows (2F x K) and ``w2`` (H x F) per expert.

    ``*_q``  uint8 ``[E * rows, K/2]`` E2M1 codes (low nibble = lower index)
    ``*_sf`` uint8 ``[E * rows / 128, K/64, 512]`` UE4M3 block scales in the tensor-core block layout
    ``*_s2`` f32 ``[E]`` per-expert second-level scales"""

    def __init__(self, E, H, F, w13_q, w13_sf, w13_s2, w2_q, w2_sf, w2_s2, act="swiglu"):
        self.E, self.H, self.F, self.act = E, H, F, act
        self.w13_q, self.w13_sf, self.w13_s2 = w13_q, w13_sf, w13_s2
        self.w2_q, self.w2_sf, self.w2_s2 = w2_q, w2_sf, w2_s2

    @property
    def device(self):
        return self.w13_q.device

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w13_q, self.w13_sf, self.w13_s2, self.w2_q, self.w2_sf, self.w2_s2))

    @staticmethod
    def quantize_matrix(w):
        """``w[rows, K]`` float -> ``(codes[rows, K/2], sf_blocks[rows/128, K/64, 512], scale2)``; rows % 128 == 0."""
        rows, K = w.shape
        amax = w.abs().max().float()
        scale2 = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
        ws = (w.float() / scale2).to(torch.bfloat16)
        if w.is_cuda:
            from . import cuda_moe
            codes, sf, _ = cuda_moe.quantize_rows(ws, nt=128)
        else:
            codes, sc = ref.quantize_nvfp4(ws)
            sf = swizzle_scales(sc)
        return codes, sf, scale2

    @staticmethod
    def from_dense(w13, w2, act="swiglu"):
        """``w13[E, 2F, H]`` and ``w2[E, H, F]`` float tensors -> packed experts (per-expert scale2)."""
        E, F2, H = w13.shape
        F = F2 // 2
        parts13 = [NVFP4Experts.quantize_matrix(w13[e]) for e in range(E)]
        parts2 = [NVFP4Experts.quantize_matrix(w2[e]) for e in range(E)]
        cat = lambda ps, i: torch.cat([p[i] for p in ps], 0)  # noqa: E731
        return NVFP4Experts(E, H, F, cat(parts13, 0), cat(parts13, 1), torch.stack([p[2] for p in parts13]).float(),
                            cat(parts2, 0), cat(parts2, 1), torch.stack([p[2] for p in parts2]).float(), act)

    @staticmethod
    def random(E, H, F, device, std=0.02, seed=0, act="swiglu", chunk=16):
        """Random-init experts quantised from ``normal(0, std)`` without ever holding them all in bf16."""
        g = torch.Generator(device=device).manual_seed(seed)
        outs = []
        for rows, K in ((2 * F, H), (H, F)):
            q, sf, s2 = [], [], []
            for e0 in range(0, E, chunk):
                n = min(chunk, E - e0)
                w = torch.empty(n, rows, K, device=device, dtype=torch.bfloat16).normal_(0.0, std, generator=g)
                for i in range(n):
                    c, s, g2 = NVFP4Experts.quantize_matrix(w[i])
                    q.append(c); sf.append(s); s2.append(g2)
            outs += [torch.cat(q, 0), torch.cat(sf, 0), torch.stack(s2).float()]
        return NVFP4Experts(E, H, F, *outs, act=act)

    def dense(self, which: str, e: int):
        """De-quantised f32 matrix of expert ``e`` (oracle use)."""
        q, sf, s2, rows, K = ((self.w13_q, self.w13_sf, self.w13_s2, 2 * self.F, self.H) if which == "w13"
                              else (self.w2_q, self.w2_sf, self.w2_s2, self.H, self.F))
        codes = q[e * rows:(e + 1) * rows].cpu()
        sc = unswizzle_scales(sf[e * rows // 128:(e + 1) * rows // 128].cpu(), rows, K // 16)
        return ref.dequantize_nvfp4(codes, sc, float(s2[e]))


def swizzle_scales(sc):
    """Row-major ``[rows, nsf]`` E4M3 bytes -> ``[rows/128, nsf/4, 512]`` blocks (rows, nsf padded with zeros)."""
    rows, nsf = sc.shape
    R, Kb = (rows + 127) // 128, (nsf + 3) // 4
    p = torch.zeros(R * 128, Kb * 4, dtype=torch.uint8, device=sc.device)
    p[:rows, :nsf] = sc
    return p.view(R, 4, 32, Kb, 4).permute(0, 3, 2, 1, 4).contiguous().view(R, Kb, 512)


def unswizzle_scales(blocks, rows, nsf):
    R, Kb, _ = blocks.shape
    return blocks.view(R, Kb, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(R * 128, Kb * 4)[:rows, :nsf]


def experts_reference(x, idx, w, ex: NVFP4Experts, shared=None):
    """Oracle of the NVFP4 expert MLP: activations are quantised (reference quantiser) before each GEMM, weights are
    the de-quantised packed values, sums in f32, outputs rounded to bf16 where the GPU path stores bf16."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32)
    xq = ref.dequantize_nvfp4(*ref.quantize_nvfp4(x.cpu().to(torch.bfloat16)))
    actf = {"swiglu": ref.swiglu, "geglu": ref.geglu, "situ": ref.situ}[ex.act]
    idx_c, w_c = idx.cpu(), w.cpu().float()
    for e in idx_c.unique().tolist():
        if e < 0:
            continue
        t, j = (idx_c == e).nonzero(as_tuple=True)
        h = xq[t] @ ex.dense("w13", e).T
        h = actf(h[:, :ex.F], h[:, ex.F:]).to(torch.bfloat16)
        hq = ref.dequantize_nvfp4(*ref.quantize_nvfp4(h))
        y = (hq @ ex.dense("w2", e).T).to(torch.bfloat16).float()
        out.index_put_((t,), y * w_c[t, j][:, None], accumulate=True)
    if shared is not None:
        out += shared.cpu().float()
    return out.to(torch.bfloat16)


def experts_forward(x, idx, w, ex: NVFP4Experts, shared=None, nt: int | None = None):
    """``sum_j w[t, j] * expert_{idx[t, j]}(x[t])`` (+ ``shared``).  ``idx`` int32 ``[T, k]`` (negative = not local)."""
    if x.is_cuda:
        from . import cuda_moe
        return cuda_moe.experts_forward(x, idx, w, ex, shared, nt)
    return experts_reference(x, idx, w, ex, shared)

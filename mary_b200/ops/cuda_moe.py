"""ctypes wrappers for the MoE kernels (plan, quantise, grouped NVFP4 GEMM, un-permute)."""
from __future__ import annotations

import torch

from ..utils.canary import empty as _empty
from .cuda import _p, _stream, check, declare, lib

declare("mary_moe_plan", "piiiiippppps")
declare("mary_moe_max_rows", "iii")
declare("mary_quant_nvfp4_rows", "plpiiiipppps")
declare("mary_moe_unpermute", "plppiiipps")
declare("mary_gemm_nvfp4_grouped", "pppppppp" + "liiilii" + "s")


def quantize_rows(x, nt: int = 128, src_of=None, identity: bool = True, rows: int | None = None, rowmajor: bool = False,
                  n_rows=None, zero_sf: bool = True):
    """NVFP4-quantise rows of ``x`` (bf16).  Returns ``(codes[rows, K/2], sf_blocks[ceil(rows/nt), K/64, 512], rowmajor|None)``.
    With ``src_of`` (int32 per destination row) rows are gathered (``identity=False``) or merely validated.  ``zero_sf=False``
    leaves the scale bytes of skipped (padding) rows unwritten: their products stay inside those rows, which nothing reads."""
    K = x.shape[1]
    rows = rows if rows is not None else x.shape[0]
    tiles = (rows + nt - 1) // nt
    xq = _empty(rows, K // 2, dtype=torch.uint8, device=x.device)
    sf = (torch.zeros if zero_sf else torch.empty)(tiles, K // 64, 512, dtype=torch.uint8, device=x.device)
    rm = _empty(rows, K // 16, dtype=torch.uint8, device=x.device) if rowmajor else None
    check(lib().mary_quant_nvfp4_rows(_p(x), x.stride(0), _p(src_of), int(identity), rows, K, nt, _p(xq), _p(sf), _p(rm),
                                      _p(n_rows), _stream()), "quant_nvfp4_rows")
    return xq, sf, rm


declare("mary_quant_nvfp4_entries", "plpiiiiipps")


def quantize_entries(x, plan, k: int, identity: bool):
    """The quantiser of the expert pipeline driven by the routed entries (``plan.row_of``): one CTA per entry instead of one per
    padded row.  Padding rows keep whatever bytes the buffers held; their products stay inside those rows, which nothing reads."""
    K = x.shape[1]
    rows, nt = plan.max_rows, plan.nt
    xq = _empty(rows, K // 2, dtype=torch.uint8, device=x.device)
    sf = _empty(rows // nt, K // 64, 512, dtype=torch.uint8, device=x.device)
    check(lib().mary_quant_nvfp4_entries(_p(x), x.stride(0), _p(plan.row_of), plan.row_of.numel(), k, int(identity), K, nt, _p(xq), _p(sf),
                                         _stream()), "quant_nvfp4_rows")
    return xq, sf


def quantize_nvfp4(x):
    """Row-major twin of the reference quantiser: ``(codes, scales[rows, K/16])``."""
    xq, _, rm = quantize_rows(x.contiguous(), nt=128, rowmajor=True)
    return xq, rm


class Plan:
    __slots__ = ("row_of", "src_of", "tiles", "meta", "counts", "max_rows", "nt")


def moe_plan(idx, E: int, nt: int) -> Plan:
    T, k = idx.shape
    p = Plan()
    p.nt = nt
    p.max_rows = lib().mary_moe_max_rows(T * k, E, nt)
    dev = idx.device
    p.row_of = _empty(T * k, dtype=torch.int32, device=dev)
    p.src_of = _empty(p.max_rows, dtype=torch.int32, device=dev)
    p.tiles = _empty(p.max_rows // nt, 4, dtype=torch.int32, device=dev)
    p.meta = _empty(2, dtype=torch.int32, device=dev)
    p.counts = _empty(E, dtype=torch.int32, device=dev)
    check(lib().mary_moe_plan(_p(idx.contiguous()), T * k, k, E, nt, p.max_rows, _p(p.row_of), _p(p.src_of), _p(p.tiles),
                              _p(p.meta), _p(p.counts), _stream()), "moe_plan")
    return p


def grouped_gemm(wq, sfw, scale2, xq, sfx, plan: Plan, n_out: int, K: int, E: int, glu: str | None):
    out = _empty(plan.max_rows, n_out, dtype=torch.bfloat16, device=xq.device)
    g = 0 if glu is None else {"geglu": 1, "swiglu": 2, "situ": 3}[glu]
    check(lib().mary_gemm_nvfp4_grouped(_p(wq), _p(sfw), _p(scale2), _p(xq), _p(sfx), _p(plan.tiles), _p(plan.meta), _p(out),
                                        out.stride(0), E, n_out, K, plan.max_rows, plan.nt, g, _stream()), "gemm_nvfp4_grouped")
    return out


declare("mary_gemm_nvfp4_grouped_glu_q", "ppppppppp" + "iiiliis")
# with 32-token tiles the w13 GEMM of ``experts_forward`` leaves its GLU result quantised (same bytes as GEMM -> bf16 ->
# quantiser, one launch less).  With 128-token tiles the GEMM has one accumulator buffer and the longer epilogue stalls its main
# loop (measured on a 4096-token prefill: +65 ms in the GEMMs against 10 ms saved), so the quantiser stays a launch of its own.
def _glu_quant_default() -> bool:
    from ..utils import flags
    return bool(flags.get("MARY_MOE_GLU_QUANT"))


FUSED_GLU_QUANT = _glu_quant_default()


def grouped_gemm_glu_q(wq, sfw, scale2, xq, sfx, plan: Plan, n_out: int, K: int, E: int, glu: str):
    """The GLU GEMM with the quantising epilogue: ``(codes [rows, n_out / 2], scale tiles)`` ready for the next NVFP4 GEMM."""
    rows, nt = plan.max_rows, plan.nt
    hq = _empty(rows, n_out // 2, dtype=torch.uint8, device=xq.device)
    sfh = _empty(rows // nt, n_out // 64, 512, dtype=torch.uint8, device=xq.device)
    g = {"geglu": 1, "swiglu": 2, "situ": 3}[glu]
    check(lib().mary_gemm_nvfp4_grouped_glu_q(_p(wq), _p(sfw), _p(scale2), _p(xq), _p(sfx), _p(plan.tiles), _p(plan.meta), _p(hq), _p(sfh),
                                              E, n_out, K, rows, nt, g, _stream()), "gemm_nvfp4_grouped")
    return hq, sfh


def unpermute(y, plan: Plan, w, T: int, k: int, add=None):
    H = y.shape[1]
    out = _empty(T, H, dtype=torch.bfloat16, device=y.device)
    check(lib().mary_moe_unpermute(_p(y), y.stride(0), _p(plan.row_of), _p(w.float().contiguous()), T, k, H, _p(add), _p(out),
                                   _stream()), "moe_unpermute")
    return out


def experts_forward(x, idx, w, ex, shared=None, nt: int | None = None):
    T, k = idx.shape
    if nt is None:
        nt = 32 if T * k <= 32 * ex.E else 128
    plan = moe_plan(idx, ex.E, nt)
    xq, sfx = quantize_entries(x, plan, k, identity=False)
    if FUSED_GLU_QUANT and nt == 32:
        hq, sfh = grouped_gemm_glu_q(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, ex.F, ex.H, ex.E, ex.act)
    else:
        h = grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, ex.F, ex.H, ex.E, ex.act)
        hq, sfh = quantize_entries(h, plan, k, identity=True)
    y = grouped_gemm(ex.w2_q, ex.w2_sf, ex.w2_s2, hq, sfh, plan, ex.H, ex.F, ex.E, None)
    return unpermute(y, plan, w, T, k, shared)


declare("mary_gemm_bf16_grouped", "ppp" + "iii" + "lll" + "i" + "l" + "pp" + "iii" + "s")


def grouped_gemm_bf16(xg, w, plan: Plan, n_out: int, glu: str | None, swap: bool = True):
    """``out[r] = act_glu(xg[r] @ w[expert of r's tile]^T)`` over the plan's padded rows; ``w [E, n_out or 2 n_out, K]`` unquantised.
    ``swap=False`` (plans with 128-row tiles, no GLU): tokens as the 128-row tensor-core operand, for prefill-sized batches."""
    E, _, K = w.shape
    out = _empty(plan.max_rows, n_out, dtype=torch.bfloat16, device=xg.device)
    g = 0 if glu is None else {"geglu": 1, "swiglu": 2, "situ": 3}[glu]
    check(lib().mary_gemm_bf16_grouped(_p(xg), _p(w), _p(out), plan.max_rows, n_out, K, xg.stride(0), w.stride(1), out.stride(0), E,
                                       w.stride(0), _p(plan.tiles), _p(plan.meta), plan.nt, g, int(swap), _stream()), "gemm_bf16_grouped")
    return out


def experts_forward_bf16(x, idx, w, gate_up, down, act: str = "geglu", e0: int = 0, nt: int | None = None):
    """Routed experts with unquantised weights (``gate_up [E, 2F, H]``, ``down [E, H, F]``; the experts held here are
    ``e0 .. e0 + E``): device routing plan, row gather, two grouped tensor-core GEMMs (the first with the GLU epilogue), weighted
    un-permute.  No host synchronisation: the launch sequence does not depend on the routing."""
    T, k = idx.shape
    E = gate_up.shape[0]
    if nt is None:
        nt = 32 if T * k <= 32 * E else (64 if T * k <= 64 * E else 128)
    local = idx - e0 if e0 else idx
    plan = moe_plan(torch.where((local >= 0) & (local < E), local, torch.full_like(local, -1)).int(), E, nt)
    xg = x.index_select(0, plan.src_of.clamp_min(0).long())          # padding rows repeat token 0; nothing reads their results
    if nt == 128 and T * k >= 256 * E:
        # prefill-sized: token-major tiles (tokens are the 128-row operand), GLU as its own kernel
        from .cuda import glu
        h = glu(grouped_gemm_bf16(xg, gate_up, plan, gate_up.shape[1], None, swap=False), act)
        y = grouped_gemm_bf16(h, down, plan, down.shape[1], None, swap=False)
    else:
        h = grouped_gemm_bf16(xg, gate_up, plan, gate_up.shape[1] // 2, act)
        y = grouped_gemm_bf16(h, down, plan, down.shape[1], None)
    return unpermute(y, plan, w, T, k)

"""CUDA (sm_100a) implementations of the ops: thin ctypes wrappers over ``_kernels.so``.

Tensors are passed as raw device pointers plus the current CUDA stream, so the launches are captured by CUDA
graphs like any other stream work.  Every wrapper checks the launcher's return code; activations are bf16."""
from __future__ import annotations

import ctypes
import math

import torch

from .. import _native
from ..utils.canary import empty as _empty

_SIG = {
    # name: argument codes — p pointer, i int32, l int64, f float, s stream
    "mary_gemm_bf16": "pppiiilllpfiiiis",
    "mary_rmsnorm": "pippiillfs",
    "mary_add_rmsnorm": "pipppiifs",
    "mary_norm_add_norm": "pippppiiffs",
    "mary_glu": "ppiiis",
    "mary_embed": "pppiifis",
    "mary_qk_norm_rope_append": "piiippipppppp" + "fils",
    "mary_short_conv": "ppppiiis",
    "mary_paged_attention": "ppppppppp" + "iii" + "llll" + "iiiiiii" + "ff" + "ps",
    "mary_paged_attention_scratch_floats": "iiii",
    "mary_paged_attention_max_rows": "i",
    "mary_last_status": "",
    "mary_sm_count": "",
}
_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int32, "l": ctypes.c_int64, "f": ctypes.c_float, "s": ctypes.c_void_p}
_RET64 = {"mary_paged_attention_scratch_floats"}
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = _native.kernels()
        for name, sig in _SIG.items():
            try:
                fn = getattr(l, name)
            except AttributeError:
                continue
            fn.argtypes = [_CT[c] for c in sig]
            fn.restype = ctypes.c_int64 if name in _RET64 else ctypes.c_int32
        _lib = l
    return _lib


def declare(name: str, sig: str, ret64: bool = False):
    """Register one more launcher signature (used by the other op modules)."""
    _SIG[name] = sig
    if ret64:
        _RET64.add(name)
    global _lib
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = [_CT[c] for c in sig]
        fn.restype = ctypes.c_int64 if ret64 else ctypes.c_int32


_STATUS = {1: "a TMA pipeline wait timed out", 2: "an accumulator wait timed out", 3: "a peer flag wait timed out",
           4: "bad argument", 5: "CUDA launch error", 6: "bounds check failed"}


class KernelError(RuntimeError):
    pass


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_NVTX = None


def _nvtx() -> bool:
    global _NVTX
    if _NVTX is None:
        from ..utils import flags
        _NVTX = bool(flags.get("MARY_NVTX"))
    return _NVTX


LAUNCHES = 0      # launcher calls made through this module (each starts at least one kernel)
TRACE = None      # an active mary_b200.utils.trace.Tracer, or None


def check(rc: int, what: str):
    global LAUNCHES
    LAUNCHES += 1
    if TRACE is not None:
        TRACE.mark(what)
    if _nvtx():
        torch.cuda.nvtx.mark(what)
    if rc != 0:
        raise KernelError(f"{what}: {_STATUS.get(rc, rc)}")


def last_status() -> int:
    """Read and clear the device status word (synchronises)."""
    return lib().mary_last_status()


def _bf16(t):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"expected a bf16 tensor, got {t.dtype}")
    return t


# --------------------------------------------------------------------------- GEMM
def gemm(x, w, out=None, bias=None, alpha: float = 1.0, glu: str | None = None, epi: str = "bf16", split_k: int = 1,
         swap: int = -1):
    """``out[M, N] = alpha * x[M, K] @ w[N, K]^T``.  ``glu``: ``w = [gate; up]`` (2N rows) and the epilogue writes
    ``act(gate) * up``.  ``epi``: ``"bf16"`` store, ``"f32"`` store, ``"red"`` accumulate into a zeroed f32 ``out``."""
    _bf16(x), _bf16(w)
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()                       # the epilogue reads an f32 bias vector
    M, K = x.shape
    n_w = w.shape[0]
    N = n_w // 2 if glu else n_w
    assert w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1
    e = {"bf16": 0, "red": 1, "f32": 2}[epi]
    if out is None:
        out = (torch.zeros if e == 1 else torch.empty)(M, N, dtype=torch.bfloat16 if e == 0 else torch.float32, device=x.device)
    g = 0 if glu is None else {"geglu": 1, "swiglu": 2, "situ": 3}[glu]
    rc = lib().mary_gemm_bf16(_p(x), _p(w), _p(out), M, N, K, x.stride(0), w.stride(0), out.stride(0), _p(bias), alpha, g, e,
                              split_k, swap, _stream())
    check(rc, "gemm_bf16")
    return out


def _auto_split_k(M: int, N: int, K: int) -> int:
    """GEMMs with few output tiles cannot fill 148 SMs; split K until they do (mirrors the launcher's tile choice)."""
    if M <= 256:
        bn = 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
        tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
    else:
        tr = (M + 127) // 128
        bn = 256
        while bn > 64 and tr * ((N + bn - 1) // bn) < 148:
            bn //= 2
        tiles = tr * ((N + bn - 1) // bn)
    # measured on a B200 at 48 and 384 rows: from ~90 tiles on, and for short K (a tile's main loop is then a few stages long and
    # the partial-tile traffic of a split outweighs the idle SMs), the unsplit kernel is the faster one
    if tiles >= 90 or K <= 2048:
        return 1
    return max(1, min(K // 512, (148 + tiles - 1) // tiles))


declare("mary_gemm_bf16_splitk", "pppiiilllpfiiiplpis")
_SK_WS: dict = {}
SK_WS_FLOATS = 4 << 20          # 16 MiB of accumulator tiles
SK_COUNTERS = 8192


def _sk_workspace(dev):
    """Scratch of the split-K GEMM (f32 accumulator tiles + per-tile arrival counters, zero between calls), one per device;
    calls on one stream share it.  Created on first use — before any stream capture, since warm-up steps run eagerly first."""
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _SK_WS:
        _SK_WS[key] = (torch.zeros(SK_WS_FLOATS, dtype=torch.float32, device=dev), torch.zeros(SK_COUNTERS, dtype=torch.int32, device=dev))
    return _SK_WS[key]


def gemm_splitk(x, w, split_k: int, out=None, f32: bool = False, bias=None, swap: int = -1):
    """``x @ w^T`` with K cut into ``split_k`` slices reduced inside the kernel (every slice adds into an f32 accumulator tile in
    scratch; the slice that finishes last converts and stores it and leaves the scratch zero): no zero-fill, no cast pass.  ``split_k=0`` is stream-K: the K-blocks of all tiles are dealt out in
    equal contiguous runs, one per SM, so every SM streams the same share of the weights whatever the tile count.  Falls back
    to the atomic path when the shape outgrows the scratch."""
    _bf16(x), _bf16(w)
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    M, K = x.shape
    N = w.shape[0]
    ws, cnt = _sk_workspace(x.device)
    if out is None:
        out = _empty(M, N, dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    rc = lib().mary_gemm_bf16_splitk(_p(x), _p(w), _p(out), M, N, K, x.stride(0), w.stride(0), out.stride(0), _p(bias), 1.0, int(f32),
                                     split_k, swap, _p(ws), ws.numel(), _p(cnt), cnt.numel(), _stream())
    if rc == 4:                                             # scratch too small for this shape
        red = gemm(x, w, epi="red", split_k=split_k or _auto_split_k(M, N, K))
        if bias is not None:
            red += bias
        out.copy_(red)
        return out
    check(rc, "gemm_bf16_splitk")
    return out


class _StaticWeights:
    """While active, the GEMM launchers of this thread are told that their ``w`` operand holds constant model weights, so that under
    programmatic dependent launch (``MARY_PDL=1``) a kernel may request its first weight tiles before its predecessor has finished."""
    depth = 0

    def __enter__(self):
        from ..utils import flags
        if flags.get("MARY_PDL"):
            _StaticWeights.depth += 1
            if _StaticWeights.depth == 1:
                lib().mary_gemm_hint_static_weights(1)

    def __exit__(self, *exc):
        from ..utils import flags
        if flags.get("MARY_PDL"):
            _StaticWeights.depth -= 1
            if _StaticWeights.depth == 0:
                lib().mary_gemm_hint_static_weights(0)


static_weights = _StaticWeights()
declare("mary_gemm_hint_static_weights", "i")


def linear(x, w, bias=None):
    with static_weights:
        return _linear(x, w, bias)


MATVEC_MAX_BYTES = 8 << 20       # one-token products up to this weight size take the SIMT matrix-vector stage (4 us against 6 us per launch)


def _linear(x, w, bias=None):
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M, K = x2.shape
    if (M == 1 and bias is None and K % 8 == 0 and K <= 8192 and w.shape[0] * K * 2 <= MATVEC_MAX_BYTES and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        return step_matvec(x2, w).reshape(*shp[:-1], w.shape[0])
    sk = _auto_split_k(M, w.shape[0], K)
    out = gemm_splitk(x2, w, 0, bias=bias) if sk > 1 else gemm(x2, w, bias=bias)
    return out.reshape(*shp[:-1], w.shape[0])


def linear_f32(x, w, split_k: int | None = None):
    """Row-parallel style GEMM whose f32 result feeds a norm kernel directly (no bf16 rounding in between)."""
    M, K = x.shape
    sk = split_k or _auto_split_k(M, w.shape[0], K)
    with static_weights:
        return gemm_splitk(x, w, 0 if split_k is None else sk, f32=True) if sk > 1 else gemm(x, w, epi="f32")


def linear_glu(x, w_gu, act: str = "geglu"):
    M = x.shape[0]
    with static_weights:
        if M <= 128:
            return gemm(x, w_gu, glu=act)
        return glu(gemm(x, w_gu), act)


# --------------------------------------------------------------------------- norms and friends
def rmsnorm(x, weight=None, eps=1e-6):
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    y = _empty(x2.shape, dtype=torch.bfloat16, device=x.device)
    check(lib().mary_rmsnorm(_p(x2), int(x2.dtype == torch.float32), _p(weight), _p(y), x2.shape[0], x2.shape[1],
                             x2.stride(0), y.stride(0), eps, _stream()), "rmsnorm")
    return y.reshape(shp)


def add_rmsnorm(x, residual, weight, eps=1e-6):
    y = torch.empty_like(residual)
    check(lib().mary_add_rmsnorm(_p(x), int(x.dtype == torch.float32), _p(residual), _p(weight), _p(y), residual.shape[0],
                                 residual.shape[1], eps, _stream()), "add_rmsnorm")
    return y, residual


def norm_add_norm(a, w_post, h, w_next, eps=1e-6, scalar=1.0):
    xo = torch.empty_like(h) if w_next is not None else None
    check(lib().mary_norm_add_norm(_p(a), int(a.dtype == torch.float32), _p(w_post), _p(h), _p(w_next), _p(xo), h.shape[0],
                                   h.shape[1], eps, scalar, _stream()), "norm_add_norm")
    return xo, h


def glu(gate_up, act="geglu"):
    T, F2 = gate_up.shape
    out = _empty(T, F2 // 2, dtype=torch.bfloat16, device=gate_up.device)
    check(lib().mary_glu(_p(gate_up.contiguous()), _p(out), T, F2 // 2, {"geglu": 0, "swiglu": 1, "situ": 2}[act], _stream()), "glu")
    return out


def embed(ids, table, scale=1.0):
    ids = ids.to(torch.int32)
    out = _empty(ids.shape[0], table.shape[1], dtype=torch.bfloat16, device=table.device)
    check(lib().mary_embed(_p(ids), _p(table), _p(out), ids.shape[0], table.shape[1], scale, table.shape[0], _stream()), "embed")
    return out


def qk_norm_rope_append(qkv, n_q, n_kv, head_dim, q_norm, k_norm, v_norm, inv_freq, meta, kcache, vcache, eps):
    T = qkv.shape[0]
    q = _empty(T, n_q, head_dim, dtype=torch.bfloat16, device=qkv.device)
    check(lib().mary_qk_norm_rope_append(_p(qkv.contiguous()), n_q, n_kv, head_dim, _p(q_norm), _p(k_norm), int(bool(v_norm)),
                                         _p(inv_freq), _p(meta.positions), _p(meta.slot_mapping), _p(q), _p(kcache), _p(vcache),
                                         eps, T, kcache.shape[0] * kcache.shape[1] if n_kv else 0, _stream()), "qk_norm_rope_append")
    return q


def short_conv(x, w, history=None):
    T, D = x.shape
    k = w.shape[1]
    hist = history.clone() if history is not None else torch.zeros(k - 1, D, dtype=torch.bfloat16, device=x.device)
    y = torch.empty_like(x)
    check(lib().mary_short_conv(_p(x.contiguous()), _p(w.float().contiguous()), _p(hist), _p(y), T, D, k, _stream()), "short_conv")
    return y, hist


# --------------------------------------------------------------------------- attention
def _q_blocks(meta, rq: int):
    key = ("qblk", rq)
    cache = meta.__dict__.setdefault("_cache", {})
    if key not in cache:
        import numpy as np
        seqs, q0 = [], []
        start = 0
        for s, n in enumerate(meta.q_lens_host.tolist()):
            for b in range(0, n, rq):
                seqs.append(s)
                q0.append(start + b)
            start += n
        dev = meta.positions.device
        cache[key] = (torch.tensor(seqs, dtype=torch.int32).to(dev, non_blocking=True),
                      torch.tensor(q0, dtype=torch.int32).to(dev, non_blocking=True), len(seqs))
    return cache[key]


declare("mary_paged_attention_decode", "ppppppppp" + "iii" + "llll" + "iiiiii" + "ff" + "ps")


DECODE_TARGET_CTAS = 2368      # CTAs the decode attention kernel aims for when it picks the number of kv splits (16 per SM)


def _paged_attention_decode(q, kcache, vcache, meta, scale, window, softcap, nsplit):
    """Decode-shaped batches (few rows per kv head, equal K and V widths of 64/128/256): the bandwidth-oriented kernel."""
    T, Hq, D = q.shape
    Hkv = kcache.shape[2]
    G = Hq // Hkv
    cap = 4 if D == 256 else 8
    rq = max(1, min(cap // G, meta.max_q_len))
    blk_seq, blk_q0, NB = _q_blocks(meta, rq)
    if nsplit is None:
        want = max(1, DECODE_TARGET_CTAS // max(1, NB * Hkv))
        span = meta.max_kv_len if window <= 0 else min(meta.max_kv_len, window + rq)
        nsplit = max(1, min(want, 32, span // 64))
    out = _empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    scratch = None
    if nsplit > 1:
        scratch = _empty(lib().mary_paged_attention_scratch_floats(NB, Hkv, nsplit, D), dtype=torch.float32, device=q.device)
    check(lib().mary_paged_attention_decode(_p(q.contiguous()), _p(kcache), _p(vcache), _p(out), _p(meta.page_table), _p(meta.kv_len),
                                            _p(meta.q_start), _p(blk_seq), _p(blk_q0), NB, meta.page_table.shape[1], meta.page_size,
                                            kcache.stride(1), kcache.stride(0), vcache.stride(1), vcache.stride(0), Hq, Hkv, D, rq,
                                            nsplit, window, scale, softcap, _p(scratch), _stream()), "paged_attention_decode")
    return out


declare("mary_paged_attention_decode_q8", "pppppp" + "ppppp" + "iii" + "llll" + "iiiiii" + "ffps")
declare("mary_kv_quant_append", "plppp" + "iiils")


def kv_quant_append(rows, slots, pages) -> None:
    T, Hkv, D = rows.shape
    assert rows.dtype == torch.bfloat16 and rows.stride(2) == 1 and rows.stride(1) == D and slots.dtype == torch.int64
    assert tuple(pages.codes.shape[2:]) == (Hkv, D) and pages.codes.is_contiguous() and pages.sz.is_contiguous()
    check(lib().mary_kv_quant_append(_p(rows), rows.stride(0), _p(slots), _p(pages.codes), _p(pages.sz), T, Hkv, D,
                                     pages.codes.shape[0] * pages.codes.shape[1], _stream()), "kv_quant_append")


def decode_q8_supported(q, kcache, meta) -> bool:
    T, Hq, D = q.shape
    Hkv = kcache.shape[2]
    return (q.dtype == torch.bfloat16 and D == kcache.shape[3] and D in (64, 128, 256) and Hq % Hkv == 0
            and Hq // Hkv <= (4 if D == 256 else 8) and meta.max_q_len <= 8)


def paged_attention_decode_q8(q, kcache, vcache, meta, scale, window=0, softcap=0.0, nsplit=None):
    """The decode kernel over an 8-bit cache (``runtime.kv_cache.Q8Pages``): rows are dequantised in registers."""
    T, Hq, D = q.shape
    Hkv = kcache.shape[2]
    G = Hq // Hkv
    cap = 4 if D == 256 else 8
    rq = max(1, min(cap // G, meta.max_q_len))
    blk_seq, blk_q0, NB = _q_blocks(meta, rq)
    if nsplit is None:
        want = max(1, DECODE_TARGET_CTAS // max(1, NB * Hkv))
        span = meta.max_kv_len if window <= 0 else min(meta.max_kv_len, window + rq)
        nsplit = max(1, min(want, 32, span // 64))
    out = _empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    scratch = None
    if nsplit > 1:
        scratch = _empty(lib().mary_paged_attention_scratch_floats(NB, Hkv, nsplit, D), dtype=torch.float32, device=q.device)
    kc, vc = kcache.codes, vcache.codes
    check(lib().mary_paged_attention_decode_q8(_p(q.contiguous()), _p(kc), _p(vc), _p(kcache.sz), _p(vcache.sz), _p(out), _p(meta.page_table),
                                               _p(meta.kv_len), _p(meta.q_start), _p(blk_seq), _p(blk_q0), NB, meta.page_table.shape[1],
                                               meta.page_size, kc.stride(1), kc.stride(0), vc.stride(1), vc.stride(0), Hq, Hkv, D, rq,
                                               nsplit, window, scale, softcap, _p(scratch), _stream()), "paged_attention_decode_q8")
    return out


declare("mary_gqa_decode_tc", "ppppppppp" + "iiiiiiiiiii" + "ffps")
declare("mary_gqa_tc_supported", "iiii")
declare("mary_gqa_tc_scratch_floats", "iiii", ret64=True)


def gqa_tc_supported(q, kcache, meta) -> bool:
    """Decode-shaped batch of a grouped-query model that the tensor-core decode kernel takes: bf16, equal K / V widths of 128 or 256,
    contiguous caches with 16- or 32-token pages, at most 64 (query token, head of the group) rows per kv head."""
    if kcache.dim() != 4 or q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or not kcache.is_contiguous():
        return False
    T, Hq, D = q.shape
    Hkv = kcache.shape[2]
    if Hq % Hkv or kcache.shape[3] != D or meta.max_q_len > 8:
        return False
    G = Hq // Hkv
    rq = max(1, min(64 // max(G, 1), meta.max_q_len))
    return bool(lib().mary_gqa_tc_supported(D, meta.page_size, G, rq)) and kcache.shape[1] == meta.page_size


def gqa_decode_tc(q, kcache, vcache, meta, scale, window=0, softcap=0.0, nsplit=None):
    """Decode attention of a grouped-query model on the tensor cores: the (token, head-of-group) rows of one kv head are one M = 64
    tile, K and V pages arrive by TMA, split-KV partials are merged by a second kernel."""
    T, Hq, D = q.shape
    Hkv = kcache.shape[2]
    G = Hq // Hkv
    rq = max(1, min(64 // G, meta.max_q_len))
    blk_seq, blk_q0, NB = _q_blocks(meta, rq)
    if nsplit is None:
        want = max(1, (296 if D == 128 else 148) // max(1, NB * Hkv))
        span = meta.max_kv_len if window <= 0 else min(meta.max_kv_len, window + rq)
        nsplit = max(1, min(want, 32, span // (4 * meta.page_size)))
    out = _empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    scratch = None
    if nsplit > 1:
        scratch = _empty(lib().mary_gqa_tc_scratch_floats(NB, Hkv, nsplit, D), dtype=torch.float32, device=q.device)
    assert vcache.is_contiguous() and vcache.shape == kcache.shape
    check(lib().mary_gqa_decode_tc(_p(q.contiguous()), _p(kcache), _p(vcache), _p(out), _p(meta.page_table), _p(meta.kv_len), _p(meta.q_start),
                                   _p(blk_seq), _p(blk_q0), NB, T, kcache.shape[0], meta.page_table.shape[1], meta.page_size, Hq, Hkv, D, rq,
                                   nsplit, window, scale, softcap, _p(scratch), _stream()), "gqa_decode_tc")
    return out


declare("mary_attention_prefill", "ppppppppp" + "iiiiiiii" + "llll" + "ifis")
declare("mary_attention_prefill_supported", "ii")
PREFILL_MIN_ROWS = 48     # mean query tokens per sequence from which the 128-row tensor-core tiles pay off


def attention_prefill(q, kcache, vcache, meta, scale, window=0):
    """Causal / sliding-window attention of whole query blocks on the tensor cores (``csrc/kernels/attention_fa.cu``):
    ``q[T, Hq, DK]``, caches ``[pages, page, Hkv, D]``; 128 query tokens of one head per CTA.  A cache with 64-token pages is
    streamed with one TMA operation per 64-key stage; a cache with smaller pages is first regrouped into 64-token pages (one
    gather, small beside the attention arithmetic) when the host knows the sequence lengths."""
    T, Hq, DK = q.shape
    Hkv, DV = kcache.shape[2], vcache.shape[-1]
    ps = meta.page_size
    assert kcache.shape[1] == ps
    if ps in (16, 32) and meta.kv_lens_host is not None:
        pick, meta = meta.repage(64)
        kcache = kcache[pick].view(-1, 64, Hkv, DK)
        vcache = vcache[pick].view(-1, 64, Hkv, DV)
        ps = 64
    assert ps in (16, 64)
    blk_seq, blk_tok0, NB = _q_blocks(meta, 128)
    out = _empty(T, Hq, DV, dtype=torch.bfloat16, device=q.device)
    check(lib().mary_attention_prefill(_p(q.contiguous()), _p(kcache), _p(vcache), _p(out), _p(meta.page_table), _p(meta.kv_len),
                                       _p(meta.q_start), _p(blk_seq), _p(blk_tok0), NB, T, Hq, Hkv, DK, DV, kcache.shape[0],
                                       meta.page_table.shape[1], kcache.stride(1), kcache.stride(0), vcache.stride(1), vcache.stride(0),
                                       int(window), float(scale), ps, _stream()), "attention_prefill")
    return out


declare("mary_paged_attention_rel", "ppppppppp" + "iii" + "llll" + "iiiiiii" + "ff" + "ppi" + "s")


def _gqa_tc_default() -> bool:
    from ..utils import flags
    return bool(flags.get("MARY_GQA_TC"))


GQA_TC = _gqa_tc_default()          # route decode-shaped grouped-query batches to the tensor-core kernel (MARY_GQA_TC)


def paged_attention(q, kcache, vcache, meta, scale, window=0, softcap=0.0, dv: int | None = None, nsplit: int | None = None,
                    kernel: str = "auto", rel_bias=None):
    """``q[T, Hq, DK]``; caches ``[pages, page, Hkv, D]`` (a latent cache is ``Hkv = 1`` with ``dv`` < DK and
    ``vcache is kcache``).  Returns ``[T, Hq, DV]``.  ``kernel``: ``auto`` picks the tensor-core prefill kernel for long query
    blocks, the bandwidth-oriented kernel for decode-shaped batches and the general split-KV kernel otherwise."""
    T, Hq, DK = q.shape
    Hkv = kcache.shape[2] if kcache.dim() == 4 else 1
    DV = dv or vcache.shape[-1]
    G = Hq // Hkv
    if rel_bias is not None:                     # ``rel_bias [T, Hq, extent]`` f32, added to the scaled score of the key ``dist`` back
        kernel = "general"
        assert rel_bias.dtype == torch.float32 and rel_bias.shape[:2] == (T, Hq) and rel_bias.is_contiguous()
    if kernel in ("auto", "prefill") and kcache.dim() == 4 and dv is None and softcap == 0.0 and meta.page_size in (16, 32, 64) \
            and lib().mary_attention_prefill_supported(DK, DV) and q.dtype == torch.bfloat16 \
            and (kernel == "prefill" or T >= PREFILL_MIN_ROWS * meta.num_seqs):
        return attention_prefill(q, kcache, vcache, meta, scale, window)
    if kernel in ("auto", "tc") and (kernel == "tc" or GQA_TC) and dv is None and gqa_tc_supported(q, kcache, meta):
        return gqa_decode_tc(q, kcache, vcache, meta, scale, window, softcap, nsplit)
    if kernel == "tc":
        raise ValueError("the tensor-core decode kernel does not take this shape")
    if kernel != "general" and kcache.dim() == 4 and DK == DV and DK in (64, 128, 256) and G <= (4 if DK == 256 else 8) \
            and (meta.max_q_len <= 8 or kernel == "decode"):
        return _paged_attention_decode(q, kcache, vcache, meta, scale, window, softcap, nsplit)
    maxr = lib().mary_paged_attention_max_rows(DV)
    if G > maxr:
        # more query heads per kv head than one CTA can hold: fold the surplus into extra "kv heads" that alias
        # the same cache rows (head stride 0 is expressed by Hkv' = Hkv * fold with DK-strided q only)
        raise NotImplementedError("GQA group larger than the row budget; use the tensor-core MLA kernel")
    rq = max(1, min(maxr // G, meta.max_q_len))
    blk_seq, blk_q0, NB = _q_blocks(meta, rq)
    if nsplit is None:
        want = max(1, 296 // max(1, NB * Hkv))
        span = meta.max_kv_len if window <= 0 else min(meta.max_kv_len, window + rq)
        nsplit = max(1, min(want, 32, span // 128))
    out = _empty(T, Hq, DV, dtype=torch.bfloat16, device=q.device)
    scratch = None
    if nsplit > 1:
        n = lib().mary_paged_attention_scratch_floats(NB, Hkv, nsplit, DV)
        scratch = _empty(n, dtype=torch.float32, device=q.device)
    ktok, kpage = kcache.stride(1), kcache.stride(0)
    vtok, vpage = vcache.stride(1), vcache.stride(0)
    if rel_bias is not None:
        check(lib().mary_paged_attention_rel(_p(q.contiguous()), _p(kcache), _p(vcache), _p(out), _p(meta.page_table), _p(meta.kv_len),
                                             _p(meta.q_start), _p(blk_seq), _p(blk_q0), NB, meta.page_table.shape[1], meta.page_size,
                                             ktok, kpage, vtok, vpage, Hq, Hkv, DK, DV, rq, nsplit, window, scale, softcap,
                                             _p(scratch), _p(rel_bias), rel_bias.shape[2], _stream()), "paged_attention_rel")
        return out
    check(lib().mary_paged_attention(_p(q.contiguous()), _p(kcache), _p(vcache), _p(out), _p(meta.page_table), _p(meta.kv_len),
                                     _p(meta.q_start), _p(blk_seq), _p(blk_q0), NB, meta.page_table.shape[1], meta.page_size,
                                     ktok, kpage, vtok, vpage, Hq, Hkv, DK, DV, rq, nsplit, window, scale, softcap,
                                     _p(scratch), _stream()), "paged_attention")
    return out


# --------------------------------------------------------------------------- selection
declare("mary_argmax", "pliififfllpps")
declare("mary_router_topk", "plpiiiiiifipppps")


def argmax(logits, softcap=0.0, temperature: float = 0.0, margin: float = 20.0, seed: int = 0, step: int = 0):
    """Per-row arg-max (first maximum wins) or, with ``temperature > 0``, a Gumbel-max sample.  Returns ``(ids, value)``."""
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    idx = _empty(rows, dtype=torch.int64, device=logits.device)
    val = _empty(rows, dtype=torch.float32, device=logits.device)
    check(lib().mary_argmax(_p(logits), logits.stride(0), rows, V, softcap, 1 if temperature > 0 else 0, temperature, margin,
                            seed, step, _p(idx), _p(val), _stream()), "argmax")
    return idx, val


declare("mary_sample_top_k_top_p", "pilii" + "fif" + "ll" + "pps")


def sample_top_k_top_p(logits, temperature: float, top_k: int = 0, top_p: float = 1.0, seed: int = 0, step: int = 0, want_prob: bool = False):
    """One token per row of ``logits [rows, V]`` (f32 or bf16) by temperature / top-k / top-p sampling in one launch, no sort and no
    read-back; the draw of row ``r`` depends on ``(seed, step, r)`` only.  Returns int32 ids (and the drawn token's probability)."""
    rows, V = logits.shape
    assert logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(1) == 1 and temperature > 0 and top_p > 0
    idx = _empty(rows, dtype=torch.int32, device=logits.device)
    prob = _empty(rows, dtype=torch.float32, device=logits.device) if want_prob else None
    check(lib().mary_sample_top_k_top_p(_p(logits), int(logits.dtype == torch.float32), logits.stride(0), rows, V, float(temperature), int(top_k),
                                        float(top_p), int(seed) & (2**63 - 1), int(step) & (2**63 - 1), _p(idx), _p(prob), _stream()),
          "sample_top_k_top_p")
    return (idx, prob) if want_prob else idx


def lm_head_argmax(h, table, softcap=0.0, vocab_limit=None):
    logits = gemm(h.contiguous(), table, epi="f32")
    if vocab_limit:
        logits = logits[:, :vocab_limit]
    return argmax(logits, softcap)


def router_topk(logits, k, mode="softmax", bias=None, n_group=1, topk_group=1, scale=1.0, renorm=True, counts=None, flag=None):
    T, E = logits.shape
    lg = logits if logits.dtype == torch.float32 else logits.float()
    idx = _empty(T, k, dtype=torch.int32, device=logits.device)
    w = _empty(T, k, dtype=torch.float32, device=logits.device)
    b = bias.float().contiguous() if bias is not None else None
    check(lib().mary_router_topk(_p(lg), lg.stride(0), _p(b), T, E, k, 0 if mode == "softmax" else 1, n_group, topk_group, scale,
                                 int(renorm), _p(idx), _p(w), _p(counts), _p(flag), _stream()), "router_topk")
    return idx, w


def quantize_nvfp4(x):
    from . import cuda_moe
    return cuda_moe.quantize_nvfp4(x)


# --------------------------------------------------------------------------- MLA
declare("mary_mla_attention", "pppppppp" + "iiii" + "ll" + "ii" + "f" + "pis")
declare("mary_mla_scratch_floats", "ii", ret64=True)
declare("mary_mla_tile_rows", "")


def _row_tiles(meta, hq: int):
    key = ("rowtiles", hq)
    cache = meta.__dict__.setdefault("_cache", {})
    if key not in cache:
        seqs, r0 = [], []
        start = 0
        tr = lib().mary_mla_tile_rows()
        for s, n in enumerate(meta.q_lens_host.tolist()):
            rows = n * hq
            for b in range(0, rows, tr):
                seqs.append(s)
                r0.append(start * hq + b)
            start += n
        dev = meta.positions.device
        cache[key] = (torch.tensor(seqs, dtype=torch.int32).to(dev, non_blocking=True),
                      torch.tensor(r0, dtype=torch.int32).to(dev, non_blocking=True), len(seqs))
    return cache[key]


def mla_attention(q, cache, meta, scale, nsplit: int | None = None):
    """``q[T, Hq, 576]`` bf16, ``cache[pages, page (16 or 32), 576]`` bf16 (finite everywhere) -> ``[T, Hq, 512]``.  With
    32-token pages the kernel fetches a whole 32-key stage with one TMA operation."""
    T, Hq, DK = q.shape
    ps = meta.page_size
    assert DK == 576 and ps in (16, 32) and cache.shape[1] == ps and cache.shape[-1] == 576
    blk_seq, blk_r0, NB = _row_tiles(meta, Hq)
    if nsplit is None:
        nsplit = max(1, min(8, 148 // max(1, NB), meta.max_kv_len // 512))
    out = _empty(T, Hq, 512, dtype=torch.bfloat16, device=q.device)
    scratch = None
    if nsplit > 1:
        scratch = _empty(lib().mary_mla_scratch_floats(NB, nsplit), dtype=torch.float32, device=q.device)
    c = cache.view(cache.shape[0], ps, 576)
    check(lib().mary_mla_attention(_p(q.contiguous()), _p(c), _p(out), _p(meta.page_table), _p(meta.kv_len), _p(meta.q_start),
                                   _p(blk_seq), _p(blk_r0), NB, T * Hq, c.shape[0], meta.page_table.shape[1], c.stride(1),
                                   c.stride(0), Hq, nsplit, scale, _p(scratch), ps, _stream()), "mla_attention")
    return out


declare("mary_mla_prep", "plippppppp" + "fils")
declare("mary_mla_q_rope", "ppppiis")
declare("mary_gemm_bf16_batched", "pppiiilll" + "illl" + "pfiiiis")


def gemm_batched(x, w, out, M, N, K, ldx, ldw, ldo, batch, bsx, bsw, bso):
    """``batch`` independent bf16 GEMMs ``out_b[M, N] = x_b[M, K] @ w_b[N, K]^T`` over strided views (element strides)."""
    check(lib().mary_gemm_bf16_batched(_p(x), _p(w), _p(out), M, N, K, ldx, ldw, ldo, batch, bsx, bsw, bso, None, 1.0, 0, 0, 1, -1,
                                       _stream()), "gemm_bf16_batched")
    return out


declare("mary_mla_q_rope_inplace", "pppiis")
declare("mary_mla_fill_k_rope", "plpils")


def mla_expand_kv(rows, w_uk_t, w_uv, H):
    """Keys and values of the expanded (non-absorbed) prefill straight into their final layout, without concatenation copies:
    ``rows [N, 576]`` latent rows -> ``k [N, H, 192]`` (``W_UK^T c_kv`` per head by a batched GEMM over the heads that shares the
    row operand and writes each head's 128 columns at pitch 192, then the 64 rotated dims every head shares copied behind them) and
    ``v [N, H, 128]`` (one GEMM).  ``w_uk_t [H * 128, 512]``, ``w_uv [H * 128, 512]``."""
    N = rows.shape[0]
    k = _empty(N, H, 192, dtype=torch.bfloat16, device=rows.device)
    with static_weights:
        gemm_batched(rows, w_uk_t, k, N, 128, 512, rows.stride(0), 512, H * 192, H, 0, 128 * 512, 192)
        v = gemm(rows[:, :512], w_uv)
    check(lib().mary_mla_fill_k_rope(_p(rows), rows.stride(0), _p(k), H, N, _stream()), "mla_fill_k_rope")
    return k, v.view(N, H, 128)


def mla_q_rope_inplace(qb, inv_freq, meta, H):
    """Rotate the 64 rope dims of every head of ``qb [T, H * 192]`` in place."""
    check(lib().mary_mla_q_rope_inplace(_p(qb), _p(inv_freq), _p(meta.positions), H, qb.shape[0], _stream()), "mla_q_rope")
    return qb


def mla_prep(qakv, q_lora, w_qa, w_kv, inv_freq, meta, cache, eps):
    T = qakv.shape[0]
    qa = _empty(T, q_lora, dtype=torch.bfloat16, device=qakv.device)
    check(lib().mary_mla_prep(_p(qakv), qakv.stride(0), q_lora, _p(w_qa), _p(w_kv), _p(inv_freq), _p(meta.positions),
                              _p(meta.slot_mapping), _p(qa), _p(cache), eps, T, cache.shape[0] * cache.shape[1], _stream()), "mla_prep")
    return qa


def mla_absorb_q(qb, w_uk, inv_freq, meta, H):
    """``qb[T, H*192]`` -> ``q_full[T, H, 576]``: nope part times ``w_uk[H, 512, 128]`` (absorbed W_UK), rope part rotated."""
    T = qb.shape[0]
    q_full = _empty(T, H, 576, dtype=torch.bfloat16, device=qb.device)
    with static_weights:
        gemm_batched(qb, w_uk, q_full, T, 512, 128, H * 192, 128, H * 576, H, 192, 512 * 128, 576)
    check(lib().mary_mla_q_rope(_p(qb), _p(inv_freq), _p(meta.positions), _p(q_full), H, T, _stream()), "mla_q_rope")
    return q_full


def mla_unabsorb_o(o_lat, w_uv, H):
    """``o_lat[T, H, 512]`` -> ``o[T, H*128]`` with ``w_uv[H, 128, 512]``."""
    T = o_lat.shape[0]
    o = _empty(T, H * 128, dtype=torch.bfloat16, device=o_lat.device)
    with static_weights:
        gemm_batched(o_lat, w_uv, o, T, 128, 512, H * 512, 512, H * 128, H, 512, 128 * 512, 128)
    return o


# ------------------------------------------------------------------------------------------------- one-token decoder layer step
declare("mary_step_matvec", "ppfpliippi" + "s")
declare("mary_step_attention", "pppppppppp" + "iiiilffp" + "s")


def step_matvec(h, w, gain=None, eps: float = 1e-6, res=None, mode: str = "plain"):
    """One-token matrix-vector stage of the fused layer step: ``W x`` (``plain``), ``res + W x`` (``residual``) or
    ``silu(W_gate x) * (W_up x)`` over ``w = [gate; up]`` (``swiglu``), with ``x = rms(h) * gain`` when ``gain`` is given,
    else ``x = h``.  ``h [1, K]`` -> ``[1, N]``."""
    m = {"plain": 0, "residual": 1, "swiglu": 2}[mode]
    K = h.shape[-1]
    N = w.shape[0] // 2 if m == 2 else w.shape[0]
    y = _empty(1, N, dtype=torch.bfloat16, device=h.device)
    check(lib().mary_step_matvec(_p(h), _p(gain), eps, _p(w), w.stride(0), N, K, _p(res), _p(y), m, _stream()), "step_matvec")
    return y


def step_attention(qkv, q_gain, k_gain, inv_freq, meta, kcache, vcache, n_q: int, n_kv: int, head_dim: int, eps: float, scale: float):
    """Head norms, rotation, cache append and attention of ONE new token of ONE sequence (head dim 128): ``qkv [1, (n_q + 2 n_kv) D]``
    -> ``[1, n_q * D]``."""
    out = _empty(1, n_q * head_dim, dtype=torch.bfloat16, device=qkv.device)
    n_slots = kcache.shape[0] * kcache.shape[1]
    check(lib().mary_step_attention(_p(qkv), _p(q_gain), _p(k_gain), _p(inv_freq), _p(meta.positions), _p(meta.slot_mapping), _p(meta.page_table),
                                    _p(meta.kv_len), _p(kcache), _p(vcache), n_q, n_kv, head_dim, meta.page_size, n_slots, eps, scale, _p(out),
                                    _stream()), "step_attention")
    return out


declare("mary_set_pdl", "i")


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the launches that follow (``MARY_PDL`` decides when nobody calls this): a gain for steps
    that are chains of small dense GEMMs, a loss with the expert pipeline in the chain."""
    lib().mary_set_pdl(int(bool(on)))

"""Kernel micro-benchmarks: CUDA-event timing after warm-up with an L2 flush between iterations, reported against
the measured peaks of the machine (``MEASURED_PEAKS.json`` at the repository root when present, else the stated
fallback).  ``python -m mary_b200.ops.bench_kernels [gemm|attn|all]``."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_flush = None


def time_op(fn, iters: int = 10, warmup: int = 3) -> float:
    """Median milliseconds of ``fn()``; a 256 MiB write between iterations evicts L2."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


GEMM_SHAPES = [(8192, 8192, 8192), (4096, 4096, 4096), (2048, 15360 * 2, 3840), (32, 6144, 3840), (32, 3840, 4096),
               (32, 30720, 3840), (32, 3840, 15360), (384, 2112, 7168), (384, 12288, 1536), (384, 7168, 8192), (128, 163840, 7168)]


def bench_gemm(shapes=None):
    from . import cuda as K
    hbm, tf, tag = peaks()
    print(f"{'M':>6} {'N':>6} {'K':>6} {'ours ms':>9} {'torch ms':>9} {'TFLOP/s':>8} {'GB/s':>7}  frac {tag}")
    for M, N, Kd in shapes or GEMM_SHAPES:
        x = torch.randn(M, Kd, device="cuda").bfloat16()
        w = (torch.randn(N, Kd, device="cuda") * 0.02).bfloat16()
        sk = K._auto_split_k(M, N, Kd)
        if sk > 1:
            out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            ours = time_op(lambda: K.gemm_splitk(x, w, 0, out=out))
        else:
            out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            ours = time_op(lambda: K.gemm(x, w, out=out))
        th = time_op(lambda: torch.matmul(x, w.T))
        fl = 2.0 * M * N * Kd / ours / 1e9
        gb = (M * Kd + N * Kd + M * N) * 2 / ours / 1e6
        frac = max(fl / tf, gb / hbm)
        print(f"{M:>6} {N:>6} {Kd:>6} {ours:>9.4f} {th:>9.4f} {fl:>8.1f} {gb:>7.0f}  {frac:.2f} ({"stream-K" if sk > 1 else "whole tiles"})")
    assert K.last_status() == 0


def bench_attn(cases=None):
    from . import cuda as K
    from ..runtime.batch import BatchMeta
    from ..runtime.kv_cache import PagedKVCache
    hbm, tf, tag = peaks()
    for (B, L, Hq, Hkv, D, win) in cases or [(32, 2304, 16, 8, 256, 0), (32, 2304, 16, 8, 256, 1024), (64, 1536, 32, 8, 128, 0)]:
        pages = B * ((L + 15) // 16) + 1
        cache = PagedKVCache(1, pages, 16, Hkv, D, dtype=torch.bfloat16, device="cuda")
        for s in range(B):
            cache.alloc.extend(s, L)
        table, lens = cache.alloc.page_table(list(range(B)))
        meta = BatchMeta.build([1] * B, lens, table, 16, "cuda")
        cache.k[0].normal_()
        cache.v[0].normal_()
        q = torch.randn(B, Hq, D, device="cuda").bfloat16()
        span = L if win == 0 else min(L, win)
        for kernel in ("general", "decode"):
            for ctas in ((592,) if kernel == "general" else (592, 1184, 2368, 4736)):
                K.DECODE_TARGET_CTAS = ctas
                ms = time_op(lambda: K.paged_attention(q, cache.k[0], cache.v[0], meta, D ** -0.5, win, kernel=kernel))
                gb = B * span * Hkv * D * 2 * 2 / ms / 1e6
                print(f"decode attn [{kernel}, target {ctas} CTAs] B={B} L={L} Hq={Hq} Hkv={Hkv} D={D} window={win}: {ms:.4f} ms, "
                      f"{gb:.0f} GB/s, {gb / hbm:.2f} {tag}")
        K.DECODE_TARGET_CTAS = 2368
        # the tensor-core kernel, with 16- and 32-token pages and a sweep of the split count
        for page in (16, 32):
            pages = B * ((L + page - 1) // page) + 1
            c2 = PagedKVCache(1, pages, page, Hkv, D, dtype=torch.bfloat16, device="cuda")
            for s in range(B):
                c2.alloc.extend(s, L)
            t2, l2 = c2.alloc.page_table(list(range(B)))
            m2 = BatchMeta.build([1] * B, l2, t2, page, "cuda")
            c2.k[0].normal_()
            c2.v[0].normal_()
            if not K.gqa_tc_supported(q, c2.k[0], m2):
                continue
            for ns in (1, 2, 4, 8, None):
                ms = time_op(lambda: K.gqa_decode_tc(q, c2.k[0], c2.v[0], m2, D ** -0.5, win, nsplit=ns))
                gb = B * span * Hkv * D * 2 * 2 / ms / 1e6
                print(f"decode attn [tensor-core, page {page}, nsplit {ns}] B={B} L={L} Hq={Hq} Hkv={Hkv} D={D} window={win}: {ms:.4f} ms, "
                      f"{gb:.0f} GB/s, {gb / hbm:.2f} {tag}")


def bench_fa(B: int = 1, L: int = 4096, Hq: int = 16, Hkv: int = 16, DK: int = 192, DV: int = 128, window: int = 0, iters: int = 5):
    """Tensor-core prefill attention: B sequences of L tokens, all of them queries (causal)."""
    from . import cuda as K
    from ..runtime.batch import BatchMeta
    from ..runtime.kv_cache import PagedKVCache
    hbm, tf, tag = peaks()
    pages = B * ((L + 15) // 16) + 1
    alloc = PagedKVCache(1, pages, 16, 1, 8, dtype=torch.bfloat16, device="cuda").alloc
    for s in range(B):
        alloc.extend(s, L)
    table, lens = alloc.page_table(list(range(B)))
    meta = BatchMeta.build([L] * B, lens, table, 16, "cuda")
    kc = torch.randn(pages, 16, Hkv, DK, device="cuda").bfloat16()
    vc = torch.randn(pages, 16, Hkv, DV, device="cuda").bfloat16()
    q = torch.randn(B * L, Hq, DK, device="cuda").bfloat16()
    ms = time_op(lambda: K.paged_attention(q, kc, vc, meta, DK ** -0.5, window, kernel="prefill"), iters=iters)
    span = L / 2 if window == 0 else min(window, L / 2)
    flops = 2.0 * B * L * Hq * span * (DK + DV)
    print(f"prefill attn B={B} L={L} Hq={Hq} Hkv={Hkv} DK={DK} DV={DV} window={window}: {ms:.4f} ms, {flops / ms / 1e9:.1f} TFLOP/s "
          f"({flops / ms / 1e9 / tf:.2f} {tag})")
    assert K.last_status() == 0


def bench_mla(B: int = 32, L: int = 4096, Hq: int = 64, q_len: int = 3, page: int = 16, iters: int = 5):
    """MLA latent attention, decode-shaped: B sequences of L cached tokens, q_len query tokens x Hq heads each."""
    from . import cuda as K
    from ..runtime.batch import BatchMeta
    from ..runtime.kv_cache import PagedKVCache
    hbm, tf, tag = peaks()
    pages = B * ((L + page - 1) // page) + 1
    cache = PagedKVCache(1, pages, page, 1, 1, dtype=torch.bfloat16, device="cuda", latent_dim=576)
    for s in range(B):
        cache.alloc.extend(s, L)
    table, lens = cache.alloc.page_table(list(range(B)))
    meta = BatchMeta.build([q_len] * B, lens, table, page, "cuda")
    cache.k[0].normal_()
    q = (torch.randn(B * q_len, Hq, 576, device="cuda") * 0.3).bfloat16()
    ms = time_op(lambda: K.mla_attention(q, cache.k[0], meta, 576 ** -0.5), iters=iters)
    flops = 2.0 * B * q_len * Hq * L * (576 + 512)
    gb = B * L * 1152 / ms / 1e6
    print(f"mla attn B={B} L={L} Hq={Hq} q_len={q_len} page={page}: {ms:.4f} ms, {flops / ms / 1e9:.1f} TFLOP/s ({flops / ms / 1e9 / tf:.2f} {tag}), "
          f"KV stream {gb:.0f} GB/s ({gb / hbm:.2f} {tag})")
    assert K.last_status() == 0


def bench_moe(E: int = 48, H: int = 7168, F: int = 2048, T: int = 384, k: int = 8, iters: int = 5):
    """Decode-shaped expert MLP: every expert is visited, so the step streams all expert weights once (HBM-bound)."""
    from . import cuda as K, cuda_moe
    from .moe import NVFP4Experts
    hbm, tf, tag = peaks()
    ex = NVFP4Experts.random(E, H, F, "cuda", seed=0)
    x = torch.randn(T, H, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, device="cuda")
    plan = cuda_moe.moe_plan(idx, E, 32)
    xq, sfx, _ = cuda_moe.quantize_rows(x, 32, plan.src_of, identity=False, rows=plan.max_rows)
    ms13 = time_op(lambda: cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, F, H, E, "swiglu"), iters=iters)
    h = cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, F, H, E, "swiglu")
    hq, sfh, _ = cuda_moe.quantize_rows(h, 32, plan.src_of, identity=True, rows=plan.max_rows)
    ms2 = time_op(lambda: cuda_moe.grouped_gemm(ex.w2_q, ex.w2_sf, ex.w2_s2, hq, sfh, plan, H, F, E, None), iters=iters)
    b13 = E * 2 * F * H * (0.5 + 1 / 16)
    b2 = E * H * F * (0.5 + 1 / 16)
    for name, ms, b in (("w13+glu", ms13, b13), ("w2", ms2, b2)):
        print(f"nvfp4 grouped {name} E={E} H={H} F={F} T={T} k={k}: {ms:.4f} ms, weights {b / 1e6:.0f} MB, {b / ms / 1e6:.0f} GB/s "
              f"({b / ms / 1e6 / hbm:.2f} {tag})")
    full = time_op(lambda: cuda_moe.experts_forward(x, idx, w, ex), iters=iters)
    print(f"whole expert MLP (plan, quantise, 2 GEMMs, un-permute): {full:.4f} ms, {(b13 + b2) / full / 1e6:.0f} GB/s "
          f"({(b13 + b2) / full / 1e6 / hbm:.2f} {tag})")
    assert K.last_status() == 0


def bench_moeprefill(E: int = 384, H: int = 7168, F: int = 2048, T: int = 4096, k: int = 8, iters: int = 5):
    """Prefill-shaped expert MLP (128-token tiles): a prompt of T tokens puts about T k / E rows on every expert, so below a few
    hundred rows per expert the layer is still bound by streaming the expert weights once."""
    from . import cuda as K, cuda_moe
    from .moe import NVFP4Experts
    hbm, tf, tag = peaks()
    ex = NVFP4Experts.random(E, H, F, "cuda", seed=0)
    x = torch.randn(T, H, device="cuda").bfloat16()
    idx, w = K.router_topk(torch.randn(T, E, device="cuda"), k, "softmax")
    plan = cuda_moe.moe_plan(idx, E, 128)
    parts = {}
    parts["quantise x"] = time_op(lambda: cuda_moe.quantize_entries(x, plan, k, False), iters=iters)
    xq, sfx = cuda_moe.quantize_entries(x, plan, k, False)
    parts["w13+glu"] = time_op(lambda: cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, F, H, E, "swiglu"), iters=iters)
    h = cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, F, H, E, "swiglu")
    parts["quantise h"] = time_op(lambda: cuda_moe.quantize_entries(h, plan, k, True), iters=iters)
    hq, sfh = cuda_moe.quantize_entries(h, plan, k, True)
    parts["w2"] = time_op(lambda: cuda_moe.grouped_gemm(ex.w2_q, ex.w2_sf, ex.w2_s2, hq, sfh, plan, H, F, E, None), iters=iters)
    y = cuda_moe.grouped_gemm(ex.w2_q, ex.w2_sf, ex.w2_s2, hq, sfh, plan, H, F, E, None)
    parts["un-permute"] = time_op(lambda: cuda_moe.unpermute(y, plan, w, T, k, None), iters=iters)
    b13 = E * 2 * F * H * (0.5 + 1 / 16)
    b2 = E * H * F * (0.5 + 1 / 16)
    fl = 2.0 * T * k * 3 * F * H
    print(f"nvfp4 expert MLP, prefill-shaped: E={E} H={H} F={F} T={T} k={k}, {int(plan.meta[0])} token tiles of 128")
    for name, ms in parts.items():
        b = b13 if name == "w13+glu" else b2 if name == "w2" else 0
        print(f"  {name:<12}{ms:8.4f} ms" + (f"  weights {b / 1e6:.0f} MB, {b / ms / 1e6:.0f} GB/s ({b / ms / 1e6 / hbm:.2f} {tag})" if b else ""))
    full = time_op(lambda: cuda_moe.experts_forward(x, idx, w, ex), iters=iters)
    print(f"  whole layer {full:8.4f} ms: weights at {(b13 + b2) / full / 1e6:.0f} GB/s ({(b13 + b2) / full / 1e6 / hbm:.2f} {tag}), "
          f"{fl / full / 1e9:.0f} TFLOP/s on the routed rows")
    assert K.last_status() == 0


def bench_membw(gib: int = 2, iters: int = 10):
    """Own read and copy sweeps over a buffer far larger than L2 (the reference's ``inkling_membw``), beside the measured copy peak."""
    from .cuda import _p, _stream, check, declare, lib
    declare("mary_stream_read", "plps")
    declare("mary_stream_copy", "ppls")
    hbm, _, tag = peaks()
    n = gib << 30
    src = torch.empty(n, dtype=torch.uint8, device="cuda").random_()
    dst = torch.empty_like(src)
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    ms = time_op(lambda: check(lib().mary_stream_read(_p(src), n, _p(sink), _stream()), "stream_read"), iters)
    print(f"stream read {gib} GiB: {ms:.3f} ms, {n / ms / 1e6:.0f} GB/s, {n / ms / 1e6 / hbm:.2f} {tag}")
    ms = time_op(lambda: check(lib().mary_stream_copy(_p(src), _p(dst), n, _stream()), "stream_copy"), iters)
    print(f"stream copy {gib} GiB: {ms:.3f} ms, {2 * n / ms / 1e6:.0f} GB/s read + write, {2 * n / ms / 1e6 / hbm:.2f} {tag}")
    assert torch.equal(src[-4096:], dst[-4096:])


def bench_bf16moe(E: int = 128, H: int = 2816, F: int = 704, T: int = 32, k: int = 8, iters: int = 10):
    """Unquantised routed experts (the grouped bf16 GEMM): device plan + gather + two grouped GEMMs + un-permute, against the per-expert
    loop.  Bytes = weights of the experts that are hit (decode streams them once)."""
    from . import bf16_experts
    hbm, _, tag = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    gate_up = (torch.randn(E, 2 * F, H, device="cuda", generator=g) * H ** -0.5).bfloat16()
    down = (torch.randn(E, H, F, device="cuda", generator=g) * F ** -0.5).bfloat16()
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(T)]).int()
    w = torch.rand(T, k, device="cuda", generator=g)
    hit = int(idx.unique().numel())
    ms = time_op(lambda: bf16_experts(x, idx, w, gate_up, down, 0, "geglu"), iters)
    gb = hit * 3 * F * H * 2 / 1e9
    print(f"bf16 experts E={E} H={H} F={F} T={T} k={k}: {ms:.4f} ms, {hit} experts hit, {gb / ms * 1e3:.0f} GB/s of expert weights, "
          f"{gb / ms * 1e3 / hbm:.2f} {tag}")


def bench_floor(reps: int = 200):
    """Per-launch cost of decode-sized kernels in steady state: ``reps`` back-to-back launches recorded in one CUDA graph and
    replayed (what a decode step sees), against the same launches issued eagerly."""
    from . import cuda as K
    x = torch.randn(48, 7168, device="cuda").bfloat16()
    cases = {
        "gemm 48x128x512 (one tile)": (lambda a=torch.randn(48, 512, device="cuda").bfloat16(), w=torch.randn(128, 512, device="cuda").bfloat16(): K.gemm(a, w)),
        "gemm 48x2112x7168 (stream-K)": (lambda w=(torch.randn(2112, 7168, device="cuda") * 0.02).bfloat16(): K.linear(x, w)),
        "gemm 48x7168x8192 (stream-K)": (lambda a=torch.randn(48, 8192, device="cuda").bfloat16(), w=(torch.randn(7168, 8192, device="cuda") * 0.02).bfloat16(): K.linear(a, w)),
        "gemm 48x384x7168 f32 (router)": (lambda w=(torch.randn(384, 7168, device="cuda") * 0.02).bfloat16(): K.linear_f32(x, w)),
        "rmsnorm 48x7168": (lambda g=torch.ones(7168, device="cuda").bfloat16(): K.rmsnorm(x, g)),
        # one token: the tensor-core GEMM against the matrix-vector stage of the fused layer step (weights L2-resident: the floor)
        "gemm 1x2048x1024": (lambda a=torch.randn(1, 1024, device="cuda").bfloat16(), w=(torch.randn(2048, 1024, device="cuda") * 0.02).bfloat16(): K.gemm(a, w)),
        "step_matvec 1x2048x1024": (lambda a=torch.randn(1, 1024, device="cuda").bfloat16(), w=(torch.randn(2048, 1024, device="cuda") * 0.02).bfloat16(): K.step_matvec(a, w)),
        "gemm 1x7168x8192 (117 MB)": (lambda a=torch.randn(1, 8192, device="cuda").bfloat16(), w=(torch.randn(7168, 8192, device="cuda") * 0.02).bfloat16(): K.linear(a, w)),
        "step_matvec 1x7168x8192 (117 MB)": (lambda a=torch.randn(1, 8192, device="cuda").bfloat16(), w=(torch.randn(7168, 8192, device="cuda") * 0.02).bfloat16(): K.step_matvec(a, w)),
        "step_matvec 1x151936x4096 (1.2 GB head)": (lambda a=torch.randn(1, 4096, device="cuda").bfloat16(), w=(torch.randn(151936, 4096, device="cuda") * 0.02).bfloat16(): K.step_matvec(a, w)),
        "gemm 1x151936x4096 (1.2 GB head)": (lambda a=torch.randn(1, 4096, device="cuda").bfloat16(), w=(torch.randn(151936, 4096, device="cuda") * 0.02).bfloat16(): K.linear(a, w)),
    }
    for name, fn in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        print(f"{name}: {a.elapsed_time(b) / reps * 1e3:.2f} us per launch in a graph of {reps}")
    assert K.last_status() == 0


def bench_matvec(N: int = 7168, K: int = 8192, iters: int = 10):
    """One-token product ``W[N, K] x``: the SIMT matrix-vector stage of the fused layer step against the tensor-core GEMM launch
    (L2 flushed between iterations: a weight stream from memory)."""
    from . import cuda as K_
    hbm, tf, tag = peaks()
    a = torch.randn(1, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    for name, fn in (("step_matvec", lambda: K_.step_matvec(a, w)), ("gemm", lambda: K_.gemm_splitk(a, w, 0) if K_._auto_split_k(1, N, K) > 1 else K_.gemm(a, w))):
        ms = time_op(fn, iters=iters)
        print(f"{name} 1 x {N} x {K}: {ms * 1e3:.1f} us, {N * K * 2 / ms / 1e6:.0f} GB/s ({N * K * 2 / ms / 1e6 / hbm:.2f} {tag})")
    assert K_.last_status() == 0


def bench_ttsframe(iters: int = 30):
    """One frame of the Qwen3-TTS code predictor at its released size (5 layers x 1024, 15 sequential steps, 2048-entry heads):
    eager launches against the one-graph replay of the same frame."""
    from ..models.qwen3tts.model import CodePredictor, Qwen3TTSConfig, Talker, init_random_
    c = Qwen3TTSConfig(talker_layers=1)
    tk, pr = Talker(c, torch.bfloat16, "cuda"), CodePredictor(c, torch.bfloat16, "cuda")
    init_random_(tk, pr, 0)
    h = (torch.randn(c.talker_hidden, device="cuda") * 0.5).to(torch.bfloat16)
    e0 = (torch.randn(c.talker_hidden, device="cuda") * 0.5).to(torch.bfloat16)
    from ..models.mistral import model as mistral
    out = {}
    for name, flag, fused in (("eager", False, True), ("graph", True, True), ("graph9", True, False)):
        pr.use_graph = flag
        pr._graph = None
        mistral.set_layer_step(fused)
        for _ in range(3):
            pr.predict_frame(h, e0)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            pr.predict_frame(h, e0)
        b.record()
        torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / iters
    w = sum(p.numel() * p.element_size() for p in pr.stack.parameters()) * (c.num_code_groups - 1)
    print(f"qwen3tts code predictor frame ({c.num_code_groups - 1} steps x {c.pred_layers} layers): eager {out['eager'] * 1e3:.0f} us, graph "
          f"{out['graph'] * 1e3:.0f} us per frame ({out['eager'] / out['graph']:.2f}x); the graph with the nine-launch layers instead of the "
          f"five-launch fused layer step: {out['graph9'] * 1e3:.0f} us; {w / 1e6:.0f} MB of weights read per frame; "
          f"a 12.5 Hz frame budget is 80000 us")
    mistral.set_layer_step(True)


def bench_talker(steps: int = 32):
    """One-token decode steps of the Qwen3-TTS talker stack (28 layers x 2048, FFN 6144, 16 / 8 heads of 128) in a CUDA graph: the
    nine-launch layers against the five-launch fused layer step (whose matrix-vector stages lose to a GEMM launch on matrices of
    this size; the launch count decides)."""
    import numpy as np
    from ..models.mistral import model as M
    from ..models.qwen3tts.model import Qwen3TTSConfig
    from ..runtime.batch import BatchMeta
    from ..runtime.kv_cache import PagedKVCache
    cfg = Qwen3TTSConfig().talker_cfg()
    model = M.MistralModel(cfg, dtype=torch.bfloat16, device="cuda")
    M.init_random_(model, 0)
    spec = model.kv_spec()
    ctx = 512
    out = {}
    saved = M._STEP_MAX_BYTES
    for name, fused in (("nine-launch layers", False), ("five-launch layer step", True)):
        M.set_layer_step(fused)
        M._STEP_MAX_BYTES = 1 << 40
        cache = PagedKVCache(spec["num_layers"], (ctx + steps) // 16 + 2, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16, device="cuda")
        cache.alloc.extend(0, ctx + steps)
        table, _ = cache.alloc.page_table([0])
        h = (torch.randn(1, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        metas = [BatchMeta.build([1], [ctx + i + 1], table, 16, "cuda") for i in range(steps)]
        with torch.no_grad():
            for m in metas:                                   # every step once eagerly: per-step descriptors are built on the host
                model.hidden_from_embeds(h, m, cache)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for m in metas:
                    model.hidden_from_embeds(h, m, cache)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                g.replay()
            b.record()
            torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / (3 * steps)
    M._STEP_MAX_BYTES = saved
    M.set_layer_step(True)
    w = sum(p.numel() * p.element_size() for n, p in model.named_parameters() if "layers" in n)
    print(f"talker one-token step ({cfg.num_hidden_layers} layers, {w / 1e6:.0f} MB of layer weights, context {ctx}): " +
          ", ".join(f"{k} {v * 1e3:.0f} us" for k, v in out.items()))


def bench_depformer(iters: int = 30):
    """The depth transformer of the full-duplex speech LM at its released size (16 steps x 6 layers x 1024, per-step weights): one frame's
    greedy chain eager against the one-graph replay."""
    from ..models.moshi.model import Depformer, MoshiConfig
    c = MoshiConfig()
    d = Depformer(c, torch.bfloat16, "cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    for n, p in d.named_parameters():
        p.data.fill_(1.0) if n in ("norm1", "norm2") else p.data.normal_(0.0, 0.03, generator=g)
    h = (torch.randn(1, c.dim, device="cuda") * 0.5).to(torch.bfloat16)
    text = torch.tensor([5], device="cuda")
    forced = [None] * 8 + [3] * 8                                          # the user's eight codebooks are forced, the agent's generated
    out = {}
    for name, flag in (("eager", False), ("graph", True)):
        d.use_graph = flag
        for _ in range(3):
            d.generate(h, text, forced)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            d.generate(h, text, forced)
        b.record()
        torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / iters
    print(f"speech LM depth transformer frame ({c.dep_q} steps x {c.dep_layers} layers): eager {out['eager'] * 1e3:.0f} us, graph "
          f"{out['graph'] * 1e3:.0f} us per frame ({out['eager'] / out['graph']:.2f}x); a 12.5 Hz frame budget is 80000 us")


def bench_speechlm(frames: int = 40):
    """The full-duplex speech LM at its released size (temporal 32 x 4096, depth 6 x 1024 x 16 steps), one conversation: milliseconds
    per 80 ms frame of ``LmGen.step`` (stream bookkeeping on the host, temporal step on the paged cache, text head, depth chain)
    with the user's eight codebooks provided every frame, and the real-time factor."""
    import time
    from ..models.moshi.model import LmGen, MoshiConfig
    c = MoshiConfig()
    m = LmGen(c, torch.bfloat16, "cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    for n, p in m.named_parameters():
        if p.dim() == 1 or n.endswith(("norm1", "norm2")):
            p.data.fill_(1.0)
        else:
            p.data.normal_(0.0, 0.02, generator=g)
    user = [7] * c.codebooks_per_stream
    for _ in range(6):
        m.step(user_audio=user)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(frames):
        m.step(user_audio=user)
    b.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / frames * 1e3
    dev = a.elapsed_time(b) / frames
    print(f"speech LM frame (temporal {c.layers} x {c.dim} + depth {c.dep_q} x {c.dep_layers} x {c.dep_dim}): {dev:.2f} ms device, {wall:.2f} ms wall "
          f"per 80 ms frame = {80.0 / wall:.1f}x real time")


def bench_vla(iters: int = 10):
    """SmolVLA at its released size (SigLIP 12 x 768 at 512 px, backbone 16 x 960, action expert 16 x 720, 10 Euler steps over a chunk of
    50 actions): one ``act`` call eager against the one-graph flow sampler."""
    from ..models.smolvla import SmolVLA, SmolVLAConfig
    c = SmolVLAConfig()
    m = SmolVLA(c)
    for p in m.parameters():
        p.data = p.data.to("cuda", torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(0)
    for n, p in m.named_parameters():
        if p.dim() == 1:
            p.data.fill_(0.0 if (n.endswith("_b") or "b_" in n.split(".")[-1]) else 1.0)
        else:
            p.data.normal_(0.0, 0.02, generator=g)
    img = (torch.rand(3, c.image_size, c.image_size, device="cuda") * 2 - 1).to(torch.bfloat16)
    state, noise = torch.randn(c.state_dim, device="cuda"), torch.randn(c.chunk_size, c.action_dim, device="cuda")
    ids = list(range(3, 51))
    out = {}
    for name, flag in (("eager", False), ("graph", True)):
        m.use_graph = flag
        for _ in range(2):
            m.act([img], ids, state, noise=noise)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            m.act([img], ids, state, noise=noise)
        b.record()
        torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / iters
    print(f"smolvla act (1 image, 48 language tokens, {c.num_steps} Euler steps x {c.expert.n_layers} expert layers): eager {out['eager']:.2f} ms, "
          f"flow sampler as one graph {out['graph']:.2f} ms per call ({out['eager'] / out['graph']:.2f}x)")


def bench_f5(frames: int = 800, nfe: int = 32):
    """F5-TTS flow sampler at the released size (DiT 22 x 1024, classifier-free guidance = two passes per step): one utterance of
    ``frames`` mel frames, eager against the replayed one-step graph (capture included in the timed call)."""
    from ..models.f5 import CFM, DiT, F5Config
    c = F5Config()
    d = DiT(c)
    for p in d.parameters():
        p.data = p.data.to("cuda", torch.bfloat16)
    for k, b in list(d._buffers.items()):
        d._buffers[k] = b.to("cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    for n, p in d.named_parameters():
        p.data.normal_(0.0, 0.02, generator=g)
    ref_mel = torch.randn(frames // 3, c.n_mels, device="cuda").to(torch.bfloat16)
    noise = torch.randn(frames, c.n_mels, device="cuda").to(torch.bfloat16)
    ids = [int(x) % (c.text_vocab - 1) for x in range(120)]
    cfm = CFM(d, nfe=nfe)
    out = {}
    for name, flag in (("eager", False), ("graph", True)):
        cfm.use_graph = flag
        cfm.sample(ref_mel, ids, frames, noise=noise)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            cfm.sample(ref_mel, ids, frames, noise=noise)
        b.record()
        torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / 3
    secs = (frames - frames // 3) * 256 / 24000
    print(f"f5 flow sampler ({frames} frames, {nfe} steps x 2 guidance passes x {c.depth} blocks): eager {out['eager']:.1f} ms, one-step graph "
          f"{out['graph']:.1f} ms per utterance ({out['eager'] / out['graph']:.2f}x); {secs:.1f} s of generated speech")


def bench_ep(world: int = 8, T: int = 48, E: int = 384, H: int = 7168, F: int = 2048, k: int = 8, iters: int = 5):
    """One expert-parallel MoE layer in all-to-all mode with all ranks on this device, phase by phase (the barriers between
    the phases are stream order here): the per-rank cost of counts, plan + dispatch, expert GEMMs and the weighted sum at the
    shape one rank of an 8-GPU decode step sees (48 home rows, 384 received rows, 48 local experts).  With
    ``torch.cuda.profiler`` the single profiled pass is bracketed for a launch list."""
    from . import cuda as K
    from .moe import NVFP4Experts
    from ..parallel.ep import EPBuffers, EPLayer, emulate
    e_local = E // world
    slab = NVFP4Experts.random(e_local, H, F, "cuda", seed=0)          # every rank reads the same bytes: what counts is the size
    bufs = [EPBuffers(world, E, H, F, t_cap=T, k=k, nt=32, device="cuda") for _ in range(world)]
    layers = [EPLayer(r, world, slab, bufs[r], bufs) for r in range(world)]
    xs = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(world)]
    routed = [K.router_topk(torch.randn(T, E, device="cuda"), k, "softmax") for _ in range(world)]
    idxs, ws = [i for i, _ in routed], [w for _, w in routed]
    ms = time_op(lambda: emulate(layers, xs, idxs, ws), iters=iters)
    torch.cuda.profiler.start()
    emulate(layers, xs, idxs, ws)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"ep all-to-all layer, {world} ranks on one device, T={T}/rank E={E} H={H} F={F} k={k}: {ms:.3f} ms for all ranks, "
          f"{ms / world * 1e3:.1f} us per rank")
    assert K.last_status() == 0


def bench_epf(world: int = 8, T: int = 48, E: int = 384, H: int = 7168, F: int = 2048, k: int = 8, iters: int = 5, shared: int = 1):
    """The same layer through the four-launch pipeline (route + dispatch by atomics, counter-mode GEMMs with the quantising GLU
    epilogue, combine), all ranks on this device phase by phase; the router GEMM is not part of either figure."""
    from . import cuda as K
    from .moe import NVFP4Experts
    from ..parallel.ep_fused import emulate, emulated_ranks
    e_local = E // world
    slab = NVFP4Experts.random(e_local + (1 if shared else 0), H, F, "cuda", seed=0)
    ranks = emulated_ranks(world, E, H, F, T, k, bool(shared), "cuda")
    xs = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(world)]
    lgs = [torch.randn(T, E, device="cuda") for _ in range(world)]
    router = dict(mode="sigmoid", bias=torch.zeros(E, device="cuda"), n_group=8, topk_group=4, scale=2.5, renorm=True)
    exs = [slab] * world
    ms = time_op(lambda: emulate(ranks, exs, xs, lgs, router), iters=iters)
    torch.cuda.profiler.start()
    emulate(ranks, exs, xs, lgs, router)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"ep fused layer, {world} ranks on one device, T={T}/rank E={E} H={H} F={F} k={k} shared={shared}: {ms:.3f} ms for all ranks, "
          f"{ms / world * 1e3:.1f} us per rank")
    assert K.last_status() == 0


if __name__ == "__main__":
    # ``gemm M N K`` / ``attn B L Hq Hkv D window`` / ``fa B L Hq Hkv DK DV window`` / ``mla B L Hq q_len`` / ``moe E H F T k`` run that one case only
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    nums = [int(v) for v in sys.argv[2:]]
    if what == "membw":
        bench_membw(*nums)
    if what == "moeprefill":
        bench_moeprefill(*nums)
    if what == "bf16moe":
        bench_bf16moe(*nums)
    if what in ("gemm", "all"):
        bench_gemm([tuple(nums)] if nums and what == "gemm" else None)
    if what in ("attn", "all"):
        bench_attn([tuple(nums)] if nums and what == "attn" else None)
    if what in ("fa", "all"):
        if nums and what == "fa":
            bench_fa(*nums)
        else:
            bench_fa()
            bench_fa(1, 4096, 16, 8, 256, 256)
            bench_fa(1, 4096, 32, 8, 128, 128)
            bench_fa(1, 4096, 16, 8, 256, 256, 1024)
    if what in ("mla", "all"):
        if nums and what == "mla":
            bench_mla(*nums)
        else:
            for pg in (16, 32):
                bench_mla(page=pg)
                bench_mla(Hq=8, page=pg)
                bench_mla(B=16, page=pg)
    if what == "matvec":
        bench_matvec(*nums)
    if what == "floor":
        bench_floor(*nums)
    if what == "ttsframe":
        bench_ttsframe(*nums)
    if what == "talker":
        bench_talker(*nums)
    if what == "depformer":
        bench_depformer(*nums)
    if what == "speechlm":
        bench_speechlm(*nums)
    if what == "vla":
        bench_vla(*nums)
    if what == "f5":
        bench_f5(*nums)
    if what == "ep":
        bench_ep(*nums)
    if what == "epf":
        bench_epf(*nums)
    if what in ("moe", "all"):
        bench_moe(*(nums if what == "moe" else []))

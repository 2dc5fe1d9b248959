"""NVFP4 quantiser, grouped block-scaled GEMM and the MoE pipeline against fp32 references (needs a B200)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from mary_b200.ops import reference as ref
from mary_b200.ops.moe import NVFP4Experts, experts_reference, swizzle_scales, unswizzle_scales


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-9)).item()


def test_swizzle_roundtrip_cpu_twin():
    sc = torch.randint(0, 255, (256, 28), dtype=torch.uint8)
    assert torch.equal(unswizzle_scales(swizzle_scales(sc), 256, 28), sc)
    from mary_b200.nn.fp4 import swizzle_scales_128x4
    assert np.array_equal(swizzle_scales_128x4(sc.numpy()), swizzle_scales(sc).numpy())


def test_activation_quantiser_is_bit_exact():
    from mary_b200.ops import cuda_moe
    torch.manual_seed(0)
    x = (torch.randn(67, 1024, device="cuda") * 3).bfloat16()
    x[0, :16] = 0
    x[1, :16] = 3e4
    x[2, 0] = -1e-30
    # exact ties on the code thresholds: block scale 1.0 (amax 6) with values .25 .75 1.25 1.75 2.5 3.5 5
    x[3, :16] = torch.tensor([6, .25, .75, 1.25, 1.75, 2.5, 3.5, 5, -.25, -.75, -1.25, -1.75, -2.5, -3.5, -5, 0.0]).bfloat16()
    codes, sf, rm = cuda_moe.quantize_rows(x, nt=128, rowmajor=True)
    wc, ws = ref.quantize_nvfp4(x.cpu())
    assert torch.equal(codes.cpu(), wc) and torch.equal(rm.cpu(), ws)
    assert torch.equal(unswizzle_scales(sf.cpu(), 67, 64), ws)
    assert codes[3, :8].tolist() == [0x17, 0x32, 0x54, 0x76, 0xA9, 0xCB, 0xED, 0x0F]


@pytest.mark.parametrize("T,k,nt", [(1200, 2, 128), (300, 8, 128), (512, 4, 32), (256, 9, 128)])
def test_token_driven_quantiser_writes_the_bytes_of_the_row_quantiser(T, k, nt):
    """Batches of 2048 entries and more quantise each token once and copy the bytes to its k padded rows: same codes and
    scales as the quantiser that works row by row."""
    from mary_b200.ops import cuda, cuda_moe
    torch.manual_seed(T)
    E, H = 16, 1024
    x = (torch.randn(T, H, device="cuda") * 2).bfloat16()
    idx, _ = cuda.router_topk(torch.randn(T, E, device="cuda"), k, "softmax")
    plan = cuda_moe.moe_plan(idx, E, nt)
    assert T * k >= 2048
    xq, sf = cuda_moe.quantize_entries(x, plan, k, identity=False)
    wq, wsf, _ = cuda_moe.quantize_rows(x, nt=nt, src_of=plan.src_of, identity=False, rows=plan.max_rows)
    torch.cuda.synchronize()
    rows = plan.row_of.long()
    assert (rows >= 0).all() and torch.equal(xq[rows], wq[rows])
    a = unswizzle_scales(sf.cpu(), sf.shape[0] * 128, H // 16).view(-1, 128, H // 16)
    b = unswizzle_scales(wsf.cpu(), wsf.shape[0] * 128, H // 16).view(-1, 128, H // 16)
    rr = rows.cpu()
    assert torch.equal(a[rr // nt, rr % nt], b[rr // nt, rr % nt])


@pytest.mark.parametrize("E,H,F,T,k,nt", [(4, 512, 256, 24, 2, 32), (16, 1024, 512, 200, 4, 32), (8, 512, 256, 700, 2, 128),
                                          (8, 1024, 256, 3, 2, 32)])
def test_moe_pipeline_matches_oracle(E, H, F, T, k, nt):
    from mary_b200.ops import cuda, cuda_moe
    torch.manual_seed(E + T)
    ex = NVFP4Experts.random(E, H, F, "cuda", std=0.05, seed=1)
    x = torch.randn(T, H, device="cuda").bfloat16()
    lg = torch.randn(T, E, device="cuda")
    idx, w = cuda.router_topk(lg, k, "softmax")
    got = cuda_moe.experts_forward(x, idx, w, ex, None, nt)
    want = experts_reference(x, idx, w, ex)
    assert cuda.last_status() == 0
    assert _rel(got.cpu(), want) < 3e-2, _rel(got.cpu(), want)


def test_grouped_gemm_is_exact_on_its_quantised_operands():
    """f64 arbiter over the SAME quantised operands: the block-scaled MMA must reproduce it to f32 accuracy."""
    from mary_b200.ops import cuda, cuda_moe
    torch.manual_seed(3)
    E, H, F, T = 3, 512, 256, 40
    ex = NVFP4Experts.random(E, H, F, "cuda", std=0.05, seed=2)
    idx = torch.randint(0, E, (T, 1), device="cuda", dtype=torch.int32)
    plan = cuda_moe.moe_plan(idx, E, 32)
    # plain (non-GLU) GEMM over w2-shaped operands: K = F on a quantised [T, F] input
    h = torch.randn(T, F, device="cuda").bfloat16()
    hq, sfh, hrm = cuda_moe.quantize_rows(h, 32, plan.src_of, identity=False, rows=plan.max_rows, rowmajor=True)
    y = cuda_moe.grouped_gemm(ex.w2_q, ex.w2_sf, ex.w2_s2, hq, sfh, plan, H, F, E, None)
    assert cuda.last_status() == 0
    row_of = plan.row_of.cpu()
    for t in range(T):
        r = int(row_of[t])
        e = int(idx[t, 0])
        a = ref.dequantize_nvfp4(hq[r:r + 1].cpu(), hrm[r:r + 1].cpu()).double()
        want = (a @ ex.dense("w2", e).double().T).float()
        assert _rel(y[r:r + 1].cpu(), want) < 1e-2      # bf16 output rounding only


@pytest.mark.parametrize("world", [2, 4])
def test_ep_all_to_all_dispatch_combine_emulated(world):
    """Expert-parallel all-to-all (dispatch by peer stores, combine from the GEMM epilogue) with all ranks on one device:
    every rank's output must equal the single-rank expert MLP over the union of the experts."""
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.models.moe.shard import slice_experts
    from mary_b200.parallel.ep import EPBuffers, EPLayer, emulate
    torch.manual_seed(world)
    E, H, F, k, T = 8 * world, 512, 256, 2, 40
    ex = NVFP4Experts.random(E, H, F, "cuda", std=0.05, seed=3)
    bufs = [EPBuffers(world, E, H, F, t_cap=64, k=k, nt=32, device="cuda") for _ in range(world)]
    layers = [EPLayer(r, world, slice_experts(ex, r, world), bufs[r], bufs) for r in range(world)]
    xs = [torch.randn(T - 3 * r, H, device="cuda").bfloat16() for r in range(world)]       # ranks hold different token counts
    routed = [cuda.router_topk(torch.randn(x.shape[0], E, device="cuda"), k, "softmax") for x in xs]
    outs = emulate(layers, xs, [i for i, _ in routed], [w for _, w in routed])
    torch.cuda.synchronize()
    assert cuda.last_status() == 0
    for x, (idx, w), got in zip(xs, routed, outs):
        want = cuda_moe.experts_forward(x, idx, w, ex, None, 32)
        assert _rel(got, want) < 2e-2, _rel(got, want)
    # a second layer call reuses the slabs
    outs2 = emulate(layers, xs, [i for i, _ in routed], [w for _, w in routed])
    for a, b in zip(outs, outs2):
        assert torch.equal(a, b)


def test_ep_all_to_all_serves_the_shared_expert_in_the_same_launches():
    """A shared NVFP4 expert kept behind every rank's routed experts: its rows never leave the rank, ride in the same grouped
    GEMM launches and come back through the combine buffer as one more entry per token."""
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.models.moe.shard import slice_experts
    from mary_b200.parallel.ep import EPBuffers, EPLayer, emulate
    world = 4
    torch.manual_seed(9)
    E, H, F, k, T = 8 * world, 512, 256, 2, 37
    ex = NVFP4Experts.random(E + 1, H, F, "cuda", std=0.05, seed=5)          # the last one is the shared expert
    bufs = [EPBuffers(world, E, H, F, t_cap=64, k=k, nt=32, device="cuda", shared=True) for _ in range(world)]
    layers = [EPLayer(r, world, slice_experts(ex, r, world, tail=1), bufs[r], bufs) for r in range(world)]
    xs = [torch.randn(T - 5 * r, H, device="cuda").bfloat16() for r in range(world)]
    routed = [cuda.router_topk(torch.randn(x.shape[0], E, device="cuda"), k, "softmax") for x in xs]
    outs = emulate(layers, xs, [i for i, _ in routed], [w for _, w in routed])
    torch.cuda.synchronize()
    assert cuda.last_status() == 0
    for x, (idx, w), got in zip(xs, routed, outs):
        n = x.shape[0]
        idx2 = torch.cat([idx.to(torch.int32), torch.full((n, 1), E, dtype=torch.int32, device="cuda")], 1)
        w2 = torch.cat([w.float(), torch.ones(n, 1, device="cuda")], 1)
        want = cuda_moe.experts_forward(x, idx2, w2, ex, None, 32)
        assert _rel(got, want) < 2e-2, _rel(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("E,H,F,T,k,act", [(8, 256, 128, 40, 2, "geglu"), (32, 512, 256, 16, 4, "swiglu"), (4, 256, 384, 700, 2, "geglu")])
def test_grouped_bf16_experts_match_the_per_expert_loop(E, H, F, T, k, act):
    """Unquantised experts through the grouped tensor-core GEMM (routing plan tiles of 32 / 64 / 128 rows, GLU epilogue, unused tiles
    skipped) against the f32 per-expert loop; a shard of the experts (``e0``) ignores entries routed elsewhere."""
    from mary_b200 import ops
    g = torch.Generator().manual_seed(E + T)
    x = torch.randn(T, H, generator=g) * 0.5
    gate_up, down = torch.randn(E, 2 * F, H, generator=g) * H ** -0.5, torch.randn(E, H, F, generator=g) * F ** -0.5
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int()
    w = torch.rand(T, k, generator=g)
    xb, gb, db = x.bfloat16(), gate_up.bfloat16(), down.bfloat16()
    want = ops.bf16_experts(xb.float(), idx, w, gb.float(), db.float(), 0, act)
    got = ops.bf16_experts(xb.cuda(), idx.cuda(), w.cuda(), gb.cuda(), db.cuda(), 0, act)
    err = (got.float().cpu() - want).norm() / want.norm()
    assert err < 0.02, float(err)
    # the upper half of the experts only
    e0 = E // 2
    want_h = ops.bf16_experts(xb.float(), idx, w, gb.float()[e0:], db.float()[e0:], e0, act)
    got_h = ops.bf16_experts(xb.cuda(), idx.cuda(), w.cuda(), gb.cuda()[e0:].contiguous(), db.cuda()[e0:].contiguous(), e0, act)
    err = (got_h.float().cpu() - want_h).norm() / want_h.norm().clamp_min(1e-6)
    assert err < 0.02, float(err)
    assert mary_status_ok()


def mary_status_ok():
    from mary_b200.ops import cuda as K
    return K.lib().mary_last_status() == 0


# ----------------------------------------------------------------------------------------------------------------------
# The four-launch expert pipeline (route + dispatch, counter-mode GEMMs, combine)
def _router(mode, E, scale=1.0):
    if mode == "softmax":
        return dict(mode="softmax", bias=None, n_group=1, topk_group=1, scale=1.0, renorm=True)
    return dict(mode="sigmoid", bias=torch.randn(E, device="cuda") * 0.1, n_group=4, topk_group=2, scale=scale, renorm=True)


def _route(lg, k, r):
    from mary_b200.ops import cuda
    return cuda.router_topk(lg, k, r["mode"], r["bias"], r["n_group"], r["topk_group"], r["scale"], r["renorm"])


@pytest.mark.parametrize("E,H,F,T,k,shared,mode", [(8, 512, 256, 40, 2, False, "softmax"), (16, 1024, 512, 96, 4, True, "sigmoid"),
                                                  (32, 512, 256, 3, 8, True, "softmax")])
def test_fused_pipeline_equals_planned_path_on_one_rank(E, H, F, T, k, shared, mode):
    """Route + dispatch by atomics, counter-mode GEMMs with the quantising GLU epilogue and the combine kernel give the SAME bits
    as router -> plan -> quantise -> GEMM -> quantise -> GEMM -> un-permute: rows are independent and slots are summed in the
    same order.  Three calls in a row: the counters are back to zero and the epoch has advanced after each."""
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.parallel.ep_fused import FusedMoE
    torch.manual_seed(E + T)
    ex = NVFP4Experts.random(E + (1 if shared else 0), H, F, "cuda", std=0.05, seed=7)
    fm = FusedMoE(0, 1, E, H, F, 128, k, shared, "cuda", True)
    r = _router(mode, E, 2.5)
    for call in range(3):
        x = torch.randn(T, H, device="cuda").bfloat16()
        lg = torch.randn(T, E, device="cuda")
        got = fm.forward(x, lg, r, ex)
        idx, w = _route(lg, k, r)
        if shared:
            idx = torch.cat([idx.to(torch.int32), torch.full((T, 1), E, dtype=torch.int32, device="cuda")], 1)
            w = torch.cat([w.float(), torch.ones(T, 1, device="cuda")], 1)
        want = cuda_moe.experts_forward(x, idx, w, ex, None, 32)
        torch.cuda.synchronize()
        assert cuda.last_status() == 0
        assert torch.equal(fm.idx_out[:T], idx.to(torch.int32)) and torch.equal(fm.w_out[:T], w.float())
        assert torch.equal(got, want), (call, _rel(got, want))
        assert int(fm.bufs["cnt"].abs().sum()) == 0 and int(fm.epoch) == call + 1
        assert _rel(got.cpu(), experts_reference(x, idx, w, ex)) < 3e-2


def test_fused_pipeline_adds_residual_and_norms():
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.parallel.ep_fused import FusedMoE
    torch.manual_seed(5)
    E, H, F, T, k = 8, 512, 256, 33, 2
    ex = NVFP4Experts.random(E, H, F, "cuda", std=0.05, seed=8)
    fm = FusedMoE(0, 1, E, H, F, 64, k, False, "cuda", True)
    r = _router("softmax", E)
    x = torch.randn(T, H, device="cuda").bfloat16()
    lg = torch.randn(T, E, device="cuda")
    add = torch.randn(T, H, device="cuda").bfloat16()
    h = torch.randn(T, H, device="cuda").bfloat16()
    gain = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    f = fm.forward(x, lg, r, ex, add=add)
    want_y, want_h = cuda.add_rmsnorm(f, h.clone(), gain, 1e-6)
    h2 = h.clone()
    y, h_out = fm.forward(x, lg, r, ex, add=add, res=h2, w_norm=gain, eps=1e-6)
    torch.cuda.synchronize()
    assert cuda.last_status() == 0 and h_out.data_ptr() == h2.data_ptr()
    assert torch.equal(h2, want_h) and torch.equal(y, want_y)
    h3 = h.clone()
    y3, _ = fm.forward(x, lg, r, ex, add=add, res=h3, w_norm=None)
    assert y3 is None and torch.equal(h3, want_h)


@pytest.mark.parametrize("world,shared", [(2, False), (4, True), (8, True)])
def test_fused_pipeline_expert_parallel_emulated(world, shared):
    """All ranks on one device, phase by phase (every waiting kernel runs after the kernels it waits for): each rank's output
    equals the single-rank expert MLP over all experts, bit for bit, on two layer calls in a row."""
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.models.moe.shard import slice_experts
    from mary_b200.parallel.ep_fused import emulate, emulated_ranks
    torch.manual_seed(world)
    E, H, F, k, T = 8 * world, 512, 256, 2, 40
    ex = NVFP4Experts.random(E + (1 if shared else 0), H, F, "cuda", std=0.05, seed=3)
    ranks = emulated_ranks(world, E, H, F, 64, k, shared, "cuda")
    exs = [slice_experts(ex, r, world, tail=1 if shared else 0) for r in range(world)]
    r_cfg = _router("sigmoid", E, 2.5)
    for call in range(2):
        xs = [torch.randn(T - 3 * r, H, device="cuda").bfloat16() for r in range(world)]
        lgs = [torch.randn(x.shape[0], E, device="cuda") for x in xs]
        outs = emulate(ranks, exs, xs, lgs, r_cfg)
        torch.cuda.synchronize()
        assert cuda.last_status() == 0
        for x, lg, got in zip(xs, lgs, outs):
            idx, w = _route(lg, k, r_cfg)
            n = x.shape[0]
            if shared:
                idx = torch.cat([idx.to(torch.int32), torch.full((n, 1), E, dtype=torch.int32, device="cuda")], 1)
                w = torch.cat([w.float(), torch.ones(n, 1, device="cuda")], 1)
            want = cuda_moe.experts_forward(x, idx, w, ex, None, 32)
            assert torch.equal(got, want), (call, _rel(got, want))
        for rk in ranks:
            assert int(rk.bufs["cnt"].abs().sum()) == 0 and int(rk.epoch) == call + 1


def test_fused_pipeline_replicated_tokens_partial_sums():
    """``local_only`` contexts of a 2-rank group with replicated tokens: every rank serves its own experts (and the shared expert
    for its share of the tokens); the partial sums add up to the single-rank result."""
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.models.moe.shard import slice_experts
    from mary_b200.parallel.ep_fused import FusedMoE
    torch.manual_seed(11)
    world, E, H, F, k, T = 2, 16, 512, 256, 2, 48
    ex = NVFP4Experts.random(E + 1, H, F, "cuda", std=0.05, seed=4)
    r_cfg = _router("softmax", E)
    x = torch.randn(T, H, device="cuda").bfloat16()
    lg = torch.randn(T, E, device="cuda")
    parts = []
    for rank in range(world):
        fm = FusedMoE(rank, world, E, H, F, 64, k, True, "cuda", True)
        parts.append(fm.forward(x, lg, r_cfg, slice_experts(ex, rank, world, tail=1)).float())
    idx, w = _route(lg, k, r_cfg)
    idx = torch.cat([idx.to(torch.int32), torch.full((T, 1), E, dtype=torch.int32, device="cuda")], 1)
    w = torch.cat([w.float(), torch.ones(T, 1, device="cuda")], 1)
    want = cuda_moe.experts_forward(x, idx, w, ex, None, 32)
    assert cuda.last_status() == 0
    assert _rel(sum(parts), want) < 1e-2


def test_fused_pipeline_refuses_batches_beyond_its_slabs():
    from mary_b200.parallel.ep_fused import FusedMoE
    fm = FusedMoE(0, 1, 8, 512, 256, 32, 2, False, "cuda", True)
    ex = NVFP4Experts.random(8, 512, 256, "cuda", std=0.05, seed=1)
    with pytest.raises(ValueError):
        fm.forward(torch.zeros(33, 512, device="cuda").bfloat16(), torch.zeros(33, 8, device="cuda"), _router("softmax", 8), ex)


@pytest.mark.parametrize("nt,T", [(32, 70), (128, 300)])
def test_glu_epilogue_quantises_like_the_standalone_quantiser(nt, T):
    """GEMM -> bf16 -> quantise and GEMM with the quantising epilogue must write the same code and scale bytes."""
    from mary_b200.ops import cuda, cuda_moe
    from mary_b200.ops.cuda import _p, _stream, check, declare, lib
    declare("mary_gemm_nvfp4_grouped_glu_q", "ppppppppp" + "iiiliis")
    torch.manual_seed(nt)
    E, H, F, k = 4, 512, 256, 2
    ex = NVFP4Experts.random(E, H, F, "cuda", std=0.05, seed=2)
    x = torch.randn(T, H, device="cuda").bfloat16()
    idx, w = cuda.router_topk(torch.randn(T, E, device="cuda"), k, "softmax")
    plan = cuda_moe.moe_plan(idx, E, nt)
    xq, sfx = cuda_moe.quantize_entries(x, plan, k, identity=False)
    h = cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, F, H, E, ex.act)
    hq, sfh = cuda_moe.quantize_entries(h, plan, k, identity=True)
    hq2 = torch.zeros_like(hq)
    sfh2 = torch.zeros_like(sfh)
    check(lib().mary_gemm_nvfp4_grouped_glu_q(_p(ex.w13_q), _p(ex.w13_sf), _p(ex.w13_s2), _p(xq), _p(sfx), _p(plan.tiles), _p(plan.meta),
                                              _p(hq2), _p(sfh2), E, F, H, plan.max_rows, nt, 2, _stream()), "gemm_nvfp4_grouped")
    torch.cuda.synchronize()
    assert cuda.last_status() == 0
    rows = plan.row_of[plan.row_of >= 0].long()
    assert torch.equal(hq2[rows], hq[rows])
    tiles = (rows // nt).unique()
    a = unswizzle_scales(sfh2.cpu(), sfh2.shape[0] * 128, F // 16).view(-1, 128, F // 16)
    b = unswizzle_scales(sfh.cpu(), sfh.shape[0] * 128, F // 16).view(-1, 128, F // 16)
    rr = rows.cpu()
    assert torch.equal(a[rr // nt, rr % nt], b[rr // nt, rr % nt]) and len(tiles) > 0


def test_grouped_gemm_flagship_shape_against_f64_arbiter():
    """The K3-class expert shapes (K = 7168 -> 28 K-stages for w13, 16 weight tiles of F = 2048; K = 2048 for w2) on 16 experts:
    f64 arbiter over the SAME quantised operands.  The f32 accumulators are compared before any bf16 rounding would hide an
    error: the quantised intermediate of the GLU epilogue equals the quantised arbiter value, and the w2 output (bf16) is
    within half a bf16 ulp of the arbiter."""
    from mary_b200.ops import cuda, cuda_moe
    torch.manual_seed(21)
    E, H, F, T, k = 16, 7168, 2048, 48, 2
    ex = NVFP4Experts.random(E, H, F, "cuda", std=0.02, seed=6)
    x = torch.randn(T, H, device="cuda").bfloat16()
    idx, w = cuda.router_topk(torch.randn(T, E, device="cuda"), k, "softmax")
    plan = cuda_moe.moe_plan(idx, E, 32)
    xq, sfx = cuda_moe.quantize_entries(x, plan, k, identity=False)
    h = cuda_moe.grouped_gemm(ex.w13_q, ex.w13_sf, ex.w13_s2, xq, sfx, plan, F, H, E, ex.act)
    hq, sfh = cuda_moe.quantize_entries(h, plan, k, identity=True)
    y = cuda_moe.grouped_gemm(ex.w2_q, ex.w2_sf, ex.w2_s2, hq, sfh, plan, H, F, E, None)
    torch.cuda.synchronize()
    assert cuda.last_status() == 0
    xd = ref.dequantize_nvfp4(*ref.quantize_nvfp4(x.cpu())).double()
    row_of, idx_c = plan.row_of.cpu().view(T, k), idx.cpu()
    worst_h = worst_y = 0.0
    for e in idx_c.unique().tolist():
        t, j = (idx_c == e).nonzero(as_tuple=True)
        rows = row_of[t, j].long()
        w13 = ex.dense("w13", e).double()
        g, u = xd[t] @ w13[:F].T, xd[t] @ w13[F:].T
        h64 = torch.nn.functional.silu(g) * u
        got_h = h[rows].cpu().double()
        worst_h = max(worst_h, ((got_h - h64).abs() / (h64.abs() + 1e-3)).max().item())
        hd = ref.dequantize_nvfp4(*ref.quantize_nvfp4(h[rows].cpu())).double()
        y64 = hd @ ex.dense("w2", e).double().T
        worst_y = max(worst_y, ((y[rows].cpu().double() - y64).abs() / (y64.abs() + 1e-3)).max().item())
    # bf16 keeps 8 bits: half an ulp is 2^-9 relative; the f32 accumulation error over K = 7168 is far below that
    assert worst_h < 2 ** -8 and worst_y < 2 ** -8, (worst_h, worst_y)

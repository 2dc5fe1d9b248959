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

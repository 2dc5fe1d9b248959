"""The all-reduce kernel's protocol and data movement on ONE GPU: all ranks run as block groups of one cooperative launch
(kernels that wait on each other are never separate launches on a GPU); plus the bounded wait."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_allreduce_matches_sum(world):
    from mary_b200.ops.cuda import _stream, check, declare, last_status, lib
    declare("mary_allreduce_bf16_emulated", "ppilllpils")
    region = 4 << 20
    bufs = [torch.zeros(2 * region, dtype=torch.uint8, device="cuda") for _ in range(world)]
    sigs = [torch.zeros(1024, dtype=torch.int32, device="cuda") for _ in range(world)]
    bp = (ctypes.c_uint64 * 8)(*[b.data_ptr() for b in bufs])
    sp = (ctypes.c_uint64 * 8)(*[s.data_ptr() for s in sigs])
    epochs = torch.zeros(16 * world, dtype=torch.int32, device="cuda")
    for n in (8, 4096 + 8, 384 * 2048):
        torch.manual_seed(n)
        xs = [torch.randn(n, device="cuda").bfloat16() for _ in range(world)]
        want = torch.stack([x.float() for x in xs]).sum(0)
        for rep in range(2):                                   # flags are reused with a growing epoch
            for b, x in zip(bufs, xs):
                b[:n * 2].view(torch.bfloat16).copy_(x)
            check(lib().mary_allreduce_bf16_emulated(bp, sp, world, 0, region, n, epochs.data_ptr(), 16, int(2e9), _stream()),
                  "allreduce_emulated")
            torch.cuda.synchronize()
            assert last_status() == 0
            for b in bufs:                                      # every rank holds the full sum
                got = b[region:region + n * 2].view(torch.bfloat16).float()
                assert (got - want).abs().max() <= 2e-2 * want.abs().max()
            assert torch.equal(bufs[0][region:region + n * 2], bufs[-1][region:region + n * 2])


@pytest.mark.parametrize("world", [2, 8])
def test_emulated_oneshot_allreduce_mixed_lengths(world):
    """The one-shot (one barrier, staged) all-reduce on calls of alternating lengths: a call that needs one block, then calls
    that need two and five.  Block ``b`` owns the same 32 KB slice of the stage in every call, so the blocks' epochs (which
    advance only in the calls they take part in) always select a half of the stage that no peer still reads."""
    from mary_b200.ops.cuda import _stream, check, declare, last_status, lib
    declare("mary_allreduce_bf16_oneshot_emulated", "pppp" + "illlpils")
    stage_bytes = 1 << 20
    bufs = [torch.zeros(2 * stage_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    sigs = [torch.zeros(1024, dtype=torch.int32, device="cuda") for _ in range(world)]
    bp = (ctypes.c_uint64 * 8)(*[b.data_ptr() for b in bufs])
    sp = (ctypes.c_uint64 * 8)(*[s.data_ptr() for s in sigs])
    epochs = torch.zeros(64 * world, dtype=torch.int32, device="cuda")
    lengths = [2048 * 8, 2688 * 8, 2048 * 8, 5 * 2048 * 8 - 64, 8, 2688 * 8, 2048 * 8]
    for call, n in enumerate(lengths):
        torch.manual_seed(100 + call)
        xs = torch.randn(world, n, device="cuda").bfloat16()
        out = torch.zeros(world, n, dtype=torch.bfloat16, device="cuda")
        grid = (n // 8 + 2047) // 2048
        check(lib().mary_allreduce_bf16_oneshot_emulated(xs.data_ptr(), out.data_ptr(), bp, sp, world, 0, stage_bytes, n,
                                                         epochs.data_ptr(), grid, int(2e9), _stream()), "allreduce_oneshot_emulated")
        torch.cuda.synchronize()
        assert last_status() == 0
        acc = torch.zeros(n, dtype=torch.float32, device="cuda")
        for r in range(world):                                 # the kernel's order: rank 0 first, f32 accumulation
            acc += xs[r].float()
        want = acc.bfloat16()
        for r in range(world):
            assert torch.equal(out[r], want), (call, n, r)
    # a grid that does not cover the vector is refused
    assert lib().mary_allreduce_bf16_oneshot_emulated(xs.data_ptr(), out.data_ptr(), bp, sp, world, 0, stage_bytes, 4096 * 8,
                                                      epochs.data_ptr(), 1, int(2e9), _stream()) == 4


def test_bounded_wait_reports_timeout_and_context_survives():
    from mary_b200.ops.cuda import _stream, check, declare, last_status, lib
    declare("mary_wait_flag", "piiiils")
    sig = torch.zeros(1024, dtype=torch.int32, device="cuda")
    sp = (ctypes.c_uint64 * 8)(sig.data_ptr())
    check(lib().mary_wait_flag(sp, 0, 1, 5, 77, int(0.2e9), _stream()), "wait_flag")     # nothing ever sets flag 5
    torch.cuda.synchronize()
    assert last_status() == 3                                   # MARY_ERR_TIMEOUT_PEER, and the kernel returned
    assert (torch.ones(8, device="cuda") * 3).sum().item() == 24
    sig[6] = 99
    check(lib().mary_wait_flag(sp, 0, 1, 6, 99, int(0.2e9), _stream()), "wait_flag")     # a satisfied wait sets nothing
    torch.cuda.synchronize()
    assert last_status() == 0


@pytest.mark.parametrize("world,T", [(2, 64), (4, 384), (8, 384)])
def test_gemm_reduce_scatter_epilogue_and_fused_norm_allgather(world, T):
    """GEMM -> reduce-scatter from the epilogue, then reduce + residual + RMSNorm -> all-gather, with the ranks as buffer
    sets on one device (no kernel waits on another, so running the ranks one after the other is exact)."""
    from mary_b200.ops import cuda
    from mary_b200.ops import reference as ref
    from mary_b200.parallel.sp import SequenceParallel
    torch.manual_seed(world)
    H, Kl = 512, 256
    rpr = T // world
    stag = [torch.zeros(world * rpr * H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    xbuf = [torch.zeros(T * H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    sps = [SequenceParallel(r, world, T, H, "cuda", stag[r], xbuf[r], [s.data_ptr() for s in stag], [x.data_ptr() for x in xbuf])
           for r in range(world)]
    xs = [torch.randn(T, Kl, device="cuda").bfloat16() for _ in range(world)]
    ws = [(torch.randn(H, Kl, device="cuda") * 0.05).bfloat16() for _ in range(world)]
    h = torch.randn(T, H, device="cuda").bfloat16()
    gain = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    slices = [h[r * rpr:(r + 1) * rpr].clone() for r in range(world)]
    for r in range(world):
        sps[r].row_linear_rs(xs[r], ws[r])
    outs = [sps[r].reduce_add_rmsnorm(slices[r], gain, 1e-6) for r in range(world)]
    torch.cuda.synchronize()
    assert cuda.last_status() == 0
    partials = [(x.float() @ w.float().T).bfloat16().float() for x, w in zip(xs, ws)]
    h_new = (h.float() + sum(partials)).bfloat16()
    want = ref.rmsnorm(h_new, gain, 1e-6)
    for r in range(world):
        assert ((outs[r].float() - want.float()).abs().max() / want.float().abs().max()).item() < 2e-2
        assert ((slices[r].float() - h_new[r * rpr:(r + 1) * rpr].float()).abs().max()).item() < 0.1
    assert torch.equal(outs[0], outs[-1])                      # every rank holds the same gathered activations
    # sandwich norms: the sum is normed before it joins the residual, the new residual is scaled, then normed again
    from mary_b200 import ops
    post = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    slices = [h[r * rpr:(r + 1) * rpr].clone() for r in range(world)]
    for r in range(world):
        sps[r].row_linear_rs(xs[r], ws[r])
    outs = [sps[r].reduce_add_rmsnorm(slices[r], gain, 1e-6, w_post=post, scalar=0.5) for r in range(world)]   # views: read after ALL ranks ran
    torch.cuda.synchronize()
    a = sum(partials).bfloat16()
    want_x, want_h = ops.norm_add_norm(a, post, h.clone(), gain, 1e-6, 0.5)
    for r in range(world):
        assert ((outs[r].float() - want_x.float()).abs().max() / want_x.float().abs().max()).item() < 2e-2
        assert ((slices[r].float() - want_h[r * rpr:(r + 1) * rpr].float()).abs().max()).item() < 0.05
    # a row count that does not divide over the ranks: the last rank's tail rows are padding
    T2 = T - 3
    rpr2 = sps[0].rows_per_rank(T2)
    slices = [sps[r].residual_slice(h[:T2]) for r in range(world)]
    for r in range(world):
        sps[r].row_linear_rs(xs[r][:T2], ws[r])
    outs = [sps[r].reduce_add_rmsnorm(slices[r], gain, 1e-6) for r in range(world)]
    torch.cuda.synchronize()
    want2 = ref.rmsnorm((h[:T2].float() + sum(p[:T2] for p in partials)).bfloat16(), gain, 1e-6)
    assert outs[0].shape == (T2, H) and rpr2 * world >= T2
    assert ((outs[0].float() - want2.float()).abs().max() / want2.float().abs().max()).item() < 2e-2
    assert cuda.last_status() == 0


@pytest.mark.parametrize("world", [2, 8])
def test_vocab_parallel_argmax_merge_emulated(world):
    """All ranks of the arg-max merge inside one cooperative launch: every rank must end with the arg-max of the whole
    vocabulary, ties going to the lower global index, on two calls in a row (epoch parity flips the pair tables)."""
    import ctypes
    from mary_b200.ops import cuda
    cuda.declare("mary_argmax_merge_emulated", "ppiiipplipilpps")
    T, Tmax, vpr = 100, 128, 1000
    bufs = [torch.zeros(2 * 8 * Tmax * 8, dtype=torch.uint8, device="cuda") for _ in range(world)]
    sigs = [torch.zeros(64 * 2 * 8, dtype=torch.int32, device="cuda") for _ in range(world)]
    bp = (ctypes.c_uint64 * 8)(*[b.data_ptr() for b in bufs])
    sp = (ctypes.c_uint64 * 8)(*[s.data_ptr() for s in sigs])
    epochs = torch.zeros(world, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(1)
    for call in range(3):
        val = torch.randn(world, T, device="cuda", generator=g)
        idx = torch.randint(0, vpr, (world, T), device="cuda", generator=g)
        val[:, :10] = 7.0                                        # ties across all ranks: lowest global index must win
        out_i = torch.empty(world, T, dtype=torch.int64, device="cuda")
        out_v = torch.empty(world, T, dtype=torch.float32, device="cuda")
        cuda.check(cuda.lib().mary_argmax_merge_emulated(val.data_ptr(), idx.data_ptr(), T, Tmax, vpr, bp, sp, 0, world, epochs.data_ptr(),
                                                         62, int(2e9), out_i.data_ptr(), out_v.data_ptr(), cuda._stream()), "merge")
        torch.cuda.synchronize()
        assert cuda.last_status() == 0
        from mary_b200.parallel.vocab import merge_candidates
        gi = idx + torch.arange(world, device="cuda")[:, None] * vpr
        want_i, want_v = merge_candidates(val, gi)
        for r in range(world):
            assert torch.equal(out_i[r], want_i) and torch.equal(out_v[r], want_v), (call, r)
    assert epochs.tolist() == [3] * world

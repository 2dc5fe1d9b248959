"""CUDA kernels against plain PyTorch fp32 references of the same op (needs a B200)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from mary_b200.ops import reference as ref


@pytest.fixture(scope="module")
def K():
    from mary_b200.ops import cuda
    cuda.lib()
    return cuda


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-9)).item()


@pytest.mark.parametrize("M,N,K_", [(128, 256, 512), (300, 520, 1096), (1024, 1024, 2048), (32, 3840, 4096), (1, 128, 64),
                                     (64, 264, 7168), (257, 4104, 1536),
                                     (2048, 3840, 512), (4096, 1344, 256), (2000, 3848, 264)])     # column tiles of 224 / 192 (wave count)
def test_gemm_bf16_vs_fp32(K, M, N, K_):
    torch.manual_seed(M + N)
    x = torch.randn(M, K_, device="cuda").bfloat16()
    w = (torch.randn(N, K_, device="cuda") * 0.05).bfloat16()
    want = x.float() @ w.float().T
    for swap in (0, 1):
        got = K.gemm(x, w, swap=swap)
        assert _rel(got, want) < 1e-2, (swap, _rel(got, want))
        g32 = K.gemm(x, w, epi="f32", swap=swap)
        assert _rel(g32, want) < 2e-5 * np.sqrt(K_), (swap, _rel(g32, want))
    assert K.last_status() == 0


def test_gemm_split_k_bias_alpha_and_strided_input(K):
    torch.manual_seed(0)
    xf = torch.randn(48, 2 * 2048, device="cuda").bfloat16()
    x = xf[:, :2048]                                   # row pitch 4096, K 2048
    w = (torch.randn(520, 2048, device="cuda") * 0.05).bfloat16()
    b = torch.randn(520, device="cuda")
    want = x.float() @ w.float().T
    for sk in (2, 4, 7):
        got = K.gemm(x, w, epi="red", split_k=sk)
        assert _rel(got, want) < 1e-4
    got = K.gemm(x, w, bias=b, alpha=0.5, epi="f32")
    assert _rel(got, 0.5 * want + b) < 1e-4
    assert K.last_status() == 0


@pytest.mark.parametrize("M,F,act", [(8, 256, "geglu"), (64, 1536, "swiglu"), (100, 520, "situ"), (1, 128, "swiglu")])
def test_gemm_glu_epilogue(K, M, F, act):
    torch.manual_seed(F)
    x = torch.randn(M, 1024, device="cuda").bfloat16()
    w = (torch.randn(2 * F, 1024, device="cuda") * 0.04).bfloat16()
    h = x.float() @ w.float().T
    want = {"geglu": ref.geglu, "swiglu": ref.swiglu, "situ": ref.situ}[act](h[:, :F], h[:, F:])
    got = K.gemm(x, w, glu=act)
    assert _rel(got, want) < 1.5e-2
    assert K.last_status() == 0


def test_norm_family(K):
    torch.manual_seed(1)
    T, H = 37, 3840
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    assert _rel(K.rmsnorm(x, w, 1e-6), ref.rmsnorm(x.float(), w.float(), 1e-6)) < 1e-2
    assert _rel(K.rmsnorm(x.float(), None, 1e-6), ref.rmsnorm(x.float(), None, 1e-6)) < 1e-2
    res = torch.randn(T, H, device="cuda").bfloat16()
    y, r = K.add_rmsnorm(x, res.clone(), w, 1e-6)
    wy, wr = ref.add_rmsnorm(x, res.clone(), w, 1e-6)
    assert torch.equal(r, wr) and _rel(y, wy) < 1e-2
    h = torch.randn(T, H, device="cuda").bfloat16()
    w2 = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    for a in (x, x.float()):
        xo, hn = K.norm_add_norm(a, w, h.clone(), w2, 1e-6, 0.5)
        whn = ((h.float() + ref.rmsnorm(a.float(), w.float(), 1e-6)) * 0.5)
        assert _rel(hn, whn) < 1e-2 and _rel(xo, ref.rmsnorm(whn, w2.float(), 1e-6)) < 2e-2
    gu = torch.randn(T, 2 * 1024, device="cuda").bfloat16()
    for act in ("geglu", "swiglu", "situ"):
        F = 1024
        want = {"geglu": ref.geglu, "swiglu": ref.swiglu, "situ": ref.situ}[act](gu[:, :F].float(), gu[:, F:].float())
        assert _rel(K.glu(gu, act), want) < 1e-2
    tab = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (50,), device="cuda")
    assert _rel(K.embed(ids, tab, 16.0), tab[ids].float() * 16.0) < 1e-2


def _mk_cache(S_lens, q_lens, Hkv, D, dtype=torch.bfloat16):
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    pages = sum((l + 15) // 16 for l in S_lens) + 4
    cache = PagedKVCache(1, pages, 16, Hkv, D, dtype=dtype, device="cuda")
    # interleave allocation so that page lists are not contiguous
    for rnd in range(max((l + 15) // 16 for l in S_lens)):
        for s, l in enumerate(S_lens):
            if rnd * 16 < l:
                cache.alloc.extend(s, min(16, l - rnd * 16))
    table, lens = cache.alloc.page_table(list(range(len(S_lens))))
    return cache, BatchMeta.build(q_lens, lens, table, 16, "cuda")


@pytest.mark.parametrize("Hq,Hkv,D,window,softcap", [(16, 8, 256, 0, 0.0), (16, 8, 256, 64, 0.0), (32, 8, 128, 0, 30.0),
                                                      (4, 1, 64, 24, 0.0), (8, 8, 128, 0, 0.0)])
def test_paged_attention_decode_and_prefill(K, Hq, Hkv, D, window, softcap):
    torch.manual_seed(D + Hq)
    for S_lens, q_lens in (([300, 17, 129, 64], [1, 1, 1, 1]), ([40, 90, 33], [40, 7, 33]), ([200, 50], [3, 3])):
        cache, meta = _mk_cache(S_lens, q_lens, Hkv, D)
        cache.k[0].normal_()
        cache.v[0].normal_()
        q = torch.randn(sum(q_lens), Hq, D, device="cuda").bfloat16()
        want = ref.paged_attention(q, cache.k[0], cache.v[0], meta, D ** -0.5, window, softcap)
        for kernel in ("general", "decode"):
            if kernel == "decode" and Hq // Hkv > (4 if D == 256 else 8):
                continue
            for nsplit in (None, 1, 3):
                got = K.paged_attention(q, cache.k[0], cache.v[0], meta, D ** -0.5, window, softcap, nsplit=nsplit, kernel=kernel)
                assert _rel(got, want) < 2e-2, (kernel, S_lens, nsplit, _rel(got, want))


@pytest.mark.parametrize("M,N,K_,sk", [(48, 2112, 7168, 8), (3, 520, 4096, 5), (384, 384, 7168, 16), (130, 1000, 2048, 3), (32, 7168, 8192, 4),
                                       (48, 2112, 7168, 0), (48, 7168, 8192, 0), (3, 520, 4096, 0), (384, 384, 7168, 0), (48, 12288, 1536, 0),
                                       (300, 1000, 2048, 0)])
def test_gemm_split_k_finished_by_the_last_slice(K, M, N, K_, sk):
    """K slices as separate CTAs that add into an accumulator tile in scratch, the slice that arrives last stores the result:
    bf16 and f32 outputs, bias, both operand orders, repeated calls (accumulators and arrival counters must come back to zero).  ``sk = 0`` is
    stream-K: equal runs of K-blocks per CTA that cross tile boundaries."""
    torch.manual_seed(M + N)
    x = torch.randn(M, K_, device="cuda").bfloat16()
    w = (torch.randn(N, K_, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda")
    want = x.float() @ w.float().T
    for rep in range(3):
        for swap in (0, 1):
            g = K.gemm_splitk(x, w, sk, swap=swap)
            assert _rel(g, want) < 1e-2, (swap, _rel(g, want))
            g32 = K.gemm_splitk(x, w, sk, f32=True, bias=bias, swap=swap)
            assert _rel(g32, want + bias) < 2e-5 * np.sqrt(K_), (swap, _rel(g32, want + bias))
    torch.cuda.synchronize()
    ws, cnt = K._sk_workspace(x.device)
    assert int(cnt.abs().sum()) == 0 and float(ws.abs().max()) == 0.0     # scratch is handed back zeroed
    assert K.last_status() == 0


@pytest.mark.parametrize("Hq,Hkv,DK,DV,window", [(4, 2, 64, 64, 0), (8, 2, 128, 128, 0), (4, 4, 128, 128, 96), (4, 2, 256, 256, 0),
                                                  (4, 2, 256, 256, 200), (6, 6, 192, 128, 0)])
def test_tensor_core_prefill_attention_matches_reference(K, Hq, Hkv, DK, DV, window):
    """128-token query tiles on tcgen05: ragged batches, prior context in the cache, tiles that end inside a sequence,
    sliding windows that skip whole key blocks, separate K / V widths."""
    torch.manual_seed(DK + Hq)
    for S_lens, q_lens in (([300, 130, 517], [300, 130, 517]), ([700, 64, 257], [190, 64, 129]), ([1500], [1500])):
        from mary_b200.runtime.batch import BatchMeta
        from mary_b200.runtime.kv_cache import PagedKVCache
        pages = sum((n + 15) // 16 for n in S_lens) + 1
        kc = torch.randn(pages, 16, Hkv, DK, device="cuda").bfloat16()
        vc = torch.randn(pages, 16, Hkv, DV, device="cuda").bfloat16()
        alloc = PagedKVCache(1, pages, 16, 1, 8, dtype=torch.bfloat16, device="cuda").alloc
        for i, n in enumerate(S_lens):
            alloc.extend(i, n)
        table, lens = alloc.page_table(list(range(len(S_lens))))
        meta = BatchMeta.build(q_lens, lens, table, 16, "cuda")
        q = torch.randn(sum(q_lens), Hq, DK, device="cuda").bfloat16()
        scale = DK ** -0.5
        want = ref.paged_attention(q, kc, vc, meta, scale, window, 0.0)
        got = K.paged_attention(q, kc, vc, meta, scale, window, kernel="prefill")     # regrouped into 64-token pages: one TMA per stage
        torch.cuda.synchronize()
        assert K.last_status() == 0
        assert got.shape == want.shape
        assert _rel(got, want) < 2e-2, (S_lens, q_lens, _rel(got, want))
        import dataclasses
        direct = dataclasses.replace(meta, kv_lens_host=None)                           # no host lengths: the 16-token pages are read in place
        got16 = K.paged_attention(q, kc, vc, direct, scale, window, kernel="prefill")
        torch.cuda.synchronize()
        assert K.last_status() == 0 and _rel(got16, want) < 2e-2, (S_lens, q_lens, _rel(got16, want))


def test_qk_norm_rope_append_matches_reference(K):
    from mary_b200 import ops
    torch.manual_seed(3)
    n_q, n_kv, D = 4, 2, 64
    cache, meta = _mk_cache([50, 20], [50, 20], n_kv, D)
    cpu_cache, cpu_meta = cache, meta
    qkv = torch.randn(70, (n_q + 2 * n_kv) * D, device="cuda").bfloat16()
    qn = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    kn = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    inv = ref.rope_inv_freq(D, 1e4, 1.0, "cuda")
    q = K.qk_norm_rope_append(qkv, n_q, n_kv, D, qn, kn, True, inv, meta, cache.k[0], cache.v[0], 1e-6)
    kc, vc = torch.zeros_like(cache.k[0]), torch.zeros_like(cache.v[0])
    T = 70
    qq, kk, vv = qkv.float().split([n_q * D, n_kv * D, n_kv * D], -1)
    wq = ref.rope(ref.rmsnorm(qq.reshape(T, n_q, D), qn.float(), 1e-6), meta.positions, inv)
    wk = ref.rope(ref.rmsnorm(kk.reshape(T, n_kv, D), kn.float(), 1e-6), meta.positions, inv)
    wv = ref.rmsnorm(vv.reshape(T, n_kv, D), None, 1e-6)
    assert _rel(q, wq) < 2e-2
    flat_k = cache.k[0].view(-1, n_kv, D)[meta.slot_mapping]
    flat_v = cache.v[0].view(-1, n_kv, D)[meta.slot_mapping]
    assert _rel(flat_k, wk) < 2e-2 and _rel(flat_v, wv) < 2e-2


def test_argmax_first_max_and_gumbel(K):
    torch.manual_seed(5)
    lg = torch.randn(9, 262144, device="cuda")
    lg[0, 100] = 50.0
    lg[0, 70000] = 50.0                                  # tie: the lower index must win
    ids, val = K.argmax(lg, softcap=30.0)
    assert ids.tolist() == ref.argmax_first(lg).tolist() and ids[0].item() == 100
    assert torch.allclose(val, 30 * torch.tanh(lg.max(-1).values / 30), atol=1e-4)
    # sampling: the empirical distribution over a 4-way logit set follows softmax(l / T)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device="cuda").repeat(4096, 1).contiguous()
    cnt = torch.zeros(4)
    for step in range(4):
        s, _ = K.argmax(small, temperature=1.0, seed=7, step=step)
        cnt += torch.bincount(s.cpu(), minlength=4).float()
    p = cnt / cnt.sum()
    assert (p - torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0)).abs().max() < 0.02
    s1, _ = K.argmax(small, temperature=1.0, seed=7, step=0)
    s2, _ = K.argmax(small, temperature=1.0, seed=7, step=0)
    assert torch.equal(s1, s2)                           # seeded: reproducible


@pytest.mark.parametrize("E,k", [(128, 8), (384, 8), (256, 6), (8, 2)])
def test_router_topk_softmax_and_sigmoid_grouped(K, E, k):
    torch.manual_seed(E)
    T = 77
    lg = torch.randn(T, E, device="cuda")
    lg[3, 5] = lg[3, 2] = 4.0                            # tie
    idx, w = K.router_topk(lg, k, "softmax")
    ri, rw = ref.router_softmax_topk(lg, k)
    assert torch.equal(idx, ri) and torch.allclose(w, rw, rtol=1e-4, atol=1e-6)
    bias = torch.randn(E, device="cuda") * 0.1
    idx, w = K.router_topk(lg, k, "sigmoid", bias=bias, scale=2.5)
    ri, rw = ref.router_sigmoid_topk(lg, bias, k, scale=2.5)
    assert torch.equal(idx, ri) and torch.allclose(w, rw, rtol=1e-4, atol=1e-6)
    if E % 8 == 0 and E >= 64:
        idx, w = K.router_topk(lg, k, "sigmoid", bias=bias, n_group=8, topk_group=4, scale=2.5)
        ri, rw = ref.router_sigmoid_topk(lg, bias, k, n_group=8, topk_group=4, scale=2.5)
        assert torch.equal(idx, ri) and torch.allclose(w, rw, rtol=1e-4, atol=1e-6)


def test_short_conv(K):
    torch.manual_seed(9)
    x = torch.randn(19, 512, device="cuda").bfloat16()
    w = torch.randn(512, 4, device="cuda") * 0.3
    hist = torch.randn(3, 512, device="cuda").bfloat16()
    y, h = K.short_conv(x, w, hist)
    wy, wh = ref.short_conv(x, w, hist)
    assert _rel(y, wy) < 1e-2 and torch.equal(h, wh)


@pytest.mark.parametrize("Hq", [64, 8, 16])
def test_mla_latent_attention_tensor_core(K, Hq):
    """tcgen05 MLA kernel against the fp32 reference: decode with speculative rows, chunked prefill, kv splits; 16-token pages
    (one TMA operation per page and chunk) and 32-token pages (one 4-D TMA operation per 32-key stage)."""
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    torch.manual_seed(Hq)
    for ps in (16, 32):
        for S_lens, q_lens in (([300, 17, 1000, 64], [3, 1, 3, 2]), ([40, 90], [40, 7]), ([4096 + 3], [3])):
            pages = sum((l + ps - 1) // ps for l in S_lens) + 3
            cache = PagedKVCache(1, pages, ps, 1, 1, dtype=torch.bfloat16, device="cuda", latent_dim=576)
            for rnd in range(max((l + ps - 1) // ps for l in S_lens)):
                for s, l in enumerate(S_lens):
                    if rnd * ps < l:
                        cache.alloc.extend(s, min(ps, l - rnd * ps))
            table, lens = cache.alloc.page_table(list(range(len(S_lens))))
            meta = BatchMeta.build(q_lens, lens, table, ps, "cuda")
            cache.k[0].normal_()
            q = (torch.randn(sum(q_lens), Hq, 576, device="cuda") * 0.5).bfloat16()
            want = ref.paged_attention(q, cache.k[0], cache.k[0], meta, 576 ** -0.5, dv=512)
            for nsplit in (1, None, 3):
                got = K.mla_attention(q, cache.k[0], meta, 576 ** -0.5, nsplit=nsplit)
                assert K.last_status() == 0
                assert _rel(got, want) < 2e-2, (ps, S_lens, nsplit, _rel(got, want))


def test_codec_cuda_arm_matches_cpu_oracle(K):
    """Streaming codec on the GPU (im2col + tensor-core GEMM convolutions, overlap-add transposed convolutions, GEMM + arg-max
    codebook search, paged sliding-window attention) against the f32 CPU arm: decoded samples, code agreement, streaming."""
    from mary_b200.models.codec import MimiCodec, MimiConfig, init_random_
    from mary_b200.models.codec.mimi_cuda import MimiCuda
    c = MimiConfig(hidden=128, n_filters=16, ratios=(4, 2), kernel=7, tr_layers=2, tr_heads=2, tr_ffn=256, tr_window=12,
                   code_dim=64, codebook_size=128, num_codebooks=4)
    m = MimiCodec(c)
    init_random_(m, 0)
    g = MimiCuda(m, "cuda", max_frames=64)
    spf = c.samples_per_frame
    torch.manual_seed(0)
    codes = torch.randint(0, c.codebook_size, (10, c.num_codebooks))
    with torch.no_grad():
        want = m.decode(codes)
    got = g.decode(codes)
    assert got.shape == want.shape
    assert _rel(got.cpu(), want) < 3e-2, _rel(got.cpu(), want)
    st, parts = None, []
    for a, b in ((0, 3), (3, 4), (4, 10)):
        w, st = g.decode_step(codes[a:b], st)
        parts.append(w)
    assert _rel(torch.cat(parts), got) < 1e-3                  # streaming equals offline on the same arithmetic
    pcm = torch.randn(spf * 10) * 0.5
    with torch.no_grad():
        cw = m.encode(pcm)
    cg = g.encode(pcm.cuda()).cpu()
    assert cg.shape == cw.shape and int(cg.max()) < c.codebook_size
    assert (cg[:, 0] == cw[:, 0]).float().mean() > 0.7         # bf16 operands may flip near-ties, most codes agree
    st, parts = None, []
    for a, b in ((0, 2), (2, 7), (7, 10)):
        cs, st = g.encode_step(pcm[a * spf:b * spf].cuda(), st)
        parts.append(cs)
    assert (torch.cat(parts).cpu() == cg).float().mean() > 0.95
    assert K.last_status() == 0


@pytest.mark.gpu
def test_out_of_range_token_ids_and_cache_slots_are_recorded_and_never_dereferenced():
    """Data-dependent indices are checked where they enter a kernel: a token id outside the table reads row 0 and a cache slot
    outside the cache is not written; both leave MARY_ERR_BOUNDS (6) in the status word and the context stays usable."""
    from mary_b200.ops import cuda as K
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    K.last_status()
    table = torch.randn(50, 64, device="cuda").bfloat16()
    out = K.embed(torch.tensor([3, 49, 50, -1], dtype=torch.int32, device="cuda"), table)
    assert K.last_status() == 6
    assert torch.equal(out[0], table[3]) and torch.equal(out[1], table[49]) and torch.equal(out[2], table[0]) and torch.equal(out[3], table[0])
    K.embed(torch.tensor([0, 49], dtype=torch.int32, device="cuda"), table)
    assert K.last_status() == 0

    cache = PagedKVCache(1, 2, 16, 1, 64, dtype=torch.bfloat16, device="cuda")
    cache.alloc.extend(0, 3)
    table_, lens = cache.alloc.page_table([0])
    meta = BatchMeta.build([3], lens, table_, 16, device="cuda")
    qkv = torch.randn(3, 3 * 64, device="cuda").bfloat16()
    inv = torch.zeros(32, device="cuda")
    K.qk_norm_rope_append(qkv, 1, 1, 64, None, None, False, inv, meta, cache.k[0], cache.v[0], 1e-6)
    assert K.last_status() == 0
    before = cache.k[0].clone()
    meta.slot_mapping[1] = 2 * 16                                # one past the last slot of a 2-page cache
    K.qk_norm_rope_append(qkv, 1, 1, 64, None, None, False, inv, meta, cache.k[0], cache.v[0], 1e-6)
    assert K.last_status() == 6
    assert torch.equal(cache.k[0], before)                       # rows 0 and 2 rewritten with the same values, row 1 skipped
    lat = PagedKVCache(1, 2, 16, 1, 576, dtype=torch.bfloat16, device="cuda", latent_dim=576)
    qakv = torch.randn(3, 128 + 576, device="cuda").bfloat16()
    w1, w2 = torch.ones(128, device="cuda").bfloat16(), torch.ones(512, device="cuda").bfloat16()
    meta.slot_mapping[1] = -5
    K.mla_prep(qakv, 128, w1, w2, torch.zeros(32, device="cuda"), meta, lat.k[0], 1e-6)
    assert K.last_status() == 6 and float(lat.k[0].view(-1, 576)[1].abs().sum()) == 0.0
    assert (torch.ones(4, device="cuda") * 2).sum().item() == 8


@pytest.mark.gpu
def test_stream_probes_copy_exactly_and_reject_misaligned_buffers():
    from mary_b200.ops.cuda import _p, _stream, declare, lib
    declare("mary_stream_read", "plps")
    declare("mary_stream_copy", "ppls")
    src = torch.empty(1 << 22, dtype=torch.uint8, device="cuda").random_()
    dst = torch.zeros_like(src)
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib().mary_stream_copy(_p(src), _p(dst), src.numel(), _stream()) == 0
    assert lib().mary_stream_read(_p(src), src.numel(), _p(sink), _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(src, dst)
    assert lib().mary_stream_copy(_p(src[1:]), _p(dst), 1024, _stream()) == 4            # MARY_ERR_BAD_ARG: not 16-byte aligned


@pytest.mark.gpu
def test_programmatic_dependent_launch_with_early_weight_requests_changes_no_bit():
    """A chain of GEMMs, norms and a GEMM over freshly written operands, eager and as a replayed CUDA graph with changing inputs:
    with MARY_PDL=1 (kernels start while their predecessor drains; weight tiles are requested before the wait) every result
    equals the serialised run bit for bit."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    digests = {}
    for M in (48, 300):
        for pdl in ("0", "1"):
            env = dict(os.environ, MARY_PDL=pdl, PYTHONPATH=os.path.dirname(here))
            r = subprocess.run([sys.executable, os.path.join(here, "pdl_worker.py"), str(M)], env=env, capture_output=True, text=True, timeout=300)
            assert r.returncode == 0, r.stderr[-2000:]
            line = [ln for ln in r.stdout.splitlines() if ln.startswith("DIGEST")][0].split()
            assert line[3] == pdl
            digests[(M, pdl)] = line[1]
        assert digests[(M, "0")] == digests[(M, "1")]


@pytest.mark.gpu
@pytest.mark.parametrize("D,Hq,Hkv,page", [(128, 8, 2, 16), (128, 32, 8, 32), (128, 16, 2, 16), (256, 16, 8, 16), (256, 8, 4, 32), (128, 4, 4, 32)])
def test_tensor_core_gqa_decode_attention_matches_the_f32_reference(K, D, Hq, Hkv, page):
    """(token, head-of-group) rows of one kv head as an M = 64 tcgen05 tile over K / V pages: ragged lengths, speculative rows,
    sliding window, soft-cap, forced and automatic kv splits, against the plain f32 operator."""
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    g = torch.Generator().manual_seed(D + Hq + page)
    lens = [1, 37, 700, 129, 2048 + 5]
    S = len(lens)
    pages = sum((n + page - 1) // page for n in lens) + 3
    cache = PagedKVCache(1, pages, page, Hkv, D, dtype=torch.bfloat16, device="cuda")
    for s, n in enumerate(lens):
        cache.alloc.extend(s, n)
    table, kv = cache.alloc.page_table(list(range(S)))
    fill = BatchMeta.build(list(lens), kv, table, page, "cuda")
    k = torch.randn(sum(lens), Hkv, D, generator=g).bfloat16()
    v = torch.randn(sum(lens), Hkv, D, generator=g).bfloat16()
    cache.k[0].view(-1, Hkv, D)[fill.slot_mapping] = k.cuda()
    cache.v[0].view(-1, Hkv, D)[fill.slot_mapping] = v.cuda()
    kc, vc = cache.k[0].float().cpu(), cache.v[0].float().cpu()
    G = Hq // Hkv
    for q_lens in ([1] * S, [1, 3, 3, 2, 3]):
        q_lens = [min(a, b) for a, b in zip(q_lens, lens)]
        if max(q_lens) * G > 64:
            continue
        m = BatchMeta.build(q_lens, kv, table, page, "cuda")
        mc = BatchMeta.build(q_lens, kv, table, page, "cpu")
        q = (torch.randn(sum(q_lens), Hq, D, generator=g) * 1.5).bfloat16()
        assert K.gqa_tc_supported(q.cuda(), cache.k[0], m)
        for window, softcap, nsplit in ((0, 0.0, 1), (0, 0.0, None), (0, 0.0, 5), (96, 0.0, None), (1024, 0.0, 3), (0, 30.0, None)):
            before = K.LAUNCHES
            got = K.paged_attention(q.cuda(), cache.k[0], cache.v[0], m, D ** -0.5, window, softcap, nsplit=nsplit, kernel="tc").float().cpu()
            assert K.LAUNCHES == before + 1 and K.last_status() == 0
            want = ref.paged_attention(q.float(), kc, vc, mc, D ** -0.5, window, softcap)
            assert torch.isfinite(got).all()
            assert (got - want).abs().max() < 0.03, (q_lens, window, softcap, nsplit, float((got - want).abs().max()))
    with pytest.raises(ValueError):
        m8 = BatchMeta.build([9] + [1] * (S - 1), [max(n, 9) for n in kv], table, page, "cuda")
        K.paged_attention(torch.zeros(9 + S - 1, Hq, D, dtype=torch.bfloat16, device="cuda"), cache.k[0], cache.v[0], m8, 1.0, kernel="tc")

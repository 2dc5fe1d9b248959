"""Property tests of the reference-faithful Inkling and K3 operators (perturb an input, assert which outputs may move)."""
import pytest
import torch

from mary_b200.models.inkling import ops as ink
from mary_b200.models.k3 import ops as k3
from mary_b200.ops import reference as ref


def _ink_params(H=64, Hq=4, Hkv=2, D=16, d_rel=4, ext=12):
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g) * 0.2  # noqa: E731
    return dict(wq=r(Hq * D, H), wk=r(Hkv * D, H), wv=r(Hkv * D, H), wo=r(H, Hq * D), wr=r(Hq * d_rel, H), rel_proj=r(d_rel, ext),
                q_norm=torch.ones(D), k_norm=torch.ones(D), k_conv=r(Hkv * D, 4), v_conv=r(Hkv * D, 4)), \
        dict(n_heads=Hq, n_kv_heads=Hkv, head_dim=D, d_rel=d_rel, window=6, log_alpha=0.3, log_n_floor=8.0)


def test_inkling_attention_cached_equals_full_and_window_reach():
    p, cfg = _ink_params()
    x = torch.randn(20, 64, generator=torch.Generator().manual_seed(1))
    for is_global in (True, False):
        full = ink.attention(x, p, cfg, is_global=is_global)
        cache = {}
        parts = [ink.attention(x[a:b], p, cfg, cache=cache, is_global=is_global) for a, b in ((0, 7), (7, 8), (8, 20))]
        assert torch.allclose(torch.cat(parts), full, atol=1e-5)
    base = ink.attention(x, p, cfg, is_global=False)
    x2 = x.clone()
    x2[3] += 1.0
    moved = (ink.attention(x2, p, cfg, is_global=False) - base).abs().amax(-1) > 1e-7
    # token 3 reaches keys 3..(3+3 conv taps) and those reach queries up to window-1 later; nothing before it moves
    assert not moved[:3].any() and moved[3] and not moved[3 + 3 + 6:].any()


def test_inkling_router_rules():
    lg = torch.tensor([[2.0, 2.0, -1.0, 0.5, 0.3, -0.2]])          # 4 routed + 2 shared
    idx, w, gam = ink.router(lg, torch.zeros(4), 2, 2, route_scale=1.5)
    assert idx.tolist() == [[0, 1]]                                  # tie -> lower index first
    assert torch.allclose(w.sum() + gam.sum(), torch.tensor(1.5))   # one softmax over chosen and shared
    idx2, _, _ = ink.router(lg, torch.tensor([0.0, 0.0, 5.0, 0.0]), 2, 2, 1.0)
    assert 2 in idx2.tolist()[0]                                     # bias steers selection ...
    _, w3, _ = ink.router(lg, torch.tensor([0.0, 0.0, 0.0, 0.0]), 2, 2, 1.0)
    _, w4, _ = ink.router(lg, torch.tensor([0.1, 0.1, 0.0, 0.0]), 2, 2, 1.0)
    assert torch.equal(w3, w4)                                       # ... but never the weights
    try:
        ink.router(torch.tensor([[float("nan")] * 6]), torch.zeros(4), 2, 2, 1.0)
        assert False
    except FloatingPointError:
        pass


def test_k3_rmsnorm_two_roundings_and_mla_cache():
    x = torch.randn(5, 64).bfloat16()
    g = (1 + 0.1 * torch.randn(64)).bfloat16()
    y = k3.rms_norm(x, g)
    one = (x.float() / torch.sqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()).bfloat16()
    assert y.dtype == torch.bfloat16 and (y.float() - one.float()).abs().max() < 0.05 and not torch.equal(y, one)
    H, nh = 64, 2
    gen = torch.Generator().manual_seed(2)
    r = lambda *s: torch.randn(*s, generator=gen) * 0.1  # noqa: E731
    p = dict(q_a=r(48, H), q_a_norm=torch.ones(48), q_b=r(nh * 192, 48), kv_a=r(512 + 64, H), kv_a_norm=torch.ones(512),
             kv_b=r(nh * 256, 512), g_proj=r(nh * 128, H), o_proj=r(H, nh * 128))
    xs = torch.randn(9, H, generator=gen)
    full = k3.mla_nope(xs, p, nh)
    cache = {}
    inc = torch.cat([k3.mla_nope(xs[:4], p, nh, cache), k3.mla_nope(xs[4:], p, nh, cache)])
    assert torch.allclose(inc, full, atol=1e-5)
    # positive control for NoPE: permuting EARLIER tokens (keys and values together) leaves the last row unchanged
    perm = torch.tensor([2, 0, 3, 1, 4, 5, 6, 7, 8])
    assert torch.allclose(k3.mla_nope(xs[perm], p, nh)[-1], full[-1], atol=1e-5)


def test_k3_kda_state_is_chunk_invariant_and_situ_bounds():
    gen = torch.Generator().manual_seed(3)
    T, dk, dv = 12, 8, 6
    q, k, v, g = (torch.randn(T, d, generator=gen) for d in (dk, dk, dv, dk))
    beta = torch.rand(T, generator=gen)
    A, dt = torch.randn(dk, generator=gen) * 0.1, torch.randn(dk, generator=gen) * 0.1
    o, S = k3.kda_recurrent(q, k, v, g, beta, A, dt)
    o1, S1 = k3.kda_recurrent(q[:5], k[:5], v[:5], g[:5], beta[:5], A, dt)
    o2, S2 = k3.kda_recurrent(q[5:], k[5:], v[5:], g[5:], beta[5:], A, dt, S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-6) and torch.allclose(S2, S, atol=1e-9)
    big = ref.situ(torch.tensor([100.0]), torch.tensor([1000.0]))
    assert abs(big.item() - 4.0 * 25.0) < 1e-3                       # both branches saturate: beta * linear_beta


def test_k3_latent_moe_and_attn_res():
    gen = torch.Generator().manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=gen) * 0.1  # noqa: E731
    H, Z, Fd, E = 32, 16, 24, 6
    p = dict(router=r(E, H), down_proj=r(Z, H), up_proj=r(H, Z), expert_norm=torch.ones(Z), w1=r(E, Fd, Z), w3=r(E, Fd, Z),
             w2=r(E, Z, Fd), shared_gate=r(Fd, H), shared_up=r(Fd, H), shared_down=r(H, Fd))
    x = torch.randn(7, H, generator=gen)
    y = k3.latent_moe(x, p, 2, 2.0)
    assert y.shape == (7, H) and torch.isfinite(y).all()
    x2 = x.clone()
    x2[2] += 0.5
    d = (k3.latent_moe(x2, p, 2, 2.0) - y).abs().amax(-1)
    assert d[2] > 0 and d[[0, 1, 3, 4, 5, 6]].max() == 0             # tokens are independent
    bank = torch.randn(3, 5, H, generator=gen)
    acc = torch.randn(5, H, generator=gen)
    mix = k3.attn_res_mix(bank, acc, torch.randn(H, generator=gen), None)
    lo = torch.minimum(bank.amin(0), acc)
    hi = torch.maximum(bank.amax(0), acc)
    assert ((mix >= lo - 1e-5) & (mix <= hi + 1e-5)).all()           # a convex combination per token


def test_inkling_layer_has_three_stateful_paths_and_mtp_heads_roll_back():
    from mary_b200.models.inkling import ops as ink
    torch.manual_seed(0)
    H, Hq, Hkv, D, F = 32, 4, 2, 8, 48
    cfg = dict(n_heads=Hq, n_kv_heads=Hkv, head_dim=D, d_rel=4, log_alpha=0.1, log_n_floor=4.0, window=6, eps=1e-6)

    def layer_params():
        r = lambda *s: torch.randn(*s) * 0.2  # noqa: E731
        return dict(wq=r(Hq * D, H), wk=r(Hkv * D, H), wv=r(Hkv * D, H), wo=r(H, Hq * D), wr=r(Hq * 4, H), rel_proj=r(4, 8),
                    q_norm=torch.ones(D), k_norm=torch.ones(D), k_conv=r(Hkv * D, 4), v_conv=r(Hkv * D, 4), attn_norm=torch.ones(H),
                    mlp_norm=torch.ones(H), attn_sconv=r(H, 4), mlp_sconv=r(H, 4), w_gate=r(F, H), w_up=r(F, H), w_down=r(H, F),
                    hidden_norm=torch.ones(H), embed_norm=torch.ones(H), input_proj=r(H, 2 * H))
    p = layer_params()
    x = torch.randn(9, H)
    full = ink.decoder_layer(x, p, cfg)
    cache = {}
    parts = [ink.decoder_layer(x[:4], p, cfg, cache)] + [ink.decoder_layer(x[t:t + 1], p, cfg, cache) for t in range(4, 9)]
    assert torch.allclose(torch.cat(parts), full, atol=1e-5)
    assert set(cache) == {"attn", "hist_attn", "hist_mlp"} and cache["attn"]["k"].shape[0] == 9
    # a cache that forgot one of the layer-level conv histories is wrong from the first decode step
    broken = {}
    ink.decoder_layer(x[:4], p, cfg, broken)
    broken.pop("hist_mlp")
    assert not torch.allclose(ink.decoder_layer(x[4:5], p, cfg, broken), full[4:5], atol=1e-4)
    # the four additive paths: zero conv taps leave x + attn + mlp
    p0 = dict(p, attn_sconv=torch.zeros(H, 4), mlp_sconv=torch.zeros(H, 4))
    h1 = x + ink.attention(ref.rmsnorm(x, p["attn_norm"], 1e-6), p0, cfg)
    want = h1 + ink.dense_mlp(ref.rmsnorm(h1, p["mlp_norm"], 1e-6), p["w_gate"], p["w_up"], p["w_down"])
    assert torch.allclose(ink.decoder_layer(x, p0, cfg), want, atol=1e-5)

    # MTP wrapper: both operand orders are reachable and differ; drafting leaves the heads' caches untouched
    emb = torch.randn(20, H)
    a = ink.mtp_input(x[:3], emb[:3], p, hidden_first=True)
    b = ink.mtp_input(x[:3], emb[:3], p, hidden_first=False)
    assert a.shape == (3, H) and not torch.allclose(a, b)
    swapped = dict(p, input_proj=torch.cat([p["input_proj"][:, H:], p["input_proj"][:, :H]], 1))
    assert torch.allclose(ink.mtp_input(x[:3], emb[:3], swapped, hidden_first=False), a, atol=1e-6)
    heads = [layer_params(), layer_params()]
    caches = [{}, {}]
    for hp, c in zip(heads, caches):
        ink.mtp_block(x[:5], emb[1:6], hp, cfg, c)
    before = [c["attn"]["k"].clone() for c in caches]
    unembed = lambda h: h.float() @ emb.t()  # noqa: E731
    toks, rows = ink.mtp_draft(heads, caches, x[5], emb, None, unembed, 7, cfg)
    assert len(toks) == 2 and rows[0].shape == (20,)
    assert all(torch.equal(c["attn"]["k"], b) for c, b in zip(caches, before))
    assert torch.allclose(ink.embed_in([3, 4], emb, torch.full((H,), 2.0)), 2.0 * ref.rmsnorm(emb[3:5], None, 1e-6))


def test_k3_config_partition_kda_shell_and_depth_mixing_layer():
    from mary_b200.models.k3 import ops as k3
    cfg = k3.K3Config(6, kda_layers=[1, 2, 4, 5], full_attn_layers=[3, 6], first_k_dense=1, snapshot_every=2, n_heads=2, kda_head_dim=8)
    assert [cfg.attn_kind(i) for i in range(6)] == ["kda", "kda", "mla", "kda", "kda", "mla"]       # one-based lists
    assert cfg.is_dense(0) and not cfg.is_dense(1) and [cfg.is_boundary(i) for i in range(5)] == [False, False, True, False, True]
    with pytest.raises(ValueError, match="missing \\[6\\]"):
        k3.K3Config(6, [1, 2, 4, 5], [3])
    with pytest.raises(ValueError, match="duplicated \\[3\\]"):
        k3.K3Config(6, [1, 2, 3, 4, 5], [3, 6])

    torch.manual_seed(0)
    H, nh, dk = 24, 2, 8
    r = lambda *s: torch.randn(*s) * 0.3  # noqa: E731
    p = dict(q_proj=r(nh * dk, H), k_proj=r(nh * dk, H), v_proj=r(nh * dk, H), q_conv=r(nh * dk, 4), k_conv=r(nh * dk, 4), v_conv=r(nh * dk, 4),
             f_a_proj=r(6, H), f_b_proj=r(nh * dk, 6), b_proj=r(nh, H), g_a_proj=r(6, H), g_b_proj=r(nh * dk, 6), A_log=r(nh), dt_bias=r(nh * dk),
             o_norm=torch.ones(dk), o_proj=r(H, nh * dk))
    x = torch.randn(10, H)
    full = k3.kda_attention(x, p, cfg)
    cache = {}
    parts = [k3.kda_attention(x[:3], p, cfg, cache)] + [k3.kda_attention(x[t:t + 1], p, cfg, cache) for t in range(3, 10)]
    assert torch.allclose(torch.cat(parts), full, atol=1e-5)                    # O(1) state + three conv histories carry everything
    assert len(cache["state"]) == nh and cache["state"][0].shape == (dk, dk) and cache["hist_q"].shape == (3, nh * dk)
    causal = k3.kda_attention(torch.cat([x[:5], torch.randn(5, H)]), p, cfg)
    assert torch.allclose(causal[:5], full[:5], atol=1e-6)

    # the layer's control flow against a hand-rolled copy, across a boundary
    lp = dict(input_layernorm=torch.ones(H), post_attention_layernorm=torch.ones(H), attn_res_q1=r(H), attn_res_q2=r(H))
    attn = lambda h: h * 0.5 + 1.0   # noqa: E731
    ffn = lambda h: h * -0.25        # noqa: E731
    mixer = k3.DepthMixer()
    h0 = torch.randn(4, H)
    out0 = k3.decoder_layer(h0, 0, cfg, mixer, attn, ffn, lp)                   # empty bank: an ordinary pre-norm residual layer
    a0 = attn(k3.rms_norm(h0, lp["input_layernorm"]))
    assert torch.allclose(out0, h0 + a0 + ffn(k3.rms_norm(h0 + a0, lp["post_attention_layernorm"])), atol=1e-6) and mixer.bank == []
    out1 = k3.decoder_layer(out0, 1, cfg, mixer, attn, ffn, lp)
    out2 = k3.decoder_layer(out1, 2, cfg, mixer, attn, ffn, lp)                 # boundary: the accumulator restarts from attn's output
    assert len(mixer.bank) == 1 and torch.equal(mixer.bank[0], out1)
    a2 = attn(k3.rms_norm(out1, lp["input_layernorm"]))                        # bank was empty before the push: mix = identity
    m2 = k3.attn_res_mix(out1[None], a2, lp["attn_res_q2"], None)
    assert torch.allclose(out2, a2 + ffn(k3.rms_norm(m2, lp["post_attention_layernorm"])), atol=1e-6)
    out3 = k3.decoder_layer(out2, 3, cfg, mixer, attn, ffn, lp)
    m3 = k3.attn_res_mix(out1[None], out2, lp["attn_res_q1"], None)             # now the first mixture reads the bank too
    a3 = attn(k3.rms_norm(m3, lp["input_layernorm"]))
    pre = out2 + a3
    assert torch.allclose(out3, pre + ffn(k3.rms_norm(k3.attn_res_mix(out1[None], pre, lp["attn_res_q2"], None), lp["post_attention_layernorm"])), atol=1e-6)


def test_inkling_hmlp_plan_is_derived_and_dmel_sums_codebooks():
    from mary_b200.models.inkling.towers import HMLP, dmel_embed, fold, plan_scales, stages
    sc = plan_scales(2, 40, 4, 3)                                   # the released geometry: widths 128, 320, 4800 follow from it
    assert sc[0] == (1, 1, 1, 3) and sc[-1][:3] == (2, 40, 40)
    st = stages(sc, 4096)
    assert [s["output_dim"] for s in st[:-1]] == [128, 320, 4800] and st[-1]["output_dim"] == 4096 and st[0]["input_dim"] == 75
    assert [s["norm"] for s in st] == [True, True, True, False] and [s["hw_fold"] for s in st] == [5, 2, 4, 1] and st[-1]["t_fold"] == 2
    assert [s["output_dim"] for s in stages(plan_scales(2, 40, 3, 3), 4096)] == [128, 1216, 4096]      # another depth, other widths
    total = 1
    for s in st:
        total *= s["t_fold"] * s["hw_fold"] ** 2
    assert total == 2 * 40 * 40
    other = plan_scales(1, 16, 2, 3)
    assert other[-1][:3] == (1, 16, 16) and [s["hw_fold"] for s in stages(other, 64)] == [4, 4]
    # fold order: folded axes outside the channel axis
    x = torch.arange(2 * 4 * 4 * 3, dtype=torch.float32).view(2, 4, 4, 3)
    f = fold(x, 2, 2)
    assert f.shape == (1, 2, 2, 24)
    assert f[0, 1, 0].view(2, 2, 2, 3)[1, 0, 1].tolist() == x[1, 2, 1].tolist()
    # a whole tower on random weights against the stage formula
    torch.manual_seed(0)
    h = HMLP(2, 4, 2, 3, text_hidden=16)
    for i, s in enumerate(h.stages):
        h.proj[i] = torch.randn(s["output_dim"], s["input_dim"]) * 0.1
        h.norm[i] = torch.ones(s["output_dim"]) if s["norm"] else None
    px = torch.randn(2, 8, 12, 3)
    out = h(px)
    assert out.shape == (1 * 2 * 3, 16)
    y = px
    for s, w, g in zip(h.stages, h.proj, h.norm):
        y = fold(y, s["t_fold"], s["hw_fold"]) @ w.T
        if s["norm"]:
            y = torch.nn.functional.gelu(y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-6))
    assert torch.allclose(out, y.reshape(-1, 16), atol=1e-5)
    table = torch.randn(3 * 4, 8)
    ids = torch.tensor([[0, 3, 1], [2, 2, 2]])
    e = dmel_embed(ids, table, torch.ones(8), levels=4)
    raw = table[0] + table[4 + 3] + table[8 + 1]
    assert torch.allclose(e[0], raw * torch.rsqrt(raw.pow(2).mean() + 1e-6), atol=1e-6)
    with pytest.raises(ValueError):
        dmel_embed(torch.tensor([[4, 0, 0]]), table, torch.ones(8), levels=4)


def test_inkling_paged_attention_matches_the_reference_operator():
    from mary_b200.models.inkling import ops as ink
    from mary_b200.models.inkling.paged import InklingPagedAttention
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    torch.manual_seed(0)
    H, Hq, Hkv, D = 32, 4, 2, 8
    cfg = dict(n_heads=Hq, n_kv_heads=Hkv, head_dim=D, d_rel=4, log_alpha=0.1, log_n_floor=4.0, window=6, eps=1e-6)
    r = lambda *s: torch.randn(*s) * 0.3  # noqa: E731
    p = dict(wq=r(Hq * D, H), wk=r(Hkv * D, H), wv=r(Hkv * D, H), wo=r(H, Hq * D), wr=r(Hq * 4, H), rel_proj=r(4, 8),
             q_norm=1 + 0.1 * r(D), k_norm=1 + 0.1 * r(D), k_conv=r(Hkv * D, 4), v_conv=r(Hkv * D, 4))
    x = torch.randn(21, H)
    for is_global in (True, False):
        want = ink.attention(x, p, cfg, is_global=is_global)
        cache = PagedKVCache(1, 4, 16, Hkv, D, dtype=torch.float32)
        att = InklingPagedAttention(p, cfg, is_global)
        outs, done = [], 0
        for n in (9, 1, 1, 7, 3):                                   # a prefill chunk, decode steps, another chunk
            cache.alloc.extend(0, n)
            table, lens = cache.alloc.page_table([0])
            outs.append(att(x[done:done + n], BatchMeta.build([n], lens, table, 16), cache.k[0], cache.v[0]))
            done += n
        assert torch.allclose(torch.cat(outs), want, atol=2e-5), (is_global, float((torch.cat(outs) - want).abs().max()))


def test_k3_gated_delta_rule_matches_the_flash_linear_attention_reference():
    """The recurrence against ``fla``'s own naive KDA implementation (the package the reference gates its port against): same
    per-dimension log-decay, same delta-rule update; L2 normalisation of q / k and the bounded gate are applied here first."""
    naive = pytest.importorskip("fla.ops.kda.naive")
    from mary_b200.models.k3 import ops as k3
    torch.manual_seed(0)
    T, dk, dv = 19, 8, 8
    q, k, v = torch.randn(T, dk), torch.randn(T, dk), torch.randn(T, dv)
    g, beta = torch.randn(T, dk), torch.rand(T)
    A_log, dt_bias = torch.tensor(0.3), torch.randn(dk) * 0.2
    S0 = torch.randn(dk, dv) * 0.1
    o, S = k3.kda_recurrent(q, k, v, g, beta, A_log, dt_bias, S0)
    a = -5.0 * torch.sigmoid(torch.exp(A_log) * (g + dt_bias))
    qn, kn = torch.nn.functional.normalize(q, dim=-1), torch.nn.functional.normalize(k, dim=-1)
    want_o, want_S = naive.naive_recurrent_kda(qn[None, :, None], kn[None, :, None], v[None, :, None], a[None, :, None], beta[None, :, None],
                                               scale=1.0, initial_state=S0[None, None], output_final_state=True)
    assert torch.allclose(o, want_o[0, :, 0], atol=1e-5) and torch.allclose(S.float(), want_S[0, 0], atol=1e-5)
    assert (a <= 0).all() and (a >= -5).all()


def test_inkling_paged_attention_batches_slots_independently():
    """Three sequences of different length in one flattened batch (prefill together, then batched decode steps): every sequence equals
    its own single-sequence run, i.e. neighbours in the batch do not contaminate each other's K / V convolution history or cache."""
    from mary_b200.models.inkling import ops as ink
    from mary_b200.models.inkling.paged import InklingPagedAttention
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    torch.manual_seed(1)
    H, Hq, Hkv, D = 32, 4, 2, 8
    cfg = dict(n_heads=Hq, n_kv_heads=Hkv, head_dim=D, d_rel=4, log_alpha=0.1, log_n_floor=4.0, window=6, eps=1e-6)
    r = lambda *s: torch.randn(*s) * 0.3  # noqa: E731
    p = dict(wq=r(Hq * D, H), wk=r(Hkv * D, H), wv=r(Hkv * D, H), wo=r(H, Hq * D), wr=r(Hq * 4, H), rel_proj=r(4, 8),
             q_norm=torch.ones(D), k_norm=torch.ones(D), k_conv=r(Hkv * D, 4), v_conv=r(Hkv * D, 4))
    lens, steps = [5, 9, 3], 4
    xs = [torch.randn(n + steps, H) for n in lens]
    want = [ink.attention(x, p, cfg, is_global=False) for x in xs]
    cache = PagedKVCache(1, 8, 16, Hkv, D, dtype=torch.float32)
    att = InklingPagedAttention(p, cfg, is_global=False)
    for s, n in enumerate(lens):
        cache.alloc.extend(s, n)
    table, kv = cache.alloc.page_table([0, 1, 2])
    out = att(torch.cat([x[:n] for x, n in zip(xs, lens)]), BatchMeta.build(lens, kv, table, 16), cache.k[0], cache.v[0])
    got = [[o] for o in out.split(lens)]
    for t in range(steps):
        for s in range(3):
            cache.alloc.extend(s, 1)
        table, kv = cache.alloc.page_table([0, 1, 2])
        o = att(torch.stack([x[n + t] for x, n in zip(xs, lens)]), BatchMeta.build([1, 1, 1], kv, table, 16), cache.k[0], cache.v[0])
        for s in range(3):
            got[s].append(o[s:s + 1])
    for s in range(3):
        assert torch.allclose(torch.cat(got[s]), want[s], atol=2e-5), s
    att.reset(1)
    assert set(att.hist) == {0, 2}

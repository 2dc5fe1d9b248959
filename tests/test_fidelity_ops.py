"""Property tests of the reference-faithful Inkling and K3 operators (perturb an input, assert which outputs may move)."""
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

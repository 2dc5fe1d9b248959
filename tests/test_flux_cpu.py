"""FLUX.2: modulation gating, joint attention of text and image tokens, the 4-axis rotary code (relative in every axis),
single-stream fusion, the shifted flow schedule, latent packing and the autoencoder's geometry, and the whole pipeline on tiny
random weights."""
import math

import pytest
import torch

from mary_b200.models.flux import (FlowMatchEuler, Flux2Config, Flux2Transformer, Flux2VAE, FluxPipeline, VAEConfig, empirical_mu,
                                  pack_latents, position_ids, unpack_latents)
from mary_b200.models.flux.transformer import rope_angles, rope_pairs


def _init(m, seed=0, std=0.2):
    g = torch.Generator().manual_seed(seed)
    for n, p in m.named_parameters():
        if p.dim() == 1:
            p.data.fill_(0.0 if "bias" in n else 1.0)
        else:
            p.data.normal_(0.0, std, generator=g)
    return m


def _inputs(c, h=3, w=4, n_text=5, seed=1):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(h * w, c.in_channels, generator=g), torch.randn(n_text, c.joint_dim, generator=g), position_ids(h, w),
            position_ids(n_text=n_text))


def test_rotary_code_is_relative_per_axis_and_rotates_pairs():
    ids = position_ids(2, 3)
    a = rope_angles(ids, (4, 4, 4, 4), 2000.0)
    assert a.shape == (6, 8) and torch.all(a[:, :2] == 0) and torch.all(a[:, 6:] == 0)        # t and l are 0 for image tokens
    assert math.isclose(float(a[4, 2]), 1.0) and math.isclose(float(a[4, 4]), 1.0)              # token (1, 1): first frequency is 1
    q, k = torch.randn(6, 2, 16), torch.randn(6, 2, 16)
    s0 = torch.einsum("shd,thd->hst", rope_pairs(q, a), rope_pairs(k, a))
    a2 = rope_angles(ids + torch.tensor([3, 5, 7, 11]), (4, 4, 4, 4), 2000.0)
    s1 = torch.einsum("shd,thd->hst", rope_pairs(q, a2), rope_pairs(k, a2))
    assert torch.allclose(s0, s1, atol=1e-4)                                                     # only differences of ids matter


@pytest.mark.parametrize("guidance", [False, True])
def test_transformer_conditioning_paths(guidance):
    c = Flux2Config.tiny(guidance)
    m = _init(Flux2Transformer(c))
    x, txt, iid, tid = _inputs(c)
    with torch.no_grad():
        v = m(x, txt, 0.7, iid, tid)
        assert v.shape == x.shape and torch.isfinite(v).all()
        assert not torch.allclose(m(x, txt, 0.2, iid, tid), v)                                   # time
        assert not torch.allclose(m(x, txt + 0.5, 0.7, iid, tid), v)                             # text reaches the image stream
        assert not torch.allclose(m(x, txt, 0.7, iid.flip(0), tid), v)                           # positions
        if guidance:
            assert not torch.allclose(m(x, txt, 0.7, iid, tid, guidance=torch.tensor([4.0])), v)
        # streaming the blocks gives the same result as resident blocks
        blocks = [("double", b) for b in m.double_blocks] + [("single", b) for b in m.single_blocks]
        assert torch.allclose(m(x, txt, 0.7, iid, tid, blocks=iter(blocks)), v)
        # zero shared modulation: all gates are 0, the blocks are the identity and the text cannot reach the output
        m.mod_img.zero_(), m.mod_txt.zero_(), m.mod_single.zero_()
        assert torch.allclose(m(x, txt, 0.7, iid, tid), m(x, txt + 3.0, 0.7, iid, tid))


def test_schedule_is_shifted_monotone_and_integrates_a_constant_field():
    mu = empirical_mu(1024, 28)
    s = FlowMatchEuler(28, 1024)
    assert s.sigmas.shape == (29,) and s.sigmas[0] == 1.0 and s.sigmas[-1] == 0.0 and (s.sigmas[1:] < s.sigmas[:-1]).all()
    u = 1.0 / 28
    assert math.isclose(float(s.sigmas[-2]), math.exp(mu) / (math.exp(mu) + (1 / u - 1)), rel_tol=1e-5)
    assert math.isclose(empirical_mu(4096, 10), 8.73809524e-05 * 4096 + 1.89833333, rel_tol=1e-6)      # the 10-step fit ...
    assert math.isclose(empirical_mu(4096, 200), 0.00016927 * 4096 + 0.45666666, rel_tol=1e-6)         # ... and the 200-step fit
    assert math.isclose(empirical_mu(5000, 4), 0.00016927 * 5000 + 0.45666666)                         # long sequences: one line
    x0 = torch.randn(5, 3)
    v = torch.randn(5, 3)
    x = x0
    for _ in range(28):
        assert 0.0 < s.t <= 1.0
        x = s.step(v, x)
    assert torch.allclose(x, x0 - v, atol=1e-5)                                                  # total dt = 0 - 1


def test_latent_packing_and_vae_geometry():
    z = torch.randn(8, 3, 5)
    assert torch.equal(unpack_latents(pack_latents(z), 3, 5), z)
    vae = _init(Flux2VAE(VAEConfig.tiny()), std=0.1)
    with torch.no_grad():
        img = torch.rand(1, 3, 16, 24) * 2 - 1
        lat = vae.encode(img)
        assert lat.shape == (1, 2, 8, 12) and vae.scale_factor == 2
        assert vae.decode(lat).shape == (1, 3, 16, 24)
        p = vae.patchify(lat)
        assert p.shape == (1, 8, 4, 6) and torch.equal(vae.unpatchify(p), lat)
        assert p[0, 3, 1, 2] == lat[0, 0, 3, 5] and p[0, 4, 0, 0] == lat[0, 1, 0, 0]            # channel-major, then (dy, dx)
        vae.bn_mean.normal_(), vae.bn_var.uniform_(0.5, 2.0)
        assert torch.allclose(vae.denormalize(vae.normalize(p)), p, atol=1e-5)


def test_pipeline_produces_a_deterministic_image():
    c = Flux2Config.tiny()
    vae = _init(Flux2VAE(VAEConfig.tiny()), 2, 0.1)
    c.in_channels = 4 * vae.c.latent_channels
    pipe = FluxPipeline(_init(Flux2Transformer(c), 1), vae)
    txt = torch.randn(5, c.joint_dim)
    a = pipe(txt, 18, 26, steps=3, seed=7)
    assert a.shape == (3, 16, 24) and a.min() >= 0 and a.max() <= 1                              # aligned down to whole packed positions
    assert torch.equal(a, pipe(txt, 18, 26, steps=3, seed=7))
    assert not torch.equal(a, pipe(txt, 18, 26, steps=3, seed=8))
    assert not torch.allclose(a, pipe(txt * 2, 18, 26, steps=3, seed=7))


def test_prompt_features_concatenate_intermediate_layers_of_the_text_decoder():
    from mary_b200.models.flux.pipeline import encode_prompt
    from mary_b200.models.mistral import MistralConfig, MistralModel, init_random_
    cfg = MistralConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1, head_dim=16,
                        vocab_size=50, qk_norm=True)
    m = MistralModel(cfg)
    init_random_(m, 0)
    f = encode_prompt(m, [1, 2, 3, 4, 5], (1, 2, 4))
    assert f.shape == (5, 96)
    assert not torch.allclose(f[:, :32], f[:, 32:64])
    # the last requested state, final-normed, is the model's own hidden output
    from mary_b200 import ops
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    cache = PagedKVCache(4, 2, 16, 1, 16, dtype=torch.float32)
    cache.alloc.extend(0, 5)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        want = m.hidden(torch.tensor([1, 2, 3, 4, 5], dtype=torch.int32), BatchMeta.build([5], lens, table, 16), cache)
    assert torch.allclose(ops.rmsnorm(f[:, 64:], m.norm, cfg.rms_norm_eps), want, atol=1e-5)

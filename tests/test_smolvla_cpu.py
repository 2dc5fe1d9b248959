"""SmolVLA: the flow time code, the backwards Euler sampler on fields with known solutions, expert layers reading the backbone's
cache (self-attention layers see prefix and suffix, cross-attention layers see only the re-projected prefix), visibility of the
prefix blocks, and the SGD overfit probe of the action expert."""
import math

import torch

from mary_b200.models.smolvla import SmolVLA, SmolVLAConfig, euler_sample, time_embedding
from mary_b200.models.smolvla.model import init_random_


def test_time_embedding_periods_are_geometric():
    e = time_embedding(torch.tensor([0.25]), 8, 4e-3, 4.0)[0]
    periods = [4e-3 * 1000 ** (i / 3) for i in range(4)]
    for i, p in enumerate(periods):
        assert math.isclose(e[i].item(), math.sin(2 * math.pi * 0.25 / p), abs_tol=1e-4)
        assert math.isclose(e[4 + i].item(), math.cos(2 * math.pi * 0.25 / p), abs_tol=1e-4)


def test_euler_sampler_integrates_from_one_to_zero():
    noise = torch.randn(2, 5, 3)
    c = torch.randn(5, 3)
    assert torch.allclose(euler_sample(lambda x, t: c.expand_as(x), noise, 10), noise - c, atol=1e-5)      # constant field: exact
    seen = []
    euler_sample(lambda x, t: (seen.append(float(t[0])), torch.zeros_like(x))[1], noise, 4)
    assert seen == [1.0, 0.75, 0.5, 0.25]
    # the rectified-flow field of a point target a: v = (x - a) / t carries any x at t = 1 to a at t = 0, exactly under Euler
    a = torch.randn(5, 3)
    out = euler_sample(lambda x, t: (x - a) / t[:, None, None], noise, 7)
    assert torch.allclose(out, a.expand_as(out), atol=1e-4)


def _model():
    torch.manual_seed(0)
    m = SmolVLA(SmolVLAConfig.tiny())
    init_random_(m, 0, std=0.2)
    return m


def test_prefix_blocks_and_expert_layers_see_what_they_should():
    m = _model()
    c = m.c
    img = torch.rand(3, 32, 32) * 2 - 1
    x, blocks = m.embed_prefix([img], [3, 4, 5], torch.randn(c.state_dim))
    assert x.shape == (4 + 3 + 1, c.vlm.width) and blocks.tolist() == [0] * 7 + [1]
    cache = m.prefix_cache(x, blocks)
    # images / language do not see the state token: changing the state leaves their keys unchanged in every layer
    x2, _ = m.embed_prefix([img], [3, 4, 5], torch.randn(c.state_dim))
    cache2 = m.prefix_cache(x2, blocks)
    for (k, v), (k2, v2) in zip(cache, cache2):
        assert torch.allclose(k[:7], k2[:7], atol=1e-6) and torch.allclose(v[:7], v2[:7], atol=1e-6)
    assert not torch.allclose(cache[1][0][7], cache2[1][0][7])
    noisy = torch.randn(c.chunk_size, c.action_dim)
    v1 = m.denoise(cache, noisy, torch.tensor(0.6))
    assert v1.shape == (c.chunk_size, c.action_dim)
    # the action tokens see each other: perturbing the last action changes the first token's velocity
    n2 = noisy.clone()
    n2[-1] += 1.0
    assert not torch.allclose(m.denoise(cache, n2, torch.tensor(0.6))[0], v1[0])
    # ... and see the prefix: another observation changes the velocity; another flow time does too
    assert not torch.allclose(m.denoise(cache2, noisy, torch.tensor(0.6)), v1)
    assert not torch.allclose(m.denoise(cache, noisy, torch.tensor(0.2)), v1)
    # odd layers read the backbone's K/V through their own kv_dim -> kv_dim projections
    kv = c.vlm.n_kv_heads * c.vlm.head_dim
    assert m.expert_layers[1].wk.shape == (kv, kv) and m.expert_layers[0].wk.shape == (kv, c.expert.width)
    act = m.act([img], [3, 4, 5], torch.randn(c.state_dim), generator=torch.Generator().manual_seed(1))
    assert act.shape == (c.chunk_size, c.expressive_dim) and torch.isfinite(act).all()


def test_sgd_overfit_probe_of_the_action_expert():
    m = _model()
    c = m.c
    img = torch.rand(3, 32, 32) * 2 - 1
    with torch.no_grad():
        cache = m.prefix_cache(*m.embed_prefix([img], [3, 4, 5], torch.randn(c.state_dim)))
    train = [p for n, p in m.named_parameters() if n.startswith(("expert_", "act_", "at_"))]
    for p in train:
        p.requires_grad_(True)
    actions = torch.randn(c.chunk_size, c.action_dim) * 0.5
    g = torch.Generator().manual_seed(3)
    pairs = [(torch.randn(c.chunk_size, c.action_dim, generator=g), float(torch.rand((), generator=g)) * 0.98 + 0.01) for _ in range(4)]
    opt = torch.optim.SGD(train, lr=0.05, momentum=0.9)
    first = last = None
    for step in range(150):
        loss = sum(m.flow_loss(cache, actions, n, t) for n, t in pairs) / len(pairs)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
    assert last < 0.2 * first, (first, last)


def test_vision_tower_and_pixel_shuffle_connector_match_the_huggingface_smolvlm_backbone():
    """The perception half of the policy is a SmolVLM backbone: same weights by name, image tokens compared (the order in which the
    pixel shuffle folds neighbouring patches into channels is invisible to any shape check)."""
    import pytest
    transformers = pytest.importorskip("transformers")
    from transformers.models.smolvlm import SmolVLMConfig, SmolVLMModel
    c = SmolVLAConfig.tiny()
    torch.manual_seed(0)
    hc = SmolVLMConfig(
        vision_config=dict(hidden_size=c.v_hidden, intermediate_size=c.v_ffn, num_hidden_layers=c.v_layers, num_attention_heads=c.v_heads,
                           image_size=c.image_size, patch_size=c.patch, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6),
        text_config=dict(hidden_size=c.vlm.width, intermediate_size=c.vlm.ffn_dim, num_hidden_layers=1, num_attention_heads=c.vlm.n_heads,
                         num_key_value_heads=c.vlm.n_kv_heads, head_dim=c.vlm.head_dim, vocab_size=c.vocab, pad_token_id=0),
        scale_factor=c.shuffle, image_token_id=c.vocab - 1, pad_token_id=0)
    hc._attn_implementation = "eager"
    hc.vision_config._attn_implementation = "eager"
    hf = SmolVLMModel(hc).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = SmolVLA(c)
    init_random_(m, 0)
    with torch.no_grad():
        v = "vision_model."
        m.patch_w.copy_(sd[v + "embeddings.patch_embedding.weight"]), m.patch_b.copy_(sd[v + "embeddings.patch_embedding.bias"])
        m.v_pos.copy_(sd[v + "embeddings.position_embedding.weight"])
        m.v_post_w.copy_(sd[v + "post_layernorm.weight"]), m.v_post_b.copy_(sd[v + "post_layernorm.bias"])
        m.connector.copy_(sd["connector.modality_projection.proj.weight"])
        for i, b in enumerate(m.v_blocks):
            p = f"{v}encoder.layers.{i}."
            b.w_qkv.copy_(torch.cat([sd[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0))
            b.b_qkv.copy_(torch.cat([sd[p + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0))
            b.w_o.copy_(sd[p + "self_attn.out_proj.weight"]), b.b_o.copy_(sd[p + "self_attn.out_proj.bias"])
            b.ln1_w.copy_(sd[p + "layer_norm1.weight"]), b.ln1_b.copy_(sd[p + "layer_norm1.bias"])
            b.ln2_w.copy_(sd[p + "layer_norm2.weight"]), b.ln2_b.copy_(sd[p + "layer_norm2.bias"])
            b.w_fc1.copy_(sd[p + "mlp.fc1.weight"]), b.b_fc1.copy_(sd[p + "mlp.fc1.bias"])
            b.w_fc2.copy_(sd[p + "mlp.fc2.weight"]), b.b_fc2.copy_(sd[p + "mlp.fc2.bias"])
    img = torch.rand(3, c.image_size, c.image_size) * 2 - 1
    with torch.no_grad():
        out = hf.get_image_features(pixel_values=img[None, None])
        want = out.pooler_output if hasattr(out, "pooler_output") else out
        want = want.reshape(-1, c.vlm.width) * math.sqrt(c.vlm.width)
        got = m.image_tokens(img)
    assert got.shape == want.shape == ((c.image_size // c.patch // c.shuffle) ** 2, c.vlm.width)
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())


def test_policy_loaded_by_released_names_reproduces_the_backbone_and_fills_every_parameter():
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.smolvlm import SmolVLMConfig, SmolVLMModel
    from mary_b200.models.smolvla import load_into
    c = SmolVLAConfig.tiny()
    torch.manual_seed(2)
    hc = SmolVLMConfig(
        vision_config=dict(hidden_size=c.v_hidden, intermediate_size=c.v_ffn, num_hidden_layers=c.v_layers, num_attention_heads=c.v_heads,
                           image_size=c.image_size, patch_size=c.patch, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6),
        text_config=dict(hidden_size=c.vlm.width, intermediate_size=c.vlm.ffn_dim, num_hidden_layers=c.vlm.n_layers,
                         num_attention_heads=c.vlm.n_heads, num_key_value_heads=c.vlm.n_kv_heads, head_dim=c.vlm.head_dim, vocab_size=c.vocab,
                         pad_token_id=0),
        scale_factor=c.shuffle, image_token_id=c.vocab - 1, pad_token_id=0)
    hc._attn_implementation = "eager"
    hc.vision_config._attn_implementation = "eager"
    hf = SmolVLMModel(hc).eval()
    sd = {"model.vlm_with_expert.vlm.model." + k: v.detach() for k, v in hf.state_dict().items()}
    e, kv = c.expert, c.vlm.n_kv_heads * c.vlm.head_dim
    g = torch.Generator().manual_seed(0)
    for i in range(e.n_layers):
        p = f"model.vlm_with_expert.lm_expert.layers.{i}."
        kin = e.width if i % c.self_attn_every == 0 else kv
        for n, s in (("input_layernorm", (e.width,)), ("post_attention_layernorm", (e.width,)), ("self_attn.q_proj", (e.n_heads * e.head_dim, e.width)),
                     ("self_attn.k_proj", (e.n_kv_heads * e.head_dim, kin)), ("self_attn.v_proj", (e.n_kv_heads * e.head_dim, kin)),
                     ("self_attn.o_proj", (e.width, e.n_heads * e.head_dim)), ("mlp.gate_proj", (e.ffn_dim, e.width)),
                     ("mlp.up_proj", (e.ffn_dim, e.width)), ("mlp.down_proj", (e.width, e.ffn_dim))):
            sd[p + n + ".weight"] = torch.randn(s, generator=g) * 0.1
    sd["model.vlm_with_expert.lm_expert.norm.weight"] = torch.ones(e.width)
    for n, (o, i) in {"state_proj": (c.vlm.width, c.state_dim), "action_in_proj": (e.width, c.action_dim), "action_out_proj": (c.action_dim, e.width),
                      "action_time_mlp_in": (e.width, 2 * e.width), "action_time_mlp_out": (e.width, e.width)}.items():
        sd[f"model.{n}.weight"], sd[f"model.{n}.bias"] = torch.randn(o, i, generator=g) * 0.1, torch.randn(o, generator=g) * 0.1
    used = set()

    class L:
        def load_tensor(self, n, dtype):
            used.add(n)
            return sd[n].to(dtype)
    m = SmolVLA(c)
    for p in m.parameters():
        p.data.fill_(float("nan"))
    load_into(m, L())
    assert all(torch.isfinite(p).all() for p in m.parameters())                         # nothing left unfilled
    unused = set(sd) - used
    assert all("text_model.norm" in n or "lm_head" in n for n in unused), sorted(unused)[:5]   # the policy reads K / V, never the final norm
    img = torch.rand(3, c.image_size, c.image_size) * 2 - 1
    with torch.no_grad():
        out = hf.get_image_features(pixel_values=img[None, None])
        want = (out.pooler_output if hasattr(out, "pooler_output") else out).reshape(-1, c.vlm.width) * math.sqrt(c.vlm.width)
        assert torch.allclose(m.image_tokens(img), want, atol=2e-4)
        chunk = m.act([img], [3, 4, 5], torch.randn(c.state_dim), generator=torch.Generator().manual_seed(0))
    assert chunk.shape[0] == c.chunk_size and torch.isfinite(chunk).all()
    assert torch.equal(m.vlm_layers[1].w_gu[:c.vlm.ffn_dim], sd["model.vlm_with_expert.vlm.model.text_model.layers.1.mlp.gate_proj.weight"])

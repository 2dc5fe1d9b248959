"""CLIP embedder against the Hugging Face implementation of the same architecture (random tiny weights loaded by name)."""
import pytest
import torch

from mary_b200.models.embed import ClipConfig, ClipEmbedder, load_into


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)


def test_clip_embeddings_match_huggingface():
    transformers = pytest.importorskip("transformers")
    c = ClipConfig.tiny()
    torch.manual_seed(0)
    hf_cfg = transformers.CLIPConfig(
        text_config=dict(vocab_size=c.t_vocab, hidden_size=c.t_hidden, intermediate_size=c.t_ffn, num_hidden_layers=c.t_layers,
                         num_attention_heads=c.t_heads, max_position_embeddings=c.t_ctx, hidden_act="quick_gelu", eos_token_id=c.t_vocab - 1,
                         projection_dim=c.dim),
        vision_config=dict(hidden_size=c.v_hidden, intermediate_size=c.v_ffn, num_hidden_layers=c.v_layers, num_attention_heads=c.v_heads,
                           image_size=c.image_size, patch_size=c.patch, hidden_act="quick_gelu", projection_dim=c.dim),
        projection_dim=c.dim)
    hf = transformers.CLIPModel(hf_cfg).eval()
    m = ClipEmbedder(c)
    load_into(m, _DictLoader({k: v.detach() for k, v in hf.state_dict().items()}))
    pixels = torch.randn(3, 3, c.image_size, c.image_size)
    ids = torch.randint(0, c.t_vocab - 1, (2, 9))
    ids[0, 6] = c.t_vocab - 1                       # end of text inside the padded row
    ids[1, 8] = c.t_vocab - 1
    with torch.no_grad():
        want_i = torch.nn.functional.normalize(hf.get_image_features(pixel_values=pixels).pooler_output
                                               if hasattr(hf.get_image_features(pixel_values=pixels), "pooler_output")
                                               else hf.get_image_features(pixel_values=pixels), dim=-1)
        tf = hf.get_text_features(input_ids=ids)
        want_t = torch.nn.functional.normalize(tf.pooler_output if hasattr(tf, "pooler_output") else tf, dim=-1)
        got_i, got_t = m.embed_image(pixels), m.embed_text(ids)
    assert torch.allclose(got_i, want_i, atol=2e-5), (got_i - want_i).abs().max()
    assert torch.allclose(got_t, want_t, atol=2e-5), (got_t - want_t).abs().max()
    assert torch.allclose(got_i.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert m.similarity(pixels, ids).shape == (3, 2)


def test_clip_preprocess_resizes_crops_and_normalises():
    m = ClipEmbedder(ClipConfig.tiny())
    img = torch.rand(3, 50, 80)
    out = m.preprocess(img)
    assert out.shape == (3, 32, 32)
    flat = torch.full((3, 40, 40), 0.5)
    out = m.preprocess(flat)
    for ch in range(3):
        assert torch.allclose(out[ch], torch.full((32, 32), (0.5 - m.MEAN[ch]) / m.STD[ch]), atol=1e-4)


def test_siglip_embeddings_match_huggingface():
    transformers = pytest.importorskip("transformers")
    from mary_b200.models.embed import SiglipConfig, SiglipEmbedder
    from mary_b200.models.embed import siglip
    c = SiglipConfig.tiny()
    torch.manual_seed(0)
    hf_cfg = transformers.SiglipConfig(
        text_config=dict(vocab_size=c.t_vocab, hidden_size=c.t_hidden, intermediate_size=c.t_ffn, num_hidden_layers=c.t_layers,
                         num_attention_heads=c.t_heads, max_position_embeddings=c.t_ctx, projection_size=c.t_hidden),
        vision_config=dict(hidden_size=c.v_hidden, intermediate_size=c.v_ffn, num_hidden_layers=c.v_layers, num_attention_heads=c.v_heads,
                           image_size=c.image_size, patch_size=c.patch))
    hf_cfg._attn_implementation = "eager"
    hf = transformers.SiglipModel(hf_cfg).eval()
    with torch.no_grad():
        hf.logit_scale.fill_(1.3)
        hf.logit_bias.fill_(-2.0)
    m = SiglipEmbedder(c)
    siglip.load_into(m, _DictLoader({k: v.detach() for k, v in hf.state_dict().items()}))
    pixels = torch.randn(3, 3, c.image_size, c.image_size)
    ids = torch.randint(0, c.t_vocab, (2, c.t_ctx))
    with torch.no_grad():
        out = hf(input_ids=ids, pixel_values=pixels)
        got_i, got_t = m.embed_image(pixels), m.embed_text(ids)
        prob = m.pair_probability(pixels, ids)
    assert torch.allclose(got_i, out.image_embeds, atol=2e-5), (got_i - out.image_embeds).abs().max()
    assert torch.allclose(got_t, out.text_embeds, atol=2e-5), (got_t - out.text_embeds).abs().max()
    assert torch.allclose(prob, torch.sigmoid(out.logits_per_image), atol=2e-5)
    assert m.preprocess(torch.full((3, 40, 70), 0.75)).allclose(torch.full((3, 32, 32), 0.5), atol=1e-5)


def test_nomic_text_embedder_matches_huggingface_and_ignores_padding():
    transformers = pytest.importorskip("transformers")
    from transformers.models.nomic_bert import NomicBertConfig, NomicBertModel
    from mary_b200.models.embed import NomicConfig, NomicTextEmbedder
    from mary_b200.models.embed import nomic
    c = NomicConfig.tiny()
    torch.manual_seed(0)
    hf_cfg = NomicBertConfig(vocab_size=c.vocab_size, hidden_size=c.hidden, num_hidden_layers=c.layers, num_attention_heads=c.heads,
                             intermediate_size=c.ffn, rope_parameters={"rope_type": "default", "rope_theta": c.rope_theta}, max_position_embeddings=64)
    hf_cfg._attn_implementation = "eager"
    hf = NomicBertModel(hf_cfg, add_pooling_layer=False).eval() if "add_pooling_layer" in NomicBertModel.__init__.__code__.co_varnames \
        else NomicBertModel(hf_cfg).eval()
    m = NomicTextEmbedder(c)
    nomic.load_into(m, _DictLoader({k: v.detach() for k, v in hf.state_dict().items()}))
    ids = torch.randint(1, c.vocab_size, (2, 11))
    mask = torch.ones(2, 11, dtype=torch.long)
    mask[1, 7:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got = m.hidden(ids, mask)
    assert torch.allclose(got[0], want[0], atol=3e-5), (got[0] - want[0]).abs().max()
    assert torch.allclose(got[1, :7], want[1, :7], atol=3e-5)
    with torch.no_grad():
        e = m.embed_text(ids, mask)
        alone = m.embed_text(ids[1:, :7])                     # padding must not change a sentence's vector
        short = m.embed_text(ids, mask, dim=16)
    assert torch.allclose(e[1], alone[0], atol=1e-5)
    assert short.shape == (2, 16) and torch.allclose(short.norm(dim=-1), torch.ones(2), atol=1e-5)


def _nomic_vision_plain(sd, c, pixels):
    """The nomic vision tower restated with torch.nn modules, complex-number rotation and explicit softmax: written from the
    architecture description, sharing no code with the embedder under test."""
    import math
    import torch.nn.functional as F
    H, nh, g = c.hidden, c.heads, c.grid
    hd = H // nh
    B = pixels.shape[0]
    # patches as a LINEAR map over (c, p1, p2)-ordered flattened patches
    pt = pixels.unfold(2, c.patch, c.patch).unfold(3, c.patch, c.patch)                 # [B, 3, g, g, p, p]
    pt = pt.permute(0, 2, 3, 1, 4, 5).reshape(B, g * g, 3 * c.patch * c.patch)
    x = pt @ sd["embeddings.proj.weight"].T + sd["embeddings.proj.bias"]
    x = torch.cat([sd["embeddings.cls_token"].expand(B, 1, H), x], 1) + sd["embeddings.pos_embed"]
    nb = hd // 4
    bands = torch.tensor([1.0 / 10000.0 ** (i / nb) for i in range(nb)], dtype=torch.float64)
    ang = torch.zeros(g * g, hd // 2, dtype=torch.float64)
    for r in range(g):
        for col in range(g):
            ang[r * g + col] = torch.cat([r * bands, col * bands])
    phase = torch.polar(torch.ones_like(ang), ang).to(torch.complex64)                 # one unit complex number per channel pair

    def rope(t):                                                                     # t [B, nh, T, hd]; class token untouched
        patches = torch.view_as_complex(t[:, :, 1:].reshape(B, nh, g * g, hd // 2, 2).contiguous()) * phase
        return torch.cat([t[:, :, :1], torch.view_as_real(patches).reshape(B, nh, g * g, hd)], 2)

    def lin(t, n):
        return t @ sd[n + ".weight"].T + sd[n + ".bias"]

    def lnorm(t, n, eps):
        return F.layer_norm(t, (t.shape[-1],), sd[n + ".weight"], sd[n + ".bias"], eps)
    res = None
    T = x.shape[1]
    for i in range(c.layers):
        p = f"layers.{i}."
        res = x if res is None else x + res
        qkv = lin(lnorm(res, p + "norm1", 1e-6), p + "attn.Wqkv")
        q, k, v = (qkv[..., j * H:(j + 1) * H].reshape(B, T, nh, hd).transpose(1, 2) for j in range(3))
        w = torch.softmax(rope(q) @ rope(k).transpose(-1, -2) / math.sqrt(hd), -1)
        res = lin((w @ v).transpose(1, 2).reshape(B, T, H), p + "attn.out_proj") + res
        h = lnorm(res, p + "norm2", 1e-6)
        x = lin(lnorm(lin(h, p + "mlp.fc11") * F.silu(lin(h, p + "mlp.fc12")), p + "mlp.norm", 1e-5), p + "mlp.fc2")
    hid = x + res
    q = lin(sd["selector.attn.latent"].expand(B, 1, H), "selector.attn.Wq").reshape(B, 1, nh, hd).transpose(1, 2)
    kv = lin(hid, "selector.attn.Wkv")
    k, v = (kv[..., j * H:(j + 1) * H].reshape(B, T, nh, hd).transpose(1, 2) for j in range(2))
    a = lin((torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(hd), -1) @ v).transpose(1, 2).reshape(B, H), "selector.attn.out_proj")
    n = lnorm(a, "selector.norm1", 1e-6)
    return a + lin(lin(n, "selector.mlp.fc11") * F.silu(lin(n, "selector.mlp.fc12")), "selector.mlp.fc2"), hid


def test_nomic_vision_embedder_against_a_plain_restatement_and_inventory():
    from mary_b200.models.embed import NomicVisionConfig, NomicVisionEmbedder
    from mary_b200.models.embed import nomic
    full = nomic.vision_tensor_shapes()
    assert len(full) == 2 + 2 + 12 * 16 + 1 + 6 + 2 + 6 and full["embeddings.pos_embed"] == (1, 197, 768)
    assert full["layers.11.mlp.norm.weight"] == (2048,) and "selector.mlp.norm.weight" not in full
    c = NomicVisionConfig.tiny()
    torch.manual_seed(3)
    sd = {n: torch.randn(s) * (0.3 if len(s) > 1 else 0.1) for n, s in nomic.vision_tensor_shapes(c).items()}
    for n in sd:
        if n.endswith("norm1.weight") or n.endswith("norm2.weight") or n.endswith("norm.weight"):
            sd[n] = 1 + sd[n]
    m = NomicVisionEmbedder(c)
    nomic.load_vision_into(m, _DictLoader(sd))
    pixels = torch.randn(2, 3, c.image_size, c.image_size)
    with torch.no_grad():
        want_pool, want_hid = _nomic_vision_plain(sd, c, pixels)
        got_hid = m.tokens(pixels)
        got = m.embed_image(pixels)
    assert torch.allclose(got_hid, want_hid, atol=2e-4, rtol=1e-4), (got_hid - want_hid).abs().max()
    want = torch.nn.functional.normalize(want_pool, dim=-1)
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()
    assert torch.allclose(got.norm(dim=-1), torch.ones(2), atol=1e-6)
    # class-token pooling is NOT the embedding
    assert not torch.allclose(torch.nn.functional.normalize(got_hid[:, 0], dim=-1), got, atol=1e-2)
    with pytest.raises(ValueError, match="image-only"):
        m.embed_text([[1, 2]])
    bad = dict(sd)
    bad["layers.0.mlp.norm.weight"] = torch.ones(c.ffn + 1)
    with pytest.raises(ValueError, match="architecture fixes"):
        nomic.load_vision_into(NomicVisionEmbedder(c), _DictLoader(bad))


def test_axial_rope_is_relative_in_both_axes_and_leaves_the_class_token():
    from mary_b200.models.embed.nomic import axial_rope_tables, rotate_pairs
    g, hd = 5, 16
    cos, sin = axial_rope_tables(g, hd)
    assert cos.shape == (g * g, hd) and torch.equal(cos[:, 0::2], cos[:, 1::2])
    assert torch.allclose(cos[0], torch.ones(hd)) and torch.allclose(sin[0], torch.zeros(hd))
    torch.manual_seed(0)
    q, k = torch.randn(hd), torch.randn(hd)

    def score(a, b):                     # token indices
        return (rotate_pairs(q, cos[a], sin[a]) * rotate_pairs(k, cos[b], sin[b])).sum()
    # the same (row, column) offset gives the same score wherever the pair sits
    assert torch.allclose(score(0 * g + 1, 2 * g + 3), score(1 * g + 2, 3 * g + 4), atol=1e-5)
    assert torch.allclose(score(2 * g + 0, 2 * g + 2), score(4 * g + 1, 4 * g + 3), atol=1e-5)
    assert not torch.allclose(score(0, 1), score(0, g), atol=1e-3)          # a column step is not a row step

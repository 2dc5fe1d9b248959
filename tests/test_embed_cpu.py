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

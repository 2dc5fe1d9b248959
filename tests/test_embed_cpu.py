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

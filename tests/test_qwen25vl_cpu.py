"""Qwen2.5-VL embedder against the Hugging Face implementation (random tiny weights loaded by name): the vision tower with
window and full-attention blocks on two images of different size, multimodal rotary positions, and the spliced decoder pass."""
import pytest
import torch

from mary_b200.models.qwen2_5_vl import BiQwenEmbedder, Qwen25VLConfig, load_into, mrope_positions


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)


def test_mrope_positions_follow_the_documented_example():
    # 2 text tokens, one image of grid (1, 4, 6) -> 2 x 3 merged tokens, 2 text tokens
    pos = mrope_positions([0, 0, 1, 1, 1, 1, 1, 1, 0, 0], [(1, 4, 6)], merge=2)
    assert pos[0].tolist() == [0, 1, 2, 2, 2, 2, 2, 2, 5, 6]
    assert pos[1].tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 5, 6]
    assert pos[2].tolist() == [0, 1, 2, 3, 4, 2, 3, 4, 5, 6]
    with pytest.raises(ValueError):
        mrope_positions([1, 1], [(1, 4, 6)])


def test_vision_tower_and_embedding_match_huggingface():
    transformers = pytest.importorskip("transformers")
    from transformers.models.qwen2_5_vl import Qwen2_5_VLConfig, Qwen2_5_VLModel
    c = Qwen25VLConfig.tiny()
    torch.manual_seed(0)
    hf_cfg = Qwen2_5_VLConfig(
        vision_config=dict(depth=c.v_depth, hidden_size=c.v_hidden, num_heads=c.v_heads, intermediate_size=c.v_ffn, patch_size=c.patch,
                           temporal_patch_size=c.temporal_patch, spatial_merge_size=c.merge, window_size=c.window,
                           fullatt_block_indexes=list(c.fullatt_blocks), out_hidden_size=c.hidden, in_channels=3, hidden_act="silu"),
        text_config=dict(vocab_size=c.vocab, hidden_size=c.hidden, num_hidden_layers=c.layers, num_attention_heads=c.heads,
                         num_key_value_heads=c.kv_heads, intermediate_size=c.ffn, rms_norm_eps=c.eps, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": c.rope_theta, "mrope_section": list(c.mrope_section)},
                         tie_word_embeddings=False),
        image_token_id=c.image_token)
    hf_cfg._attn_implementation = "eager"
    hf_cfg.vision_config._attn_implementation = "eager"
    hf_cfg.text_config._attn_implementation = "eager"
    hf = Qwen2_5_VLModel(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.copy_((1.0 if "norm" in n or "ln_q" in n else 0.0) + 0.1 * torch.randn_like(p))
    m = BiQwenEmbedder(c)
    load_into(m, _DictLoader({k: v.detach() for k, v in hf.state_dict().items()}))

    grids = [(1, 8, 12), (1, 4, 4)]                             # two images: 96 and 16 patches; windows of 2 x 2 merge blocks
    n_patch = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(n_patch, 3 * c.temporal_patch * c.patch * c.patch)
    with torch.no_grad():
        want = hf.visual(patches, grid_thw=torch.tensor(grids)).pooler_output
        got = m.visual(patches, grids)
    assert got.shape == (n_patch // 4, c.hidden)
    assert torch.allclose(got, want, atol=3e-5), float((got - want).abs().max())

    ids = [5, 6] + [c.image_token] * 24 + [7, 8, 9] + [c.image_token] * 4 + [10, 11]
    pos3 = mrope_positions([int(i == c.image_token) for i in ids], grids, c.merge)
    with torch.no_grad():
        out = hf(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor(grids),
                 position_ids=pos3[:, None, :]).last_hidden_state[0, -1]
        e = m.embed(ids, patches, grids)
    want_e = torch.nn.functional.normalize(out.float(), dim=-1)
    assert torch.allclose(e, want_e, atol=3e-5), float((e - want_e).abs().max())
    with torch.no_grad():
        t_only = m.embed([5, 6, 7, 8])
        want_t = torch.nn.functional.normalize(hf.language_model(input_ids=torch.tensor([[5, 6, 7, 8]])).last_hidden_state[0, -1], dim=-1)
    assert torch.allclose(t_only, want_t, atol=3e-5)

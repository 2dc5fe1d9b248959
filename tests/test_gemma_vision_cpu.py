"""Gemma-4 vision tower against the Hugging Face implementation (random tiny weights loaded by name): a non-square image, with and
without clipped linears, through patch embedding, 2-D rotary blocks, position pooling and the multimodal projection."""
import pytest
import torch

from mary_b200.models.gemma4.vision import Gemma4VisionConfig, Gemma4VisionTower, load_into, patchify


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def has_weight(self, n):
        return n in self.sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)


@pytest.mark.parametrize("clipped", [False, True])
def test_soft_tokens_match_huggingface(clipped):
    pytest.importorskip("transformers")
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig, Gemma4VisionConfig as HFV
    from transformers.models.gemma4.modeling_gemma4 import Gemma4MultimodalEmbedder, Gemma4VisionModel
    c = Gemma4VisionConfig.tiny()
    torch.manual_seed(0)
    hv = HFV(hidden_size=c.hidden, intermediate_size=c.ffn, num_hidden_layers=c.layers, num_attention_heads=c.heads,
             num_key_value_heads=c.kv_heads, head_dim=c.head_dim, patch_size=c.patch, position_embedding_size=c.pos_size,
             pooling_kernel_size=c.pool, rope_parameters={"rope_type": "default", "rope_theta": c.theta}, use_clipped_linears=clipped)
    hv._attn_implementation = "eager"
    tower = Gemma4VisionModel(hv).eval()
    emb = Gemma4MultimodalEmbedder(hv, Gemma4TextConfig(hidden_size=c.text_hidden, num_hidden_layers=2, num_attention_heads=2,
                                                        intermediate_size=32, vocab_size=64, head_dim=8, global_head_dim=8)).eval()
    with torch.no_grad():
        for n, p in tower.named_parameters():
            p.copy_((1.0 + 0.1 * torch.randn_like(p)) if p.dim() == 1 else 0.2 * torch.randn_like(p))
        if clipped:
            for mod in tower.modules():
                if hasattr(mod, "input_min"):
                    mod.input_min.fill_(-0.8), mod.input_max.fill_(0.9), mod.output_min.fill_(-1.5), mod.output_max.fill_(1.2)
    sd = {"model.vision_tower." + k: v.detach() for k, v in tower.state_dict().items()}
    sd.update({"model.embed_vision." + k: v.detach() for k, v in emb.state_dict().items()})
    m = Gemma4VisionTower(c)
    load_into(m, _DictLoader(sd))

    image = torch.rand(3, 4 * c.patch, 6 * c.patch)                    # 4 x 6 patches -> 2 x 3 soft tokens
    patches, pos = patchify(image, c.patch)
    with torch.no_grad():
        want = emb(tower(pixel_values=patches[None], pixel_position_ids=pos[None]).last_hidden_state)
        got = m(patches, pos)
    assert got.shape == (6, c.text_hidden)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), float((got - want).abs().max())
    if clipped:
        assert all(L.q.clipped for L in m.layers)


def test_patchify_orders_patches_row_major_with_xy_positions():
    img = torch.arange(3 * 4 * 6, dtype=torch.float32).reshape(3, 4, 6)
    p, pos = patchify(img, 2)
    assert p.shape == (6, 12) and pos.tolist() == [[0, 0], [1, 0], [2, 0], [0, 1], [1, 1], [2, 1]]
    assert p[1, :3].tolist() == [img[0, 0, 2].item(), img[1, 0, 2].item(), img[2, 0, 2].item()]


def test_soft_tokens_replace_placeholder_rows_in_the_decoder():
    from mary_b200.models.gemma4.config import Gemma4TextConfig
    from mary_b200.models.gemma4.model import Gemma4Model
    from mary_b200.models.gemma4.weights import init_random_
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=32, intermediate_size=96, vocab_size=100,
                           hidden_size_per_layer_input=8)
    m = Gemma4Model(cfg)
    init_random_(m, 0, std=0.05)

    def run(ids, soft=None):
        spec = m.kv_spec()
        cache = PagedKVCache(spec["num_layers"], 4, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
        cache.alloc.extend(0, len(ids))
        table, lens = cache.alloc.page_table([0])
        with torch.no_grad():
            return m(torch.tensor(ids, dtype=torch.int32), BatchMeta.build([len(ids)], lens, table, 16), cache, soft=soft)
    ids = [2, 7, 99, 99, 9]
    rows = torch.tensor([2, 3])
    # soft tokens equal to the scaled embedding of token 0 must reproduce the prompt with token 0 in the placeholder rows
    emb0 = (m.embed[0] * m.embed_scale).expand(2, -1)
    assert torch.allclose(run(ids, (rows, emb0)), run([2, 7, 0, 0, 9]), atol=1e-5)
    other = run(ids, (rows, torch.randn(2, 64)))
    assert (other[-1] - run(ids)[-1]).abs().max() > 1e-4


def test_lm_multimodal_completion_equals_token_completion_when_soft_tokens_are_token_embeddings():
    from mary_b200.models.gemma4.config import Gemma4TextConfig
    from mary_b200.models.gemma4.lm import GemmaLM
    from mary_b200.models.gemma4.model import Gemma4Model
    from mary_b200.models.gemma4.weights import init_random_
    cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=32, intermediate_size=96, vocab_size=100)
    m = Gemma4Model(cfg)
    init_random_(m, 0, std=0.05)
    lm = GemmaLM(m, max_seq=64, max_batch=2)
    want = lm.complete_ids([2, 7, 0, 0, 9], 6)
    emb0 = (m.embed[0] * m.embed_scale).expand(2, -1)
    got = lm.complete_multimodal([2, 7, 99, 99, 9], [2, 3], emb0, 6, stop_on_eos=False)
    assert got == want
    assert lm.cache.alloc.free_pages == lm.cache.alloc.num_pages            # the private sequence was released


def test_multimodal_prompt_end_to_end_matches_huggingface():
    """Image patches -> vision tower -> soft tokens spliced into a prompt -> decoder with per-layer embeddings: logits of the whole
    prompt against the library's multimodal model (placeholder rows look up the pad token for both embedding tables; the soft tokens
    are not scaled by sqrt(hidden); the per-layer projection reads the merged embeddings)."""
    pytest.importorskip("transformers")
    from transformers.models.gemma4 import Gemma4Config, Gemma4ForConditionalGeneration
    from mary_b200.models.gemma4.config import Gemma4TextConfig
    from mary_b200.models.gemma4.model import Gemma4Model
    from mary_b200.models.gemma4.weights import load_into as load_text
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    vc = Gemma4VisionConfig.tiny()
    vc.text_hidden = 64
    torch.manual_seed(0)
    text = dict(vocab_size=120, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                head_dim=32, global_head_dim=32, sliding_window=16, layer_types=["sliding_attention", "full_attention"],
                hidden_size_per_layer_input=16, vocab_size_per_layer_input=120, final_logit_softcapping=30.0, pad_token_id=0,
                rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                 "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1e6}})
    vision = dict(hidden_size=vc.hidden, intermediate_size=vc.ffn, num_hidden_layers=vc.layers, num_attention_heads=vc.heads,
                  num_key_value_heads=vc.kv_heads, head_dim=vc.head_dim, patch_size=vc.patch, position_embedding_size=vc.pos_size,
                  pooling_kernel_size=vc.pool, rope_parameters={"rope_type": "default", "rope_theta": vc.theta})
    hc = Gemma4Config(text_config=text, vision_config=vision, audio_config=None, image_token_id=119)
    for c in (hc, hc.text_config, hc.vision_config):
        c._attn_implementation = "eager"
    hf = Gemma4ForConditionalGeneration(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
            elif "vision_tower" in n or "embed_vision" in n:
                p.copy_(0.2 * torch.randn_like(p))
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    loader = _DictLoader(sd)
    loader.load_host_f32 = lambda n: sd[n].float().numpy()
    cfg = Gemma4TextConfig.from_json(hc.text_config.to_dict())
    m = Gemma4Model(cfg)
    load_text(m, loader)
    tower = Gemma4VisionTower(vc)
    load_into(tower, loader)
    image = torch.rand(3, 4 * vc.patch, 6 * vc.patch)
    patches, pos = patchify(image, vc.patch)
    ids = [2, 7, 8] + [119] * 6 + [9, 10]
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=patches[None], image_position_ids=pos[None]).logits[0]
        soft = tower(patches, pos)
        spec = m.kv_spec()
        cache = PagedKVCache(spec["num_layers"], 2, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
        cache.alloc.extend(0, len(ids))
        table, lens = cache.alloc.page_table([0])
        got = m(torch.tensor(ids, dtype=torch.int32), BatchMeta.build([len(ids)], lens, table, 16), cache, soft=(torch.arange(3, 9), soft))
    assert torch.allclose(got, want, atol=3e-4, rtol=3e-4), float((got - want).abs().max())

"""Gemma-4 text decoder against the Hugging Face implementation of the same architecture (an independent oracle: same weights
by name, logits compared): the plain decoder, K = V global layers with their own KV head count, KV-shared layers with the
double-wide MLP, per-layer embeddings, and the routed-expert block beside the dense MLP."""
import pytest
import torch

from mary_b200.models.gemma4.config import Gemma4TextConfig
from mary_b200.models.gemma4.model import Gemma4Model
from mary_b200.models.gemma4.weights import load_into
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def has_weight(self, n):
        return n in self.sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)

    def load_host_f32(self, n):
        return self.sd[n].float().numpy()


VARIANTS = {
    "plain": {},
    "k_eq_v": dict(attention_k_eq_v=True, num_global_key_value_heads=1, global_head_dim=64),
    "kv_shared_wide": dict(num_kv_shared_layers=2, use_double_wide_mlp=True),
    "ple": dict(hidden_size_per_layer_input=24, vocab_size_per_layer_input=300),
    "moe": dict(enable_moe_block=True, num_experts=8, top_k_experts=2, moe_intermediate_size=48),
    "all": dict(attention_k_eq_v=True, num_global_key_value_heads=1, global_head_dim=64, num_kv_shared_layers=2,
                use_double_wide_mlp=True, hidden_size_per_layer_input=24, vocab_size_per_layer_input=300,
                enable_moe_block=True, num_experts=8, top_k_experts=2, moe_intermediate_size=48),
}


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_logits_and_paged_decode_match_huggingface(variant):
    transformers = pytest.importorskip("transformers")
    from transformers.models.gemma4 import Gemma4ForCausalLM
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig as HFConfig
    torch.manual_seed(0)
    lt = ["sliding_attention", "full_attention"] * 3
    base = dict(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=6, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, global_head_dim=32, sliding_window=8, layer_types=lt, rms_norm_eps=1e-6,
                final_logit_softcapping=30.0, hidden_size_per_layer_input=0, max_position_embeddings=256,
                rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                 "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1e6}})
    base.update(VARIANTS[variant])
    hf_cfg = HFConfig(**base)
    hf_cfg._attn_implementation = "eager"
    hf = Gemma4ForCausalLM(hf_cfg).eval().float()
    with torch.no_grad():                                   # break the symmetry of ones / zeros initialisations
        for n, p in hf.named_parameters():
            if p.dim() == 1 or n.endswith(("router.scale", "per_expert_scale")):
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
            elif "experts" in n:
                p.copy_(0.05 * torch.randn_like(p))
        for i, layer in enumerate(hf.model.layers):
            layer.layer_scalar.fill_(1.0 - 0.05 * i)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = Gemma4TextConfig.from_json(hf_cfg.to_dict())
    assert cfg.enable_moe_block == bool(base.get("enable_moe_block")) and cfg.hidden_size_per_layer_input == base["hidden_size_per_layer_input"]
    m = Gemma4Model(cfg)
    load_into(m, _DictLoader(sd))

    ids = torch.randint(3, 300, (21,))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 16, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    cache.alloc.extend(0, 21)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        got = m(ids.int(), BatchMeta.build([21], lens, table, 16), cache)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), float((got - want).abs().max())

    # the same sequence as a 13-token prefill plus 8 single-token steps over the paged cache
    cache = PagedKVCache(spec["num_layers"], 16, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    cache.alloc.extend(0, 13)
    table, lens = cache.alloc.page_table([0])
    with torch.no_grad():
        first = m(ids[:13].int(), BatchMeta.build([13], lens, table, 16), cache)
        assert torch.allclose(first, want[:13], atol=2e-4, rtol=2e-4)
        for t in range(13, 21):
            cache.alloc.extend(0, 1)
            table, lens = cache.alloc.page_table([0])
            step = m(ids[t:t + 1].int(), BatchMeta.build([1], lens, table, 16), cache)
            assert torch.allclose(step[0], want[t], atol=2e-4, rtol=2e-4), (t, float((step[0] - want[t]).abs().max()))

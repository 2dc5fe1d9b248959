"""Mistral / Qwen3 shell decoder on CPU against the Hugging Face implementation of the same architecture (an independent
oracle: same weights by name, logits compared), the YaRN band rules, and paged-cache decode equal to one full forward."""
import numpy as np
import pytest
import torch

from mary_b200.models.mistral import MistralConfig, MistralModel, init_random_, load_into, yarn_inv_freq
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def has_weight(self, n):
        return n in self.sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)


def _logits(m, ids):
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 16, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    cache.alloc.extend(0, len(ids))
    table, lens = cache.alloc.page_table([0])
    meta = BatchMeta.build([len(ids)], lens, table, 16)
    with torch.no_grad():
        return m(torch.as_tensor(ids, dtype=torch.int32), meta, cache)


@pytest.mark.parametrize("kind", ["mistral", "qwen3"])
def test_logits_match_huggingface_reference_implementation(kind):
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    kw = dict(hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
              vocab_size=300, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=False,
              attention_dropout=0.0)
    if kind == "mistral":
        hf = transformers.MistralForCausalLM(transformers.MistralConfig(sliding_window=None, **kw))
    else:
        hf = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(**kw))
    hf.eval()
    cfg = MistralConfig(2, 64, 160, 4, 2, 32, 300, 10000.0, 1e-5, 256, tie_word_embeddings=False, qk_norm=(kind == "qwen3"))
    m = MistralModel(cfg)
    load_into(m, _DictLoader({k: v.detach() for k, v in hf.state_dict().items()}))
    ids = np.random.default_rng(0).integers(0, 300, 23)
    with torch.no_grad():
        want = hf(torch.as_tensor(ids)[None]).logits[0]
    got = _logits(m, ids)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()


def test_paged_decode_equals_full_forward():
    cfg = MistralConfig(2, 64, 128, 4, 2, 16, 200, 1e4, 1e-5, 128, tie_word_embeddings=True, qk_norm=True)
    m = MistralModel(cfg)
    init_random_(m, 0, std=0.1)
    ids = list(np.random.default_rng(1).integers(0, 200, 12))
    full = _logits(m, ids)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 8, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    outs = []
    for t, tok in enumerate(ids):
        cache.alloc.extend(0, 1)
        table, lens = cache.alloc.page_table([0])
        meta = BatchMeta.build([1], lens, table, 16)
        with torch.no_grad():
            outs.append(m(torch.tensor([tok], dtype=torch.int32), meta, cache)[0])
    assert torch.allclose(torch.stack(outs), full, atol=1e-4)


def test_yarn_bands():
    inv, m = yarn_inv_freq(128, 1e6, 16384, 16.0, 32.0, 1.0)
    base = 1e6 ** (-2.0 * torch.arange(64, dtype=torch.float64) / 128)
    wl = 2 * np.pi / base
    hi, lo = 16384 / 32.0, 16384 / 1.0
    assert torch.allclose(inv[wl < hi].double(), base[wl < hi], rtol=1e-6)                   # short wavelengths untouched
    assert torch.allclose(inv[wl > lo].double(), base[wl > lo] / 16.0, rtol=1e-6)            # long wavelengths fully scaled
    mid = (wl >= hi) & (wl <= lo)
    assert mid.any() and bool(((inv[mid].double() < base[mid] + 1e-12) & (inv[mid].double() > base[mid] / 16.0 - 1e-12)).all())
    assert m == 1.0
    assert yarn_inv_freq(128, 1e6, 4096, 40.0, mscale=1.0, mscale_all_dim=1.0)[1] == pytest.approx(1 + np.log(40.0) / 10.0)
    presets = [MistralConfig.ministral_3b(), MistralConfig.ministral_8b(), MistralConfig.ministral_14b(), MistralConfig.deepseek_r1_qwen3_8b()]
    assert [p.num_hidden_layers for p in presets] == [26, 34, 40, 36] and presets[3].qk_norm and not presets[2].tie_word_embeddings

"""The CPU configuration: tiny Gemma-4-style decoder on CPU from a pile; token-exact, logits within 1e-4 relative."""
import numpy as np
import pytest
import torch

from mary_b200.models.gemma4 import GemmaLM, Gemma4Model, tiny_config
from mary_b200.models.gemma4.weights import random_weights, write_random_pile
from mary_b200.oracle.gemma4 import Gemma4Oracle
from mary_b200.runtime.batch import BatchMeta
from mary_b200.runtime.kv_cache import PagedKVCache


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    from mary_b200.pile import Pile, signing_key_file
    d = tmp_path_factory.mktemp("gemma")
    cfg = tiny_config()
    p = Pile.open(str(d / "g.pile"))
    write_random_pile(p, signing_key_file(str(d / "k")), cfg, seed=0)
    p.close()
    prompt = np.random.default_rng(0).integers(0, 4096, 32).tolist()
    return cfg, str(d / "g.pile"), prompt


def test_greedy_decode_is_token_exact_vs_oracle(tiny):
    cfg, path, prompt = tiny
    lm = GemmaLM.from_pile(path)                       # config-free: hyper-parameters come from facts
    assert lm.model.cfg == cfg
    out = lm.complete_ids(prompt, 32)
    ref, _ = Gemma4Oracle(cfg, dict(random_weights(cfg, 0))).generate(prompt, 32)
    assert out == ref


def test_logits_within_1e4_relative(tiny):
    cfg, path, prompt = tiny
    lm = GemmaLM.from_pile(path)
    orc = Gemma4Oracle(cfg, dict(random_weights(cfg, 0)))
    ref = orc.forward(prompt)
    cache = lm.cache
    cache.alloc.extend(99, len(prompt))
    table, lens = cache.alloc.page_table([99])
    meta = BatchMeta.build([len(prompt)], lens, table, cache.page_size)
    got = lm.model(torch.tensor(prompt), meta, cache).numpy()
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    assert rel < 1e-4, rel
    # one cached decode step
    tok = int(ref[-1].argmax())
    ref2 = orc.forward([tok])
    cache.alloc.extend(99, 1)
    table, lens = cache.alloc.page_table([99])
    meta = BatchMeta.build([1], lens, table, cache.page_size)
    got2 = lm.model(torch.tensor([tok]), meta, cache).numpy()
    assert np.abs(got2 - ref2).max() / np.abs(ref2).max() < 1e-4


def test_oracle_mutant_is_detected(tiny):
    """Positive control: an oracle with the attention scale changed must NOT match."""
    cfg, path, prompt = tiny
    w = dict(random_weights(cfg, 0))
    w["model.layers.0.self_attn.q_norm.weight"] = w["model.layers.0.self_attn.q_norm.weight"] * 0.5
    lm = GemmaLM.from_pile(path)
    bad, _ = Gemma4Oracle(cfg, w).generate(prompt, 8)
    assert lm.complete_ids(prompt, 8) != bad


def test_sliding_window_reach_property():
    """Perturbing a key outside the window of a sliding layer must not move the output; inside it must."""
    from mary_b200.ops import reference as ref
    torch.manual_seed(0)
    L, Hq, Hkv, D, W = 40, 4, 2, 16, 8
    cache = PagedKVCache(1, 8, 16, Hkv, D, dtype=torch.float32)
    cache.alloc.extend(1, L)
    table, lens = cache.alloc.page_table([1])
    meta = BatchMeta.build([L], lens, table, 16)
    k, v, q = torch.randn(L, Hkv, D), torch.randn(L, Hkv, D), torch.randn(L, Hq, D)
    ref.kv_append(k, v, cache.k[0], cache.v[0], meta.slot_mapping)
    base = ref.paged_attention(q, cache.k[0], cache.v[0], meta, 1.0, window=W)
    k2 = k.clone()
    k2[10] += 5.0
    ref.kv_append(k2, v, cache.k[0], cache.v[0], meta.slot_mapping)
    out = ref.paged_attention(q, cache.k[0], cache.v[0], meta, 1.0, window=W)
    moved = (out - base).abs().amax(dim=(1, 2)) > 0
    assert moved[10:18].all() and not moved[:10].any() and not moved[18:].any()
    # GQA group reach: perturbing kv head 1 moves only query heads 2,3
    v2 = v.clone()
    v2[:, 1] += 1.0
    ref.kv_append(k, v2, cache.k[0], cache.v[0], meta.slot_mapping)
    out = ref.paged_attention(q, cache.k[0], cache.v[0], meta, 1.0, window=W)
    d = (out - base).abs().amax(dim=(0, 2))
    assert d[0] == 0 and d[1] == 0 and d[2] > 0 and d[3] > 0


def test_kv_shared_and_k_eq_v_layers_match_oracle(tmp_path):
    """The last layers read the cache of an earlier layer (no K/V projections of their own) and full-attention layers take keys
    and values from one projection (no v_proj tensor): token-exact and within 1e-4 against the NumPy oracle, through a pile."""
    from mary_b200.models.gemma4 import Gemma4TextConfig
    from mary_b200.pile import Pile, signing_key_file
    lt = ["sliding_attention", "full_attention"] * 3
    cfg = Gemma4TextConfig(hidden_size=128, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                           intermediate_size=256, vocab_size=512, layer_types=lt, sliding_window=8, attention_k_eq_v=True,
                           num_kv_shared_layers=2)
    assert [cfg.kv_source(i) for i in range(6)] == [None, None, None, None, 2, 3]
    assert [cfg.k_eq_v(i) for i in range(6)] == [False, True] * 3
    w = dict(random_weights(cfg, 1, std=0.08))
    assert "model.layers.1.self_attn.v_proj.weight" not in w and "model.layers.0.self_attn.v_proj.weight" in w
    assert "model.layers.4.self_attn.k_proj.weight" not in w and "model.layers.5.self_attn.k_norm.weight" not in w
    p = Pile.open(str(tmp_path / "g.pile"))
    write_random_pile(p, signing_key_file(str(tmp_path / "k")), cfg, seed=1, std=0.08) if "std" in write_random_pile.__code__.co_varnames \
        else write_random_pile(p, signing_key_file(str(tmp_path / "k")), cfg, seed=1)
    p.close()
    lm = GemmaLM.from_pile(str(tmp_path / "g.pile"))
    assert lm.model.cfg.num_kv_shared_layers == 2 and lm.model.cfg.attention_k_eq_v
    std = 0.08 if "std" in write_random_pile.__code__.co_varnames else 0.02
    orc = Gemma4Oracle(cfg, dict(random_weights(cfg, 1, std=std)))
    prompt = np.random.default_rng(2).integers(0, 512, 21).tolist()
    ref_tokens, _ = Gemma4Oracle(cfg, dict(random_weights(cfg, 1, std=std))).generate(prompt, 12)
    assert lm.complete_ids(prompt, 12) == ref_tokens
    ref = orc.forward(prompt)
    lm2 = GemmaLM.from_pile(str(tmp_path / "g.pile"))
    cache = lm2.cache
    cache.alloc.extend(7, len(prompt))
    table, lens = cache.alloc.page_table([7])
    got = lm2.model(torch.tensor(prompt), BatchMeta.build([len(prompt)], lens, table, cache.page_size), cache).numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-4

"""MTP speculative decoding: emitted tokens must equal plain greedy decoding; rejected rows leave no trace."""
import numpy as np
import pytest
import torch

from mary_b200.models.moe import MoEDecoder, init_random_, tiny_moe_config
from mary_b200.runtime.kv_cache import PagedKVCache
from mary_b200.runtime.spec_decode import SpecDecoder


def _decoder(k, seed=0, B=3, dtype=torch.float32, device="cpu", graph=False):
    torch.manual_seed(seed)
    cfg = tiny_moe_config("mla")
    m = MoEDecoder(cfg, dtype=dtype, device=device)
    init_random_(m, seed)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], B * 8 + 2, 16, spec["kv_heads"], spec["head_dim"], dtype=dtype, device=device,
                         latent_dim=spec.get("latent_dim"))
    return SpecDecoder(m, cache, B, spec_k=k, max_len=128, device=device, use_graph=graph)


def _run(dec, prompts, n_steps):
    dec.prefill(prompts, chunk=7)
    out = [[int(t)] for t in dec.fed[:, 0].tolist()]
    accepted = 0
    for _ in range(n_steps):
        dec.step()
        em, ne = dec.emitted.cpu().numpy(), dec.n_emitted.cpu().numpy()
        for b in range(dec.B):
            out[b].extend(int(t) for t in em[b, :ne[b]])
            accepted += int(ne[b]) - 1
    return out, accepted


def test_speculative_equals_plain_greedy_cpu():
    prompts = np.random.default_rng(0).integers(0, 2048, (3, 19))
    plain, _ = _run(_decoder(0), prompts, 12)
    for k in (1, 2):
        spec, acc = _run(_decoder(k), prompts, 12)
        for b in range(3):
            n = min(len(plain[b]), len(spec[b]))
            assert spec[b][:n] == plain[b][:n], (k, b)
            assert len(spec[b]) >= len(plain[b])          # speculation never emits fewer tokens per step


def test_forced_correct_drafts_are_all_accepted_cpu():
    """Positive control for acceptance: feed the true continuation as drafts and every draft must be kept."""
    prompts = np.random.default_rng(1).integers(0, 2048, (3, 10))
    plain, _ = _run(_decoder(0), prompts, 6)
    dec = _decoder(2)
    dec.prefill(prompts, chunk=16)
    truth = torch.tensor([p[1:3] for p in plain], dtype=torch.int32)
    dec.fed[:, 1:] = truth
    dec.step()
    assert dec.n_emitted.tolist() == [3, 3, 3]
    assert dec.emitted[:, :2].tolist() == truth.tolist()
    assert dec.kv_before.tolist() == [13, 13, 13]
    # and wrong drafts are all rejected: exactly one token, cache grows by one
    dec2 = _decoder(2)
    dec2.prefill(prompts, chunk=16)
    dec2.fed[:, 1:] = (truth + 1) % 2048
    dec2.step()
    assert dec2.n_emitted.tolist() == [1, 1, 1] and dec2.kv_before.tolist() == [11, 11, 11]
    assert dec2.emitted[:, 0].tolist() == [p[1] for p in plain]


@pytest.mark.gpu
def test_speculative_graph_replay_matches_eager_gpu():
    prompts = np.random.default_rng(2).integers(0, 2048, (3, 21))
    eager, _ = _run(_decoder(2, dtype=torch.bfloat16, device="cuda"), prompts, 8)
    dec = _decoder(2, dtype=torch.bfloat16, device="cuda", graph=True)
    dec.prefill(prompts, chunk=7)
    dec.capture()
    out = [[int(t)] for t in dec.fed[:, 0].tolist()]
    for _ in range(8):
        dec.step()
        em, ne = dec.emitted.cpu().numpy(), dec.n_emitted.cpu().numpy()
        for b in range(3):
            out[b].extend(int(t) for t in em[b, :ne[b]])
    assert out == eager
    from mary_b200.ops import cuda
    assert cuda.last_status() == 0


def test_mla_expanded_prefill_equals_absorbed_attention_cpu():
    """The non-absorbed prefill path (keys / values expanded per head from the latent rows) must give the scores of the
    absorbed latent attention: same layer, same cache, long query blocks vs the same tokens fed in short blocks."""
    from mary_b200.models.moe.model import MLAAttention
    from mary_b200.runtime.batch import BatchMeta
    torch.manual_seed(0)
    cfg = tiny_moe_config("mla")
    m = MoEDecoder(cfg, dtype=torch.float32)
    init_random_(m, 0)
    attn = m.layers[0].attn
    assert isinstance(attn, MLAAttention)
    lens = [70, 55]
    x = torch.randn(sum(lens), cfg.hidden_size) * 0.5
    outs = []
    for thresh in (1, 10 ** 6):                       # expanded path for every block / never
        attn.PREFILL_MIN_ROWS = thresh
        spec = m.kv_spec()
        cache = PagedKVCache(spec["num_layers"], 12, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32, latent_dim=576)
        for s, n in enumerate(lens):
            cache.alloc.extend(s, n)
        table, kl = cache.alloc.page_table([0, 1])
        meta = BatchMeta.build(lens, kl, table, 16)
        with torch.no_grad():
            outs.append(attn(x, meta, cache))
    del attn.PREFILL_MIN_ROWS
    assert torch.allclose(outs[0], outs[1], atol=1e-4, rtol=1e-3), (outs[0] - outs[1]).abs().max()

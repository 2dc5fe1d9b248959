"""The five-launch one-token layer step (``csrc/kernels/layer_step.cu``) against the nine-launch path of the same decoder: hidden
states and cache rows over several decode steps after a shared prefill."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qk_norm,heads,kv_heads,hidden,ffn", [(True, 16, 8, 1024, 3072), (False, 8, 8, 2048, 2816), (True, 8, 2, 520, 1032)])
def test_fused_layer_step_equals_the_unfused_decode_path(qk_norm, heads, kv_heads, hidden, ffn):
    from mary_b200.models.mistral import model as M
    from mary_b200.ops import cuda
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    cfg = M.MistralConfig(3, hidden, ffn, heads, kv_heads, 128, 512, 1e6, 1e-6, 4096, qk_norm=qk_norm, name="tiny")
    model = M.MistralModel(cfg, dtype=torch.bfloat16, device="cuda")
    M.init_random_(model, 0, std=0.05)
    if qk_norm:
        for L in model.layers:
            L.q_norm.data.uniform_(0.5, 1.5)
            L.k_norm.data.uniform_(0.5, 1.5)
    rng = np.random.default_rng(0)
    prompt = torch.from_numpy(rng.integers(0, 512, 37)).to(torch.int32).cuda()
    outs, caches = [], []
    for fused in (False, True):
        M.set_layer_step(fused)
        cache = PagedKVCache(3, 8, 16, kv_heads, 128, dtype=torch.bfloat16, device="cuda")
        cache.alloc.extend(0, 37 + 20)
        table, _ = cache.alloc.page_table([0])
        with torch.no_grad():
            model.hidden(prompt, BatchMeta.build([37], [37], table, 16, "cuda"), cache)          # prefill: the unfused path either way
            hs = []
            launches0 = cuda.LAUNCHES
            for step in range(20):
                tok = torch.tensor([int(rng.integers(0, 512)) if step == 0 else 5 + step], dtype=torch.int32, device="cuda")
                hs.append(model.hidden(tok, BatchMeta.build([1], [38 + step], table, 16, "cuda"), cache).float().cpu())
            per_step = (cuda.LAUNCHES - launches0) / 20
        assert (per_step <= 3 * 5 + 2) if fused else (per_step >= 3 * 8), per_step      # five launches per layer + embedding + final norm
        outs.append(torch.stack(hs))
        caches.append((cache.k[1].float().cpu(), cache.v[2].float().cpu()))
        rng = np.random.default_rng(0)
        rng.integers(0, 512, 37)
    M.set_layer_step(True)
    a, b = outs
    err = (a - b).abs().max().item() / b.abs().max().item()
    assert err < 3e-2, err
    for x, y in zip(caches[0], caches[1]):
        assert (x - y).abs().max().item() < 3e-2 * y.abs().max().item()
    assert cuda.last_status() == 0

"""One tiny end-to-end pass on ``cuda:0`` through the hand-written kernels (used by ``__graft_entry__.smoke``):
the flagship decoder (MLA attention, NVFP4 routed experts, MTP speculative decoding), the continuous-batching engine on a
Gemma-4 decoder, and one LoRA forward + backward + fused AdamW step."""
from __future__ import annotations

import numpy as np
import torch


def _flagship(dev):
    from .models.moe import MoEDecoder, init_random_, tiny_moe_config
    from .runtime.kv_cache import PagedKVCache
    from .runtime.spec_decode import SpecDecoder
    cfg = tiny_moe_config("mla")
    m = MoEDecoder(cfg, dtype=torch.bfloat16, device=dev)
    init_random_(m, 0)
    spec = m.kv_spec()
    B = 4
    cache = PagedKVCache(spec["num_layers"], B * 8 + 2, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16, device=dev,
                         latent_dim=spec.get("latent_dim"))
    dec = SpecDecoder(m, cache, B, spec_k=2, max_len=128, device=dev, use_graph=True)
    dec.prefill(np.random.default_rng(0).integers(0, cfg.vocab_size, (B, 21)), chunk=16)
    dec.capture()
    n = 0
    for _ in range(4):
        dec.step()
        n += int(dec.n_emitted.sum())
    assert n >= 4 * B
    return n


def _gemma_engine(dev):
    from .models.gemma4 import Gemma4Model, Gemma4TextConfig
    from .models.gemma4.weights import init_random_
    from .runtime.engine import Engine
    from .runtime.kv_cache import PagedKVCache
    cfg = Gemma4TextConfig(hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                           intermediate_size=1024, vocab_size=2048, sliding_window=32)
    m = Gemma4Model(cfg, dtype=torch.bfloat16, device=dev)
    init_random_(m, 0)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 64, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16, device=dev)
    e = Engine(m, cache, max_tokens=256, max_seqs=4, device=dev)
    out = e.generate([[1, 2, 3, 4, 5, 6, 7], [9, 8, 7]], 4)
    assert all(len(o) == 4 for o in out)
    return m, out


def _lora_step(m, dev):
    from .train.trainer import LoraTrainer
    tr = LoraTrainer(m, rank=8, alpha=16.0, lr=1e-3)
    ids = torch.randint(0, 2048, (2, 32), device=dev)
    l0 = tr.step(ids)
    l1 = tr.step(ids)
    assert np.isfinite(l0) and np.isfinite(l1)
    return l0, l1


def run_smoke() -> None:
    from .ops import cuda
    cuda.lib()                                       # fails loudly when the kernel library is missing
    dev = "cuda:0"
    torch.cuda.set_device(0)
    n = _flagship(dev)
    m, out = _gemma_engine(dev)
    losses = _lora_step(m, dev)
    torch.cuda.synchronize()
    st = cuda.last_status()
    assert st == 0, f"kernel status {st}"
    print(f"smoke ok: flagship emitted {n} tokens in 4 speculative steps; gemma {out}; lora loss {losses[0]:.3f} -> {losses[1]:.3f}; "
          f"{cuda.LAUNCHES} kernel launches")

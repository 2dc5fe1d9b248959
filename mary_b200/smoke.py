"""One tiny end-to-end pass on ``cuda:0`` through the hand-written kernels (used by ``__graft_entry__.smoke``)."""
from __future__ import annotations

import torch


def run_smoke() -> None:
    from .models.gemma4 import Gemma4Model, Gemma4TextConfig
    from .models.gemma4.weights import init_random_
    from .ops import cuda
    from .runtime.engine import Engine
    from .runtime.kv_cache import PagedKVCache

    cuda.lib()                                       # fails loudly when the kernel library is missing
    dev = "cuda:0"
    torch.cuda.set_device(0)
    cfg = Gemma4TextConfig(hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                           intermediate_size=1024, vocab_size=2048, sliding_window=32)
    m = Gemma4Model(cfg, dtype=torch.bfloat16, device=dev)
    init_random_(m, 0)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 64, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.bfloat16, device=dev)
    e = Engine(m, cache, max_tokens=256, max_seqs=4, device=dev)
    out = e.generate([[1, 2, 3, 4, 5, 6, 7], [9, 8, 7]], 4)
    torch.cuda.synchronize()
    st = cuda.last_status()
    assert st == 0, f"kernel status {st}"
    assert all(len(o) == 4 for o in out)
    print("smoke ok:", out)

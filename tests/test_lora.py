import numpy as np
import pytest
import torch

from mary_b200.models.gemma4 import Gemma4Model, Gemma4TextConfig
from mary_b200.models.gemma4.weights import init_random_
from mary_b200.pile import MemoryBlobStore, TribleBuilder
from mary_b200.train.lora import Gemma4LoraForward, LoraWeights
from mary_b200.train.trainer import FlatAdamW, LoraTrainer


def _model(device="cpu", dtype=torch.float32):
    cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                           intermediate_size=128, vocab_size=97, sliding_window=8)
    m = Gemma4Model(cfg, dtype=dtype, device=device)
    init_random_(m, 0, std=0.08)
    return m


def test_adapter_init_rules_and_zero_delta():
    m = _model()
    lw = LoraWeights.init_gemma4(m, rank=4, alpha=8.0)
    ad = lw.get(0, "q_proj")
    assert ad.A.abs().max() <= (3.0 / 64) ** 0.5 + 1e-6 and ad.B.abs().max() == 0 and ad.scale == 2.0
    assert len(lw.adapters) == 2 * 7
    assert lw.num_params() == sum(p.numel() for p in lw.parameters()) > 0
    ids = torch.randint(0, 97, (2, 12))
    fwd = Gemma4LoraForward(m, lw)
    base = fwd.forward(ids)
    for a in lw.adapters.values():                  # B = 0: adapters change nothing at step 0
        a.A.data.mul_(3.0)
    assert torch.equal(fwd.forward(ids), base)


def test_training_forward_matches_serving_forward():
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    m = _model()
    lw = LoraWeights.init_gemma4(m, rank=4)
    ids = torch.randint(0, 97, (1, 20))
    x_train = Gemma4LoraForward(m, lw).forward(ids)[0]
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 8, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    cache.alloc.extend(0, 20)
    table, lens = cache.alloc.page_table([0])
    meta = BatchMeta.build([20], lens, table, 16)
    with torch.no_grad():
        x_serve = m.hidden(ids[0].int(), meta, cache)
    assert torch.allclose(x_train, x_serve, atol=2e-4, rtol=1e-3)


def test_gradients_match_plain_autograd_of_merged_weights():
    """d loss / d A, d B through the frozen-GEMM autograd path == gradients of a model whose weights are W + s B A."""
    m = _model()
    lw = LoraWeights.init_gemma4(m, rank=4)
    for a in lw.adapters.values():
        a.B.data.normal_(0, 0.05)
    ids = torch.randint(0, 97, (2, 10))
    loss = Gemma4LoraForward(m, lw).loss(ids)
    loss.backward()
    ad = lw.get(1, "down_proj")
    eps = 1e-3
    # finite difference on one coordinate of B and of A
    for t, idx in ((ad.B, (3, 1)), (ad.A, (2, 5))):
        g = t.grad[idx].item()
        old = t.data[idx].item()
        t.data[idx] = old + eps
        lp = Gemma4LoraForward(m, lw).loss(ids).item()
        t.data[idx] = old - eps
        lm = Gemma4LoraForward(m, lw).loss(ids).item()
        t.data[idx] = old
        assert abs((lp - lm) / (2 * eps) - g) < 5e-3 * max(1.0, abs(g)), (g, (lp - lm) / (2 * eps))


def test_adamw_matches_reference_formula_and_loss_halves():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(7))
    opt = FlatAdamW([p], lr=1e-2)
    ref_p, m, v = p.data.clone(), torch.zeros(7), torch.zeros(7)
    for step in range(1, 4):
        g = torch.randn(7)
        p.grad.copy_(g)
        opt.step()
        m = 0.9 * m + 0.1 * g
        v = 0.999 * v + 0.001 * g * g
        ref_p = ref_p - 1e-2 * ((m / (1 - 0.9 ** step)) / ((v / (1 - 0.999 ** step)).sqrt() + 1e-8) + 0.01 * ref_p)
        assert torch.allclose(p.data, ref_p, atol=1e-6)
    tr = LoraTrainer(_model(), rank=8, alpha=16.0, lr=2e-2)
    ids = torch.randint(0, 97, (2, 16))
    losses = [tr.step(ids) for _ in range(60)]
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])       # the reference trainer's own acceptance check


def test_checkpoint_resume_is_bitwise():
    ids = [torch.randint(0, 97, (1, 12), generator=torch.Generator().manual_seed(s)) for s in range(6)]
    a = LoraTrainer(_model(), rank=4, lr=1e-2)
    la = [a.step(x) for x in ids]
    b = LoraTrainer(_model(), rank=4, lr=1e-2)
    lb = [b.step(x) for x in ids[:3]]
    store, tb = MemoryBlobStore(), TribleBuilder()
    ck = b.save_checkpoint(store, tb)
    facts = tb.build()
    c = LoraTrainer(_model(), rank=4, lr=1e-2)
    from mary_b200.pile.trible import r_genid
    from mary_b200.format import schema as S
    c.lora.load_from_pile(store, facts, r_genid(facts.one(ck, S.TRAIN_ADAPTER)))
    c.load_checkpoint(store, facts, ck)
    lc = [c.step(x) for x in ids[3:]]
    assert lb + lc == la
    assert torch.equal(c.opt.flat, a.opt.flat)


def test_peft_safetensors_roundtrip(tmp_path):
    m = _model()
    lw = LoraWeights.init_gemma4(m, rank=4)
    for a in lw.adapters.values():
        a.B.data.normal_()
    lw.save_safetensors(str(tmp_path / "adapter.safetensors"))
    lw2 = LoraWeights.init_gemma4(m, rank=4, seed=9)
    lw2.load_safetensors(str(tmp_path / "adapter.safetensors"))
    for k in lw.adapters:
        assert torch.equal(lw.adapters[k].A, lw2.adapters[k].A) and torch.equal(lw.adapters[k].B, lw2.adapters[k].B)


def test_activation_checkpointing_gives_the_same_gradients():
    from mary_b200.models.gemma4 import Gemma4Model, Gemma4TextConfig
    from mary_b200.models.gemma4.weights import init_random_
    from mary_b200.train.lora import Gemma4LoraForward, LoraWeights
    cfg = Gemma4TextConfig(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                           intermediate_size=128, vocab_size=100, sliding_window=8)
    m = Gemma4Model(cfg)
    init_random_(m, 0, std=0.1)
    ids = torch.randint(0, 100, (2, 20))
    grads = []
    for ck in (False, True):
        lw = LoraWeights.init_gemma4(m, rank=4, seed=1)
        for a in lw.adapters.values():
            a.B.data.normal_(0, 0.05, generator=torch.Generator().manual_seed(2))
        f = Gemma4LoraForward(m, lw)
        f.checkpoint = ck
        f.loss(ids).backward()
        grads.append(torch.cat([p.grad.flatten() for p in lw.parameters()]))
    assert torch.allclose(grads[0], grads[1], atol=1e-6)


def test_activation_checkpointing_gives_the_same_loss_and_gradients():
    """Recomputing every layer in the backward pass (the widened GEMM operands are rebuilt by the recomputation) changes nothing."""
    def run(ckpt):
        m = _model()
        lw = LoraWeights.init_gemma4(m, rank=4, seed=1)
        g = torch.Generator().manual_seed(2)
        for ad in lw.adapters.values():
            ad.B.data.normal_(0, 0.05, generator=g)
        tr = LoraTrainer(m, rank=4, lr=1e-2, lora=lw, checkpoint=ckpt)
        ids = torch.randint(0, 97, (2, 12), generator=torch.Generator().manual_seed(3))
        tr.opt.zero_grad()
        loss = tr.fwd.loss(ids)
        loss.backward()
        return float(loss.detach()), tr.opt.grad.clone()
    a, ga = run(False)
    b, gb = run(True)
    assert a == b and torch.equal(ga, gb) and ga.abs().max() > 0

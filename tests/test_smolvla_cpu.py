"""SmolVLA: the flow time code, the backwards Euler sampler on fields with known solutions, expert layers reading the backbone's
cache (self-attention layers see prefix and suffix, cross-attention layers see only the re-projected prefix), visibility of the
prefix blocks, and the SGD overfit probe of the action expert."""
import math

import torch

from mary_b200.models.smolvla import SmolVLA, SmolVLAConfig, euler_sample, time_embedding
from mary_b200.models.smolvla.model import init_random_


def test_time_embedding_periods_are_geometric():
    e = time_embedding(torch.tensor([0.25]), 8, 4e-3, 4.0)[0]
    periods = [4e-3 * 1000 ** (i / 3) for i in range(4)]
    for i, p in enumerate(periods):
        assert math.isclose(e[i].item(), math.sin(2 * math.pi * 0.25 / p), abs_tol=1e-4)
        assert math.isclose(e[4 + i].item(), math.cos(2 * math.pi * 0.25 / p), abs_tol=1e-4)


def test_euler_sampler_integrates_from_one_to_zero():
    noise = torch.randn(2, 5, 3)
    c = torch.randn(5, 3)
    assert torch.allclose(euler_sample(lambda x, t: c.expand_as(x), noise, 10), noise - c, atol=1e-5)      # constant field: exact
    seen = []
    euler_sample(lambda x, t: (seen.append(float(t[0])), torch.zeros_like(x))[1], noise, 4)
    assert seen == [1.0, 0.75, 0.5, 0.25]
    # the rectified-flow field of a point target a: v = (x - a) / t carries any x at t = 1 to a at t = 0, exactly under Euler
    a = torch.randn(5, 3)
    out = euler_sample(lambda x, t: (x - a) / t[:, None, None], noise, 7)
    assert torch.allclose(out, a.expand_as(out), atol=1e-4)


def _model():
    torch.manual_seed(0)
    m = SmolVLA(SmolVLAConfig.tiny())
    init_random_(m, 0, std=0.2)
    return m


def test_prefix_blocks_and_expert_layers_see_what_they_should():
    m = _model()
    c = m.c
    img = torch.rand(3, 32, 32) * 2 - 1
    x, blocks = m.embed_prefix([img], [3, 4, 5], torch.randn(c.state_dim))
    assert x.shape == (4 + 3 + 1, c.vlm.width) and blocks.tolist() == [0] * 7 + [1]
    cache = m.prefix_cache(x, blocks)
    # images / language do not see the state token: changing the state leaves their keys unchanged in every layer
    x2, _ = m.embed_prefix([img], [3, 4, 5], torch.randn(c.state_dim))
    cache2 = m.prefix_cache(x2, blocks)
    for (k, v), (k2, v2) in zip(cache, cache2):
        assert torch.allclose(k[:7], k2[:7], atol=1e-6) and torch.allclose(v[:7], v2[:7], atol=1e-6)
    assert not torch.allclose(cache[1][0][7], cache2[1][0][7])
    noisy = torch.randn(c.chunk_size, c.action_dim)
    v1 = m.denoise(cache, noisy, torch.tensor(0.6))
    assert v1.shape == (c.chunk_size, c.action_dim)
    # the action tokens see each other: perturbing the last action changes the first token's velocity
    n2 = noisy.clone()
    n2[-1] += 1.0
    assert not torch.allclose(m.denoise(cache, n2, torch.tensor(0.6))[0], v1[0])
    # ... and see the prefix: another observation changes the velocity; another flow time does too
    assert not torch.allclose(m.denoise(cache2, noisy, torch.tensor(0.6)), v1)
    assert not torch.allclose(m.denoise(cache, noisy, torch.tensor(0.2)), v1)
    # odd layers read the backbone's K/V through their own kv_dim -> kv_dim projections
    kv = c.vlm.n_kv_heads * c.vlm.head_dim
    assert m.expert_layers[1].wk.shape == (kv, kv) and m.expert_layers[0].wk.shape == (kv, c.expert.width)
    act = m.act([img], [3, 4, 5], torch.randn(c.state_dim), generator=torch.Generator().manual_seed(1))
    assert act.shape == (c.chunk_size, c.expressive_dim) and torch.isfinite(act).all()


def test_sgd_overfit_probe_of_the_action_expert():
    m = _model()
    c = m.c
    img = torch.rand(3, 32, 32) * 2 - 1
    with torch.no_grad():
        cache = m.prefix_cache(*m.embed_prefix([img], [3, 4, 5], torch.randn(c.state_dim)))
    train = [p for n, p in m.named_parameters() if n.startswith(("expert_", "act_", "at_"))]
    for p in train:
        p.requires_grad_(True)
    actions = torch.randn(c.chunk_size, c.action_dim) * 0.5
    g = torch.Generator().manual_seed(3)
    pairs = [(torch.randn(c.chunk_size, c.action_dim, generator=g), float(torch.rand((), generator=g)) * 0.98 + 0.01) for _ in range(4)]
    opt = torch.optim.SGD(train, lr=0.05, momentum=0.9)
    first = last = None
    for step in range(150):
        loss = sum(m.flow_loss(cache, actions, n, t) for n, t in pairs) / len(pairs)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
    assert last < 0.2 * first, (first, last)

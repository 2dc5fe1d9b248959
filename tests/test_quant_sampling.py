import pytest
import numpy as np
import torch

from mary_b200.nn.q4 import QLinear, dequantize_q4, dequantize_q8, quantize_q4, quantize_q8
from mary_b200.ops.sampling import filter_top_k_top_p, sample
from mary_b200.runtime.kv_quant import (QuantizedKVCache, TurboQuant, hadamard, pack_int4, quantize_absmax, unpack_int4)


def test_q4_q8_block_formats():
    w = np.random.default_rng(0).standard_normal((8, 96)).astype(np.float32)
    q = quantize_q4(w)
    assert q.shape == (8, 3, 18)
    assert np.abs(dequantize_q4(q) - w).max() <= np.abs(w).reshape(8, 3, 32).max(-1).max() / 8 * 1.01
    assert np.abs(dequantize_q8(quantize_q8(w)) - w).max() < np.abs(w).max() / 127 * 1.01
    # the element of largest magnitude in a block is reproduced exactly up to the f16 scale (code 0 = -8 * d)
    x = torch.randn(96)
    lin = QLinear(w, "q4")
    assert torch.allclose(lin(x), torch.from_numpy(dequantize_q4(q)) @ x, atol=1e-4)
    sw = QLinear(np.concatenate([w, w * 0.5]), "q8", swiglu=True)
    y = torch.from_numpy(dequantize_q8(quantize_q8(np.concatenate([w, w * 0.5])))) @ x
    assert torch.allclose(sw(x), torch.nn.functional.silu(y[:8]) * y[8:], atol=1e-4)


def test_int8_int4_kv_cache():
    torch.manual_seed(0)
    k, v = torch.randn(5, 2, 64), torch.randn(5, 2, 64)
    for bits, tol in ((8, 0.02), (4, 0.2)):
        c = QuantizedKVCache(bits)
        c.append(k[:3], v[:3])
        c.append(k[3:], v[3:])
        assert (c.keys() - k).abs().max() < tol * k.abs().max() and (c.values() - v).abs().max() < tol * v.abs().max()
    codes, _ = quantize_absmax(k, 4)
    assert torch.equal(unpack_int4(pack_int4(codes)), codes)
    assert QuantizedKVCache(4).nbytes() == 0


def test_turboquant_rotation_and_inner_products():
    torch.manual_seed(1)
    x = torch.randn(200, 128)
    assert torch.allclose(hadamard(hadamard(x)), x, atol=1e-4)            # orthonormal involution
    tq = TurboQuant(128, bits=3, seed=0)
    assert torch.allclose(tq.unrotate(tq.rotate(x)), x, atol=1e-4)
    codes, n, bits, rn = tq.encode(x)
    rec = tq.decode(codes, n)
    rel = (rec - x).norm(dim=-1) / x.norm(dim=-1)
    assert rel.mean() < 0.2                                                # 3-bit Lloyd-Max on Gaussian coordinates
    # quantisation shrinks vectors, so <rec, x> underestimates |x|^2 systematically; the 1-bit sketch of the residual
    # removes that bias (it is unbiased, at the price of variance)
    nx = (x * x).sum(-1)
    plain = (((rec * x).sum(-1) - nx) / nx).mean()
    sketched = (((tq.decode(codes, n, bits, rn) * x).sum(-1) - nx) / nx).mean()
    assert plain < -0.02 and abs(sketched) < abs(plain) / 2, (plain, sketched)
    assert (TurboQuant(128, bits=4).decode(*TurboQuant(128, bits=4).encode(x)[:2]) - x).norm() < (rec - x).norm()


def test_sampling_rules():
    lg = torch.tensor([[1.0, 3.0, 3.0, -2.0]])
    assert sample(lg).tolist() == [1]                                       # greedy: first maximum
    f = filter_top_k_top_p(lg, top_k=2)
    assert torch.isinf(f[0, 0]) and torch.isinf(f[0, 3]) and f[0, 1] == 3
    p = filter_top_k_top_p(torch.tensor([[2.0, 1.0, 0.0, -1.0]]), top_p=0.7)
    assert torch.isfinite(p[0, :2]).all() and torch.isinf(p[0, 2:]).all()   # 0.64 < 0.7 -> second token still needed
    big = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(4000, 1)
    cnt = torch.zeros(4)
    for s in range(3):
        cnt += torch.bincount(sample(big, temperature=1.0, seed=5, step=s), minlength=4).float()
    assert ((cnt / cnt.sum()) - torch.softmax(big[0], 0)).abs().max() < 0.03
    assert torch.equal(sample(big, temperature=0.7, seed=1, step=2), sample(big, temperature=0.7, seed=1, step=2))


def test_reference_sampler_properties_of_the_speech_models_rule():
    from mary_b200.ops.sampling import draw_uniform, sample_reference
    g = torch.Generator().manual_seed(3)
    row = torch.randn(200, generator=g) * 3
    order = torch.sort(row, descending=True, stable=True).indices.tolist()
    # top-k truncation: only the k highest survive; ties at the cut keep the lower index
    tok, kept = sample_reference(row, 1.0, top_k=7, u=0.5)
    assert sorted(kept) == sorted(order[:7]) and tok in kept
    tied = torch.tensor([1.0, 3.0, 3.0, 3.0, 0.0])
    assert sample_reference(tied, 1.0, top_k=2, u=0.1)[1] == [1, 2]
    # nucleus: smallest prefix whose mass reaches p, at least one token
    p = torch.softmax(row.double(), 0)[order]
    n = int((torch.cumsum(p, 0) >= 0.6).nonzero()[0]) + 1
    assert sorted(sample_reference(row, 1.0, top_p=0.6, u=0.3)[1]) == sorted(order[:n])
    assert sample_reference(row, 1.0, top_p=1e-9, u=0.9)[1] == [order[0]]
    # temperature -> 0 is the arg-max; non-finite logits never win; an all-non-finite row falls back to the arg-max rule
    assert sample_reference(row, 1e-4, u=0.999)[0] == order[0]
    bad = row.clone()
    bad[order[0]] = float("nan")
    bad[order[1]] = float("inf")
    assert order[0] not in sample_reference(bad, 1.0, top_k=5, u=0.0)[1] and order[1] not in sample_reference(bad, 1.0, top_k=5, u=0.0)[1]
    assert sample_reference(torch.full((4,), float("nan")), 1.0, u=0.5)[1] == []
    # the draw follows the distribution: frequencies over many uniforms
    small = torch.tensor([2.0, 1.0, 0.0, -1.0])
    cnt = torch.zeros(4)
    for s in range(4000):
        cnt[sample_reference(small, 1.0, u=draw_uniform(9, s, 0))[0]] += 1
    assert (cnt / 4000 - torch.softmax(small, 0)).abs().max() < 0.03
    us = [draw_uniform(1, s, r) for s in range(50) for r in range(4)]
    assert len(set(us)) == 200 and all(0.0 <= u < 1.0 for u in us) and draw_uniform(1, 2, 3) == draw_uniform(1, 2, 3)


@pytest.mark.gpu
def test_device_sampler_picks_the_reference_token_for_every_setting():
    from mary_b200.ops import cuda as K
    from mary_b200.ops.sampling import draw_uniform, sample, sample_reference
    g = torch.Generator().manual_seed(4)
    for V, scale in ((2048, 3.0), (32000, 2.0), (50, 1.0), (262144, 1.5)):
        rows = 6 if V > 100000 else 17
        lg = (torch.randn(rows, V, generator=g) * scale)
        lg[0, 5] = float("nan")
        lg[1, 7] = float("inf")
        lg[2, :V // 2] = float("-inf")
        dev = lg.cuda()
        for T, k, p in ((1.0, 0, 1.0), (0.8, 250, 1.0), (0.7, 0, 0.9), (1.2, 50, 0.8), (0.9, 1, 1.0), (1.0, 3, 1e-6), (0.5, 10 ** 6, 0.999)):
            for step in (0, 1):
                got, prob = K.sample_top_k_top_p(dev, T, k, p, seed=11, step=step, want_prob=True)
                assert K.last_status() == 0
                for r in range(rows):
                    tok, kept = sample_reference(lg[r], T, k, p, draw_uniform(11, step, r))
                    assert int(got[r]) in kept, (V, T, k, p, r)
                    assert int(got[r]) == tok, (V, T, k, p, r, int(got[r]), tok)
                assert (prob > 0).all() and (prob <= 1.0001).all()
    # bf16 logits: many exact ties at the thresholds; the kept set must still be the stable-sort prefix
    lg = (torch.randn(9, 4096, generator=g) * 2).bfloat16()
    got = K.sample_top_k_top_p(lg.cuda(), 1.0, 40, 0.95, seed=3, step=7)
    for r in range(9):
        tok, kept = sample_reference(lg[r].float(), 1.0, 40, 0.95, draw_uniform(3, 7, r))
        assert int(got[r]) == tok
    # an all-non-finite row yields index 0 and the status stays clean; the public entry agrees host and device
    assert int(K.sample_top_k_top_p(torch.full((1, 64), float("nan"), device="cuda"), 1.0)[0]) == 0
    x = torch.randn(5, 300, generator=g)
    assert sample(x, 0.8, 20, 0.9, seed=2, step=3).tolist() == sample(x.cuda(), 0.8, 20, 0.9, seed=2, step=3).tolist()
    # frequencies follow the distribution
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).cuda().expand(4096, 4).contiguous()
    ids = K.sample_top_k_top_p(small, 1.0, seed=5, step=0)
    freq = torch.bincount(ids.long(), minlength=4).float().cpu() / 4096
    assert (freq - torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0)).abs().max() < 0.03


def _q8_case(seed=0, S=3, Hq=8, Hkv=2, D=64, page=16, lens=(40, 17, 70), device="cpu", dtype=torch.float32):
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import PagedKVCache
    g = torch.Generator().manual_seed(seed)
    pages = sum((n + page - 1) // page for n in lens) + 2
    full = PagedKVCache(1, pages, page, Hkv, D, dtype=dtype, device=device)
    q8 = PagedKVCache(1, pages, page, Hkv, D, dtype=dtype, device=device, kv_dtype="int8")
    for s, n in enumerate(lens):
        full.alloc.extend(s, n)
        q8.alloc.extend(s, n)
    table, kv = full.alloc.page_table(list(range(S)))
    meta_fill = BatchMeta.build(list(lens), kv, table, page, device)
    T = sum(lens)
    k = (torch.randn(T, Hkv, D, generator=g) * 1.5 + 0.3).to(dtype).to(device)
    v = torch.randn(T, Hkv, D, generator=g).to(dtype).to(device)
    return full, q8, meta_fill, k, v, table, kv, g


def test_int8_kv_pages_quantise_like_the_reference_and_serve_attention():
    from mary_b200 import ops
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import Q8Pages
    full, q8, meta, k, v, table, kv, g = _q8_case()
    # the rule: per (token, head) range / 255, zero = min, round half up; a constant row keeps scale 1
    codes, sz = Q8Pages.quantize(torch.tensor([[0.0, 1.0, 2.55], [3.0, 3.0, 3.0]]))
    assert codes.tolist() == [[0, 100, 255], [0, 0, 0]] and torch.allclose(sz, torch.tensor([[0.01, 0.0], [1.0, 3.0]]))
    full.k[0].view(-1, 2, 64)[meta.slot_mapping] = k
    full.v[0].view(-1, 2, 64)[meta.slot_mapping] = v
    ops.kv_quant_append(k, meta.slot_mapping, q8.k[0])
    ops.kv_quant_append(v, meta.slot_mapping, q8.v[0])
    back = q8.k[0].dequantize(dtype=torch.float32).view(-1, 2, 64)[meta.slot_mapping]
    step = (k.max(-1).values - k.min(-1).values) / 255
    assert ((back - k).abs() <= step[..., None] * 0.5001 + 1e-6).all()
    assert q8.bytes() < 0.6 * full.bytes() * (2 / 4)                                      # half of a bf16 cache, plus the pairs
    # decode rows and a prefill chunk against the unquantised cache: the error is the quantisation step, not more
    for q_lens in ([1, 1, 1], [3, 0, 2], [40, 17, 70]):
        m = BatchMeta.build(q_lens, kv, table, 16, "cpu")
        q = torch.randn(sum(q_lens), 8, 64, generator=g)
        for window in (0, 24):
            want = ops.paged_attention(q, full.k[0], full.v[0], m, 0.125, window)
            got = ops.paged_attention(q, q8.k[0], q8.v[0], m, 0.125, window)
            assert (got - want).abs().max() < 0.03 and not torch.equal(got, want)
            exact = ops.paged_attention(q, q8.k[0].dequantize(dtype=torch.float32), q8.v[0].dequantize(dtype=torch.float32), m, 0.125, window)
            assert torch.allclose(got, exact, atol=1e-5)
    with pytest.raises(ValueError):
        from mary_b200.runtime.kv_cache import PagedKVCache
        PagedKVCache(1, 4, 16, 1, 64, latent_dim=576, kv_dtype="int8")


@pytest.mark.gpu
def test_int8_kv_append_and_dequantising_decode_kernel_match_the_host_rule():
    from mary_b200 import ops
    from mary_b200.ops import cuda as K
    from mary_b200.ops import reference as ref
    from mary_b200.runtime.batch import BatchMeta
    from mary_b200.runtime.kv_cache import Q8Pages
    for D, Hq, Hkv, lens in ((64, 8, 2, (40, 17, 700)), (128, 8, 1, (300, 5, 64)), (256, 8, 4, (1000, 33, 250))):
        full, q8, meta, k, v, table, kv, g = _q8_case(seed=D, Hq=Hq, Hkv=Hkv, D=D, lens=lens, device="cuda", dtype=torch.bfloat16)
        before = K.LAUNCHES
        ops.kv_quant_append(k, meta.slot_mapping, q8.k[0])
        ops.kv_quant_append(v, meta.slot_mapping, q8.v[0])
        assert K.LAUNCHES == before + 2 and K.last_status() == 0
        codes, sz = Q8Pages.quantize(k.cpu())
        got_codes = q8.k[0].codes.view(-1, Hkv, D)[meta.slot_mapping].cpu()
        assert (got_codes.int() - codes.int()).abs().max() <= 1 and (got_codes == codes).float().mean() > 0.99     # approximate division may move a value that sits at a rounding boundary
        assert torch.allclose(q8.k[0].sz.view(-1, Hkv, 2)[meta.slot_mapping].cpu(), sz, rtol=1e-5, atol=1e-7)
        kd, vd = q8.k[0].dequantize(dtype=torch.float32).cpu(), q8.v[0].dequantize(dtype=torch.float32).cpu()
        for q_lens in ([1, 1, 1], [2, 1, 2]):
            m = BatchMeta.build(q_lens, kv, table, 16, "cuda")
            mc = BatchMeta.build(q_lens, kv, table, 16, "cpu")
            q = torch.randn(sum(q_lens), Hq, D, generator=g).bfloat16()
            for window, softcap in ((0, 0.0), (128, 0.0), (0, 30.0)):
                assert K.decode_q8_supported(q.cuda(), q8.k[0], m)
                before = K.LAUNCHES
                got = ops.paged_attention(q.cuda(), q8.k[0], q8.v[0], m, D ** -0.5, window, softcap).float().cpu()
                assert K.LAUNCHES > before and K.last_status() == 0
                want = ref.paged_attention(q.float(), kd, vd, mc, D ** -0.5, window, softcap)
                assert (got - want).abs().max() < 0.02, (D, q_lens, window, softcap)
        # a prefill chunk takes the dequantise-the-batch path and agrees as well
        m = BatchMeta.build(list(lens), kv, table, 16, "cuda")
        mc = BatchMeta.build(list(lens), kv, table, 16, "cpu")
        q = torch.randn(sum(lens), Hq, D, generator=g).bfloat16()
        got = ops.paged_attention(q.cuda(), q8.k[0], q8.v[0], m, D ** -0.5).float().cpu()
        want = ref.paged_attention(q.float(), kd, vd, mc, D ** -0.5)
        assert (got - want).abs().max() < 0.03
    # out-of-range slot: refused through the status word, nothing written
    bad = torch.tensor([10 ** 9], dtype=torch.int64, device="cuda")
    K.lib().mary_kv_quant_append(k[:1].data_ptr(), k.stride(0), bad.data_ptr(), q8.k[0].codes.data_ptr(), q8.k[0].sz.data_ptr(), 1, Hkv, D,
                                 q8.k[0].codes.shape[0] * 16, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert K.last_status() != 0 and K.last_status() == 0                                 # reading clears it

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

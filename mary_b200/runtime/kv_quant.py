"""KV-cache quantisation: int8 / int4 per-(token, head) absmax codes and TurboQuant.

Reference: host int8/int4 caches with an optional 1-bit residual (src/models/gemma/layers.rs:76-520), the device
variant packing four int8 per word (src/models/gemma/gpu_quant.rs:28-166) and TurboQuant — a randomised Hadamard
rotation, per-coordinate Lloyd-Max scalar quantisation of the rotated (near-Gaussian) vector and a 1-bit
Johnson-Lindenstrauss sketch of the residual that makes inner products unbiased (src/models/gemma/turbo_quant.rs:29-52,
arXiv 2504.19874).  Everything here is torch tensor code, so it runs on the GPU as written."""
from __future__ import annotations

import math

import torch

# Lloyd-Max reconstruction levels for a unit Gaussian (positive half; symmetric).
_LLOYD = {1: [0.7979], 2: [0.4528, 1.5104], 3: [0.2451, 0.7560, 1.3439, 2.1520],
          4: [0.1284, 0.3881, 0.6568, 0.9424, 1.2562, 1.6180, 2.0690, 2.7326]}


def quantize_absmax(x, bits: int = 8):
    """``x[..., D]`` -> ``(codes int8[..., D], scale f32[..., 1])`` with ``x ~ codes * scale``."""
    qmax = (1 << (bits - 1)) - 1
    s = x.float().abs().amax(-1, keepdim=True) / qmax
    s = torch.where(s > 0, s, torch.ones_like(s))
    return torch.clamp(torch.round(x.float() / s), -qmax, qmax).to(torch.int8), s


def dequantize_absmax(codes, scale):
    return codes.float() * scale


def pack_int4(codes):
    """int8 codes in [-7, 7] -> two per byte (low nibble first)."""
    u = (codes + 8).to(torch.uint8)
    return u[..., 0::2] | (u[..., 1::2] << 4)


def unpack_int4(packed):
    lo, hi = (packed & 0xF).to(torch.int8) - 8, (packed >> 4).to(torch.int8) - 8
    return torch.stack([lo, hi], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def hadamard(x):
    """Fast Walsh-Hadamard transform over the last dim (a power of two), orthonormal."""
    d = x.shape[-1]
    assert d & (d - 1) == 0
    y = x.float()
    h = 1
    while h < d:
        y = y.reshape(*y.shape[:-1], d // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], -2).reshape(*y.shape[:-3], d)
        h *= 2
    return y / math.sqrt(d)


class TurboQuant:
    """``bits``-bit Lloyd-Max codes of the randomly rotated vector + 1-bit QJL sketch of the residual."""

    def __init__(self, dim: int, bits: int = 3, seed: int = 0, device="cpu"):
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.dim, self.bits = dim, bits
        self.signs = (torch.randint(0, 2, (dim,), generator=g).float() * 2 - 1).to(device)
        self.jl = torch.randn(dim, dim, generator=g).to(device)                 # sketch matrix for the residual
        lv = torch.tensor(_LLOYD[bits])
        self.levels = torch.cat([-lv.flip(0), lv]).to(device)
        self.bounds = ((self.levels[1:] + self.levels[:-1]) / 2).to(device)

    def rotate(self, x):
        return hadamard(x.float() * self.signs)

    def unrotate(self, y):
        return hadamard(y) * self.signs

    def encode(self, x):
        """Returns ``(codes uint8[..., D], norm f32[..., 1], sketch bits bool[..., D], residual norm f32[..., 1])``."""
        n = x.float().norm(dim=-1, keepdim=True)
        n = torch.where(n > 0, n, torch.ones_like(n))
        y = self.rotate(x) / n * math.sqrt(self.dim)                              # ~ N(0, 1) coordinates
        codes = torch.bucketize(y, self.bounds).to(torch.uint8)
        rec = self.levels[codes.long()]
        r = y - rec
        rn = r.norm(dim=-1, keepdim=True)
        bits = (r @ self.jl.t()) >= 0
        return codes, n, bits, rn

    def decode(self, codes, n, bits=None, rn=None):
        y = self.levels[codes.long()]
        if bits is not None:
            # QJL estimate of the residual: E[sign(S r) S] = sqrt(2/pi) r / |r|
            s = bits.float() * 2 - 1
            y = y + (s @ self.jl) * (math.sqrt(math.pi / 2) / self.dim) * rn
        return self.unrotate(y * n / math.sqrt(self.dim))


class QuantizedKVCache:
    """Append-only per-layer cache holding K/V as int8 (or packed int4) codes with per-(token, head) scales."""

    def __init__(self, bits: int = 8):
        assert bits in (8, 4)
        self.bits = bits
        self.k, self.v = [], []

    def append(self, k, v):
        for dst, t in ((self.k, k), (self.v, v)):
            c, s = quantize_absmax(t, self.bits)
            dst.append((pack_int4(c) if self.bits == 4 else c, s))

    def _all(self, items):
        cs = torch.cat([unpack_int4(c) if self.bits == 4 else c for c, _ in items], 0)
        ss = torch.cat([s for _, s in items], 0)
        return dequantize_absmax(cs, ss)

    def keys(self):
        return self._all(self.k)

    def values(self):
        return self._all(self.v)

    def nbytes(self):
        return sum(c.numel() * c.element_size() + s.numel() * 4 for c, s in self.k + self.v)

"""Bit-exact FP4 codecs on the host (NumPy): E2M1 codes, E4M3 / E8M0 block scales, NVFP4 and MXFP4.

Rules (reference: src/models/inkling/nvfp4.rs:21-135, src/nn/mxfp4.rs:113-361,
src/models/inkling/fp4quant.rs:10-54,79-170):

* E2M1 magnitudes ``[0, .5, 1, 1.5, 2, 3, 4, 6]``, sign in bit 3; two codes per byte, the LOW nibble
  holds the lower index.
* NVFP4: ``value = E2M1[code] * E4M3(block scale, one per 16) * scale2`` (fp32 per tensor); the block
  scale is applied first.
* MXFP4: one E8M0 scale ``2^(e-127)`` per 32 elements, same codes.
* Activation quantiser: per 16 contiguous elements ``amax -> sf = min(amax/6, 448) -> E4M3 (round to
  nearest even) -> s = decode(sf)``; the code comes from the thresholds ``.25 .75 1.25 1.75 2.5 3.5 5`` on
  ``|x/s|`` with ``>=`` (ties away from zero); a negative input that rounds to zero keeps its sign
  (code 0x8); an all-zero block has scale byte 0 and codes 0.  There is no second-level scale.
* MXFP4 -> NVFP4 relabel is exact when the per-tensor exponent span fits E4M3's powers of two:
  ``global = 2^(e_max-8)``, every block scale becomes an exact power-of-two E4M3 and is duplicated for
  both 16-element halves; a wider span is refused.
"""
from __future__ import annotations

import numpy as np

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_SIGNED = np.concatenate([E2M1, -E2M1]).astype(np.float32)
_THRESH = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
E4M3_MAX = 448.0


# --------------------------------------------------------------------------- scale formats
def e4m3_decode(b: np.ndarray) -> np.ndarray:
    """E4M3 (fn variant: bias 7, no infinities, 0x7F/0xFF are NaN) -> float32."""
    b = np.asarray(b, dtype=np.uint8)
    s = np.where(b & 0x80, -1.0, 1.0).astype(np.float32)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 7).astype(np.float32)
    sub = (m / 8.0) * np.float32(2.0 ** -6)
    nor = (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float32))
    out = np.where(e == 0, sub, nor).astype(np.float32) * s
    return np.where((b & 0x7F) == 0x7F, np.float32(np.nan), out).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Non-negative float32 (<= 448) -> E4M3 byte, round to nearest even."""
    x = np.asarray(x, dtype=np.float32)
    if np.any(x < 0) or np.any(x > E4M3_MAX):
        raise ValueError("e4m3_encode expects values in [0, 448]")
    out = np.zeros(x.shape, dtype=np.uint8)
    # subnormal range: multiples of 2^-9 below 2^-6
    subn = x < np.float32(2.0 ** -6)
    q = np.rint(x.astype(np.float64) * 512.0).astype(np.int64)  # x / 2^-9, RNE
    out = np.where(subn, q.astype(np.uint8), out)               # q == 8 is exactly byte 0x08 (2^-6)
    mant, exp = np.frexp(x.astype(np.float64))                  # x = mant * 2^exp, mant in [0.5, 1)
    e = exp - 1
    frac = mant * 2.0 - 1.0
    m = np.rint(frac * 8.0).astype(np.int64)
    carry = m == 8
    e = np.where(carry, e + 1, e)
    m = np.where(carry, 0, m)
    byte = ((e + 7) << 3) | m
    byte = np.minimum(byte, 0x7E)
    return np.where(subn, out, byte.astype(np.uint8)).astype(np.uint8)


def e8m0_decode(b: np.ndarray) -> np.ndarray:
    return np.exp2(np.asarray(b, dtype=np.int32).astype(np.float32) - 127.0).astype(np.float32)


# --------------------------------------------------------------------------- codes
def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """uint8[..., k/2] -> uint8[..., k] codes (low nibble first)."""
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = p >> 4
    return out


def pack_codes(codes: np.ndarray) -> np.ndarray:
    c = np.asarray(codes, dtype=np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def decode_codes(packed: np.ndarray) -> np.ndarray:
    return E2M1_SIGNED[unpack_codes(packed)]


def encode_e2m1(y: np.ndarray) -> np.ndarray:
    """Scaled values -> 4-bit codes by the threshold rule (ties away from zero, signed zero kept)."""
    y = np.asarray(y, dtype=np.float32)
    mag = np.abs(y)
    code = np.zeros(y.shape, dtype=np.uint8)
    for t in _THRESH:
        code += (mag >= t).astype(np.uint8)
    return np.where(np.signbit(y), code | 8, code).astype(np.uint8)


# --------------------------------------------------------------------------- NVFP4
def decode_nvfp4(codes: np.ndarray, scales: np.ndarray, scale2: float = 1.0) -> np.ndarray:
    """``codes uint8[rows,k/2]``, ``scales E4M3 uint8[rows,k/16]`` -> float32 ``[rows,k]``."""
    v = decode_codes(codes)
    s = np.repeat(e4m3_decode(scales), 16, axis=-1)
    return ((v * s) * np.float32(scale2)).astype(np.float32)


def quantize_act_nvfp4(x: np.ndarray):
    """The activation quantiser (no second-level scale).  Returns ``(codes uint8[rows,k/2], scales uint8[rows,k/16])``."""
    x = np.asarray(x, dtype=np.float32)
    rows, k = x.shape
    if k % 16:
        raise ValueError("k must be a multiple of 16")
    blk = x.reshape(rows, k // 16, 16)
    amax = np.max(np.abs(blk), axis=-1)
    sf = np.minimum(amax / np.float32(6.0), np.float32(E4M3_MAX)).astype(np.float32)
    sb = e4m3_encode(sf)
    s = e4m3_decode(sb)
    safe = np.where(s > 0, s, np.float32(1.0))
    y = blk / safe[..., None]
    codes = encode_e2m1(y)
    zero = (s == 0)[..., None]
    codes = np.where(zero, np.uint8(0), codes).astype(np.uint8)
    return pack_codes(codes.reshape(rows, k)), sb.astype(np.uint8)


def quantize_weight_nvfp4(w: np.ndarray):
    """Weight quantiser: per-tensor ``scale2 = amax/(6*448)`` then the block rule on ``w/scale2``.
    Returns ``(codes, scales, scale2)``."""
    w = np.asarray(w, dtype=np.float32)
    amax = float(np.max(np.abs(w))) if w.size else 0.0
    scale2 = np.float32(amax / (6.0 * E4M3_MAX)) if amax > 0 else np.float32(1.0)
    codes, scales = quantize_act_nvfp4(w / scale2)
    return codes, scales, float(scale2)


# --------------------------------------------------------------------------- MXFP4
def decode_mxfp4(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    v = decode_codes(codes)
    s = np.repeat(e8m0_decode(scales), 32, axis=-1)
    return (v * s).astype(np.float32)


def quantize_mxfp4(w: np.ndarray):
    """Power-of-two block scales per 32 elements (E8M0), codes by the threshold rule."""
    w = np.asarray(w, dtype=np.float32)
    rows, k = w.shape
    blk = w.reshape(rows, k // 32, 32)
    amax = np.max(np.abs(blk), axis=-1)
    e = np.where(amax > 0, np.ceil(np.log2(np.maximum(amax, 1e-38) / 6.0)), -127.0)
    e = np.clip(e, -127, 127)
    sb = (e + 127).astype(np.uint8)
    y = blk / np.exp2(e.astype(np.float32))[..., None]
    return pack_codes(encode_e2m1(y).reshape(rows, k)), sb


class SpanError(ValueError):
    pass


def transcode_mxfp4_to_nvfp4(codes: np.ndarray, scales_e8m0: np.ndarray):
    """Exact relabel MXFP4 -> NVFP4 (src/nn/mxfp4.rs:296-340).  Returns ``(codes, e4m3 scales, scale2)``.

    ``global = 2^(e_max-8)``; block scale ``2^(e-127)`` becomes the E4M3 power of two ``2^(e-e_max+8)``,
    which exists for ``e >= e_max-17``.  Blocks below that are accepted only if all their codes are zero
    magnitudes; otherwise the span is refused."""
    sc = np.asarray(scales_e8m0, dtype=np.int32)
    cz = unpack_codes(codes).reshape(sc.shape + (32,)) & 7
    live = np.any(cz != 0, axis=-1)
    if not np.any(live):
        e_max = 127
    else:
        e_max = int(sc[live].max())
    rel = sc - e_max + 8                      # exponent of the E4M3 scale
    bad = live & (rel < -9)
    if np.any(bad):
        span = e_max - int(sc[live].min())
        raise SpanError(f"exponent span of {span} octaves exceeds the 17 that E4M3 powers of two cover")
    rel = np.clip(rel, -9, 8)
    # E4M3 byte of 2^rel: normal for rel >= -6 (exp field rel+7), subnormal below (mantissa 2^(rel+9))
    byte = np.where(rel >= -6, (rel + 7) << 3, 1 << np.maximum(rel + 9, 0)).astype(np.uint8)
    byte = np.where(live, byte, np.uint8(0))
    scale2 = float(np.exp2(np.float64(e_max - 8 - 127)))
    return np.asarray(codes, dtype=np.uint8), np.repeat(byte, 2, axis=-1), scale2


# --------------------------------------------------------------------------- scale layout for the tensor cores
def swizzle_scales_128x4(scales: np.ndarray) -> np.ndarray:
    """Row-major block scales ``[rows, nsf]`` -> the 512-byte tile layout that ``tcgen05.cp`` moves into
    TMEM: tiles of 128 rows x 4 scales, tile order (row tile, k tile) with k fastest, and inside a tile
    byte offset ``(r % 32) * 16 + (r // 32) * 4 + j``.  Rows and nsf are zero-padded to multiples of 128 / 4."""
    s = np.asarray(scales, dtype=np.uint8)
    rows, nsf = s.shape
    R, K = (rows + 127) // 128, (nsf + 3) // 4
    p = np.zeros((R * 128, K * 4), dtype=np.uint8)
    p[:rows, :nsf] = s
    t = p.reshape(R, 4, 32, K, 4)            # [R, r//32, r%32, K, j]
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(R, K, 512)

"""GGUF-style block quantisation (Q4_0, Q8_0) and the batch-1 matvec layers built on it.

Reference: src/nn/q4.rs:264-470 (``Q4Linear``, ``quantize_q4``, ``f16_matvec``).  Q4_0: 32 elements per block, scale
``d = m / -8`` where ``m`` is the element of largest magnitude (sign kept), ``q = clamp(round(x / d) + 8, 0, 15)``; element
``j`` of a block sits in the low nibble of byte ``j``, element ``j + 16`` in the high nibble.  Q8_0: ``d = max|x| / 127``."""
from __future__ import annotations

import numpy as np
import torch


def quantize_q4(w: np.ndarray) -> np.ndarray:
    """float ``[rows, cols]`` -> uint8 ``[rows, cols/32, 18]`` (f16 scale + 16 nibble bytes)."""
    w = np.asarray(w, dtype=np.float32)
    rows, cols = w.shape
    b = w.reshape(rows, cols // 32, 32)
    idx = np.abs(b).argmax(-1)
    m = np.take_along_axis(b, idx[..., None], -1)[..., 0]
    d = (m / -8.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0.0)
    q = np.clip(np.rint(b * inv[..., None]) + 8, 0, 15).astype(np.uint8)
    out = np.empty((rows, cols // 32, 18), dtype=np.uint8)
    out[..., :2] = d[..., None].view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out


def dequantize_q4(q: np.ndarray) -> np.ndarray:
    rows, nb, _ = q.shape
    d = np.ascontiguousarray(q[..., :2]).view(np.float16).astype(np.float32)[..., 0]
    qs = q[..., 2:]
    v = np.concatenate([(qs & 0xF).astype(np.float32) - 8, (qs >> 4).astype(np.float32) - 8], -1)
    return (v * d[..., None]).reshape(rows, nb * 32)


def quantize_q8(w: np.ndarray) -> np.ndarray:
    w = np.asarray(w, dtype=np.float32)
    rows, cols = w.shape
    b = w.reshape(rows, cols // 32, 32)
    d = (np.abs(b).max(-1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0.0)
    q = np.clip(np.rint(b * inv[..., None]), -127, 127).astype(np.int8)
    out = np.empty((rows, cols // 32, 34), dtype=np.uint8)
    out[..., :2] = d[..., None].view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out


def dequantize_q8(q: np.ndarray) -> np.ndarray:
    rows, nb, _ = q.shape
    d = np.ascontiguousarray(q[..., :2]).view(np.float16).astype(np.float32)[..., 0]
    return (np.ascontiguousarray(q[..., 2:]).view(np.int8).astype(np.float32) * d[..., None]).reshape(rows, nb * 32)


class QLinear:
    """Batch-1 linear layer over bf16 / Q8_0 / Q4_0 weights; ``swiglu=True`` treats the rows as [gate; up]."""

    FMT = {"bf16": 0, "q8": 1, "q4": 2}

    def __init__(self, weight: np.ndarray, fmt: str = "q4", device="cpu", swiglu: bool = False):
        self.fmt, self.swiglu = fmt, swiglu
        self.rows, self.cols = weight.shape
        if fmt == "q4":
            self.packed = torch.from_numpy(quantize_q4(weight)).to(device)
            self.dense = torch.from_numpy(dequantize_q4(self.packed.cpu().numpy()))
        elif fmt == "q8":
            self.packed = torch.from_numpy(quantize_q8(weight)).to(device)
            self.dense = torch.from_numpy(dequantize_q8(self.packed.cpu().numpy()))
        else:
            self.packed = torch.from_numpy(np.asarray(weight, dtype=np.float32)).to(torch.bfloat16).to(device)
            self.dense = self.packed.float().cpu()

    def __call__(self, x):
        out_rows = self.rows // 2 if self.swiglu else self.rows
        if x.is_cuda:
            from ..ops.cuda import _p, _stream, check, declare, lib
            declare("mary_matvec", "pippiiis")
            y = torch.empty(out_rows, dtype=torch.bfloat16, device=x.device)
            check(lib().mary_matvec(_p(self.packed), self.FMT[self.fmt], _p(x.to(torch.bfloat16).contiguous()), _p(y), out_rows, self.cols,
                                    1 if self.swiglu else 0, _stream()), "matvec")
            return y
        y = self.dense @ x.float().cpu()
        if self.swiglu:
            y = torch.nn.functional.silu(y[:out_rows]) * y[out_rows:]
        return y.to(x.dtype)

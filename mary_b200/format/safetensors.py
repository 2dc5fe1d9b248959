"""Minimal safetensors reader/writer (mmap, zero-copy) — import source and LoRA/PEFT export target.

File = ``u64 header_len | JSON header | raw little-endian tensor data``; the header maps a tensor name to
``{"dtype", "shape", "data_offsets"}``."""
from __future__ import annotations

import json
import mmap
import struct

import numpy as np

_DT = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "F64": np.float64, "I64": np.int64,
       "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_RDT = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.float64): "F64",
        np.dtype(np.int64): "I64", np.dtype(np.int32): "I32", np.dtype(np.uint8): "U8"}


class SafeTensors:
    def __init__(self, path: str):
        self.path = str(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._mm[:8])
        self.header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n

    def keys(self):
        return list(self.header.keys())

    def info(self, name: str):
        h = self.header[name]
        return h["dtype"], tuple(h["shape"])

    def raw(self, name: str) -> tuple[str, tuple, memoryview]:
        h = self.header[name]
        a, b = h["data_offsets"]
        return h["dtype"], tuple(h["shape"]), memoryview(self._mm)[self._base + a:self._base + b]

    def array(self, name: str) -> np.ndarray:
        dt, shape, mv = self.raw(name)
        return np.frombuffer(mv, dtype=_DT[dt]).reshape(shape)

    def f32(self, name: str) -> np.ndarray | None:
        """bf16/f16/f64 -> f32 (src/nn/weight_loader.rs:31-59); ``None`` for non-float tensors."""
        dt, shape, mv = self.raw(name)
        if dt == "F32":
            return np.frombuffer(mv, dtype=np.float32).reshape(shape)
        if dt == "F16":
            return np.frombuffer(mv, dtype=np.float16).reshape(shape).astype(np.float32)
        if dt == "F64":
            return np.frombuffer(mv, dtype=np.float64).reshape(shape).astype(np.float32)
        if dt == "BF16":
            return (np.frombuffer(mv, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(shape)
        return None

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass  # views are still alive; the mapping goes away with them
        self._f.close()


def save_file(tensors: dict, path: str, metadata: dict | None = None, bf16: set | None = None) -> None:
    """Write NumPy arrays; names in ``bf16`` hold uint16 bit patterns and are labelled BF16."""
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        dt = "BF16" if (bf16 and name in bf16) else _RDT[a.dtype]
        b = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)

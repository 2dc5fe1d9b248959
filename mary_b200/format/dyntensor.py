"""``DynTensor``: a self-describing tensor blob — one blob kind for any rank, dtype and shape, readable without a schema.

Wire layout (little-endian), as in the reference (src/models/gemma/dyntensor.rs:7-16): ``magic u32 "DTNS" = 0x534E5444``,
``dtype tag u8``, ``rank u8``, two reserved bytes, ``rank`` dims as ``u32``, zero padding up to the dtype's alignment, then the
data.  The tag numbering is the reference's (src/models/gemma/dyntensor.rs:35-52): f32 0, bf16 1, f16 2, f64 3, flex32 4, i64 5,
i32 6, i16 7, i8 8, u64 9, u32 10, u16 11, u8 12, bool 13.  Decoding is zero-copy: the returned array / tensor aliases the blob
(a pile hands out memory-mapped buffers, so a decoded tensor costs no copy until it moves to a device)."""
from __future__ import annotations

import struct

import numpy as np

MAGIC = 0x534E5444
HEADER_BASE = 8

_TAGS = {0: "f32", 1: "bf16", 2: "f16", 3: "f64", 4: "flex32", 5: "i64", 6: "i32", 7: "i16", 8: "i8", 9: "u64", 10: "u32", 11: "u16",
         12: "u8", 13: "bool"}
_NP = {"f32": np.float32, "f16": np.float16, "f64": np.float64, "flex32": np.float32, "i64": np.int64, "i32": np.int32, "i16": np.int16,
       "i8": np.int8, "u64": np.uint64, "u32": np.uint32, "u16": np.uint16, "u8": np.uint8, "bool": np.bool_, "bf16": np.uint16}
_TAG_OF = {v: k for k, v in _TAGS.items()}


class DynTensorError(ValueError):
    pass


def _align(name: str) -> int:
    return np.dtype(_NP[name]).itemsize


def encode(array, dtype: str | None = None) -> bytes:
    """``array``: a NumPy array, or a torch tensor (bf16 tensors keep their bit pattern).  ``dtype`` overrides the tag (e.g.
    ``"bf16"`` for a ``uint16`` array of bf16 bits)."""
    name = dtype
    try:
        import torch
        if isinstance(array, torch.Tensor):
            t = array.detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                array, name = t.view(torch.uint16).numpy(), name or "bf16"
            else:
                array = t.numpy()
    except ImportError:
        pass
    a = np.asarray(array)
    if not a.flags.c_contiguous:
        a = a.copy(order="C")
    if name is None:
        name = {np.dtype(v): k for k, v in _NP.items() if k not in ("flex32", "bf16")}.get(a.dtype)
    if name not in _TAG_OF:
        raise DynTensorError(f"unsupported dtype {a.dtype}")
    if np.dtype(_NP[name]).itemsize != a.dtype.itemsize:
        raise DynTensorError(f"dtype tag {name} does not match the {a.dtype.itemsize}-byte elements given")
    if a.ndim > 255 or any(d >= 1 << 32 for d in a.shape):
        raise DynTensorError("rank or dimension out of range")
    head = struct.pack("<IBBH", MAGIC, _TAG_OF[name], a.ndim, 0) + struct.pack(f"<{a.ndim}I", *a.shape)
    pad = (-len(head)) % _align(name)
    return head + b"\0" * pad + a.tobytes()


def header(blob) -> tuple[str, tuple[int, ...], int]:
    """``(dtype name, shape, data offset)`` of a blob; raises on a bad magic, tag, or a length that does not match the shape."""
    mv = memoryview(blob)
    if len(mv) < HEADER_BASE:
        raise DynTensorError("blob shorter than the header")
    magic, tag, rank, _ = struct.unpack_from("<IBBH", mv, 0)
    if magic != MAGIC:
        raise DynTensorError(f"bad magic {magic:#x}")
    if tag not in _TAGS:
        raise DynTensorError(f"unknown dtype tag {tag}")
    if len(mv) < HEADER_BASE + 4 * rank:
        raise DynTensorError("blob shorter than its dims")
    shape = struct.unpack_from(f"<{rank}I", mv, HEADER_BASE)
    name = _TAGS[tag]
    off = HEADER_BASE + 4 * rank
    off += (-off) % _align(name)
    n = int(np.prod(shape, dtype=np.int64)) if rank else 1
    if len(mv) - off != n * _align(name):
        raise DynTensorError(f"payload of {len(mv) - off} bytes does not hold {n} {name} elements")
    return name, tuple(int(d) for d in shape), off


def decode(blob) -> tuple[np.ndarray, str]:
    """Zero-copy view ``(array, dtype name)``; bf16 comes back as its ``uint16`` bits (see ``decode_torch``)."""
    name, shape, off = header(blob)
    a = np.frombuffer(blob, dtype=_NP[name], offset=off, count=int(np.prod(shape, dtype=np.int64)) if shape else 1)
    return a.reshape(shape), name


def decode_torch(blob):
    import torch
    a, name = decode(blob)
    if not a.flags.writeable:
        a = a.copy() if a.size == 0 else a               # torch warns on read-only buffers; the view is kept (never written)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        t = torch.from_numpy(a)
    return t.view(torch.bfloat16) if name == "bf16" else t

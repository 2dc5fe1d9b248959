"""Typed tensor leaves: ONE blob per tensor, with the dims in the blob header.

Reference: src/leaf.rs.  A leaf entity carries exactly one payload attribute.  In the typed form the
attribute id is derived from ``(anchor, element, rank)`` (:51-61) and the value is the handle of a
``Tensor<Elem, RANK>`` blob; the legacy form is two blobs, ``data`` (f32 or f16 payload) plus ``shape``
(u64 dims).  ``resolve`` reads the typed form first, then the legacy one, and refuses an entity that has
two payloads (:336-461).  Ranks 0..=6 are accepted; rank 7 and above are refused rather than flattened
(:272-297).  The entity id is derived from the content handle, so identical tensors dedupe (:299-312).

Blob layout used here (little endian): a 256-byte header ``"MTNS" | elem u32 | rank u32 | reserved u32 |
dims u64[6] | payload_bytes u64`` followed by the payload, so that the payload of a blob stored in a pile
(whose blobs start at 256-byte aligned offsets) is itself 256-byte aligned for direct H2D copies.

Elements beyond the reference's F32/F16: BF16, and the block-scaled FP4 containers
``NVFP4 = [codes rows*k/2 B][E4M3 scales rows*k/16 B][scale2 f32]`` with LOGICAL dims ``[rows, k]``
(src/models/inkling/pile.rs:343-399) and ``MXFP4 = [codes rows*k/2 B][E8M0 scales rows*k/32 B]``.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from enum import IntEnum

import numpy as np

from ..pile.trible import TribleBuilder, TribleSet, content_id, derived_id, v_handle
from . import schema as S

MAX_RANK = 6
HEADER = 256
_MAGIC = b"MTNS"


class Elem(IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 2
    NVFP4 = 3
    MXFP4 = 4
    I32 = 5
    I64 = 6
    U8 = 7


_NP = {Elem.F32: np.float32, Elem.F16: np.float16, Elem.BF16: np.uint16, Elem.I32: np.int32,
       Elem.I64: np.int64, Elem.U8: np.uint8}


class LeafError(ValueError):
    pass


def leaf_attr(elem: Elem, rank: int) -> bytes:
    return derived_id(S.LEAF_ANCHOR, bytes([int(elem)]), bytes([rank]))


_ATTR_TABLE = {leaf_attr(e, r): (e, r) for e in Elem for r in range(MAX_RANK + 1)}


def payload_bytes(elem: Elem, dims: tuple[int, ...]) -> int:
    n = 1
    for d in dims:
        n *= int(d)
    if elem == Elem.NVFP4:
        if len(dims) != 2 or dims[1] % 16:
            raise LeafError("NVFP4 leaves are rank 2 with k % 16 == 0")
        return n // 2 + n // 16 + 4
    if elem == Elem.MXFP4:
        if len(dims) != 2 or dims[1] % 32:
            raise LeafError("MXFP4 leaves are rank 2 with k % 32 == 0")
        return n // 2 + n // 32
    return n * np.dtype(_NP[elem]).itemsize


def tensor_blob(elem: Elem, dims, payload) -> bytes:
    dims = tuple(int(d) for d in dims)
    if len(dims) > MAX_RANK:
        raise LeafError(f"rank {len(dims)} exceeds the ranks this format stores (0..={MAX_RANK}); "
                        "refusing rather than flattening")
    mv = memoryview(payload).cast("B")
    want = payload_bytes(elem, dims)
    if len(mv) != want:
        raise LeafError(f"payload is {len(mv)} bytes, dims {dims} of {elem.name} need {want}")
    hdr = _MAGIC + struct.pack("<III", int(elem), len(dims), 0)
    hdr += struct.pack("<6Q", *(dims + (0,) * (6 - len(dims)))) + struct.pack("<Q", want)
    return hdr.ljust(HEADER, b"\x00") + bytes(mv)


@dataclass
class Leaf:
    """A resolved leaf: element type, dims and a zero-copy view of its payload."""
    elem: Elem
    dims: tuple[int, ...]
    payload: memoryview
    handle: bytes

    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def array(self) -> np.ndarray:
        """Zero-copy NumPy view (BF16 comes back as uint16 bit patterns)."""
        if self.elem in (Elem.NVFP4, Elem.MXFP4):
            raise LeafError("block-scaled leaves have no flat array view; use fp4_parts()")
        return np.frombuffer(self.payload, dtype=_NP[self.elem]).reshape(self.dims)

    def view_f32(self) -> np.ndarray:
        if self.elem != Elem.F32:
            raise LeafError(f"leaf is {self.elem.name}, not F32")
        return self.array()

    def view_f16(self) -> np.ndarray:
        if self.elem != Elem.F16:
            raise LeafError(f"leaf is {self.elem.name}, not F16")
        return self.array()

    def to_f32(self) -> np.ndarray:
        if self.elem == Elem.F32:
            return self.array()
        if self.elem == Elem.F16:
            return self.array().astype(np.float32)
        if self.elem == Elem.BF16:
            return (self.array().astype(np.uint32) << 16).view(np.float32)
        if self.elem == Elem.NVFP4:
            from ..nn.nvfp4 import decode_nvfp4
            codes, scales, scale2 = self.fp4_parts()
            return decode_nvfp4(codes, scales, scale2)
        if self.elem == Elem.MXFP4:
            from ..nn.mxfp4 import decode_mxfp4
            codes, scales, _ = self.fp4_parts()
            return decode_mxfp4(codes, scales)
        return self.array().astype(np.float32)

    def fp4_parts(self):
        """``(codes uint8[rows,k/2], scales uint8[rows,k/blk], scale2 float|None)`` of a block-scaled leaf."""
        rows, k = self.dims
        buf = np.frombuffer(self.payload, dtype=np.uint8)
        nc = rows * k // 2
        if self.elem == Elem.NVFP4:
            ns = rows * k // 16
            scale2 = float(np.frombuffer(self.payload[nc + ns:nc + ns + 4], dtype=np.float32)[0])
            return buf[:nc].reshape(rows, k // 2), buf[nc:nc + ns].reshape(rows, k // 16), scale2
        if self.elem == Elem.MXFP4:
            ns = rows * k // 32
            return buf[:nc].reshape(rows, k // 2), buf[nc:nc + ns].reshape(rows, k // 32), None
        raise LeafError("not a block-scaled leaf")

    def torch(self):
        """Zero-copy torch view over the mapping (read-only memory: clone before writing)."""
        import torch
        import warnings
        if self.elem == Elem.BF16:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                return torch.frombuffer(self.payload, dtype=torch.bfloat16).reshape(self.dims)
        if self.elem in (Elem.NVFP4, Elem.MXFP4):
            raise LeafError("use fp4_parts() for block-scaled leaves")
        dt = {Elem.F32: torch.float32, Elem.F16: torch.float16, Elem.I32: torch.int32, Elem.I64: torch.int64,
              Elem.U8: torch.uint8}[self.elem]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            return torch.frombuffer(self.payload, dtype=dt).reshape(self.dims)


def read_blob(blob, handle: bytes = b"") -> Leaf:
    mv = memoryview(blob).cast("B")
    if len(mv) < HEADER or bytes(mv[:4]) != _MAGIC:
        raise LeafError("not a tensor blob")
    elem, rank, _ = struct.unpack("<III", mv[4:16])
    if rank > MAX_RANK:
        raise LeafError(f"tensor blob claims rank {rank}")
    dims = struct.unpack("<6Q", mv[16:64])[:rank]
    (nbytes,) = struct.unpack("<Q", mv[64:72])
    e = Elem(elem)
    if nbytes != payload_bytes(e, dims) or len(mv) != HEADER + nbytes:
        raise LeafError("tensor blob length does not match its header")
    return Leaf(e, tuple(int(d) for d in dims), mv[HEADER:], handle)


def put_leaf(store, tb: TribleBuilder, elem: Elem, dims, payload, id: bytes | None = None) -> bytes:
    """Store one tensor as a typed leaf; the blob is decoded again and compared before it is written
    (src/leaf.rs:238-259).  Returns the leaf entity id (content-derived unless ``id`` is given)."""
    blob = tensor_blob(elem, dims, payload)
    back = read_blob(blob)
    if back.dims != tuple(int(d) for d in dims) or bytes(back.payload) != bytes(memoryview(payload).cast("B")):
        raise LeafError("typed leaf did not round-trip its own bytes")
    h = store.put(blob)
    return tb.entity([(leaf_attr(elem, len(back.dims)), v_handle(h))], id=id)


def put_leaf_legacy(store, tb: TribleBuilder, arr: np.ndarray, f16: bool = False, id: bytes | None = None) -> bytes:
    """Legacy two-blob leaf: ``data`` (or ``data_f16``) + ``shape`` (src/format.rs:141-177)."""
    a = np.ascontiguousarray(arr, dtype=np.float16 if f16 else np.float32)
    hd = store.put(a.tobytes())
    hs = store.put(np.asarray(a.shape, dtype=np.uint64).tobytes())
    return tb.entity([(S.DATA_F16 if f16 else S.DATA, v_handle(hd)), (S.SHAPE, v_handle(hs))], id=id)


def put_array(store, tb: TribleBuilder, arr, elem: Elem | None = None, id: bytes | None = None) -> bytes:
    """Convenience: store a NumPy array (float32/float16/int32/int64/uint8, or uint16 bit patterns as BF16)."""
    a = np.ascontiguousarray(arr)
    if elem is None:
        elem = {np.dtype(np.float32): Elem.F32, np.dtype(np.float16): Elem.F16, np.dtype(np.int32): Elem.I32,
                np.dtype(np.int64): Elem.I64, np.dtype(np.uint8): Elem.U8, np.dtype(np.uint16): Elem.BF16}[a.dtype]
    return put_leaf(store, tb, elem, a.shape, a.tobytes() if a.size else b"", id=id)


def resolve(store, facts: TribleSet, entity: bytes) -> Leaf:
    """Read a leaf entity: typed first, legacy second; two payloads are an error (src/leaf.rs:336-461)."""
    typed, legacy, shape = [], [], None
    for a, v in facts.of_entity(entity):
        if a in _ATTR_TABLE:
            typed.append((a, v))
        elif a in (S.DATA, S.DATA_F16):
            legacy.append((a, v))
        elif a == S.SHAPE:
            shape = v
    if len(typed) + len(legacy) != 1:
        raise LeafError(f"leaf {entity.hex()} has {len(typed) + len(legacy)} payloads, expected exactly 1")
    if typed:
        a, h = typed[0]
        leaf = read_blob(store.get(h), h)
        e, r = _ATTR_TABLE[a]
        if leaf.elem != e or len(leaf.dims) != r:
            raise LeafError(f"leaf {entity.hex()}: blob is {leaf.elem.name} rank {len(leaf.dims)}, "
                            f"attribute says {e.name} rank {r}")
        return leaf
    if shape is None:
        raise LeafError(f"legacy leaf {entity.hex()} has no shape")
    a, h = legacy[0]
    dims = tuple(int(d) for d in np.frombuffer(store.get(shape), dtype=np.uint64))
    e = Elem.F16 if a == S.DATA_F16 else Elem.F32
    payload = store.get(h)
    if len(payload) != payload_bytes(e, dims):
        raise LeafError(f"legacy leaf {entity.hex()}: payload does not match shape {dims}")
    return Leaf(e, dims, payload, h)


def is_leaf(facts: TribleSet, entity: bytes) -> bool:
    return any(a in _ATTR_TABLE or a in (S.DATA, S.DATA_F16) for a, _ in facts.of_entity(entity))

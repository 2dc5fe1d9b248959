"""Tribles: 64-byte facts ``(entity 16 B, attribute 16 B, value 32 B)`` and sets of them.

This is the fact model that the reference takes from the external ``triblespace`` crate
(usage: src/format.rs:52, src/persist.rs:1613-1618, src/ingest.rs:156-176):

* ids are 16 bytes, written as 32 hex digits; values are always 32 bytes (a value schema
  says how to read them);
* ``entity({...})`` derives the entity id from the entity's own attribute/value pairs, so
  the same content always gets the same id and identical tensors dedupe across models
  (src/leaf.rs:299-312);
* a set is canonical (sorted, unique) and its archive form is the plain concatenation of
  its tribles, so equal sets hash to the same blob.

Sets are NumPy ``uint8[N, 64]`` arrays; queries go through lazily built sorted indexes.
"""
from __future__ import annotations

import os
import struct
from typing import Iterable, Iterator

import numpy as np

from .hashing import blake3

ID_LEN, VALUE_LEN, TRIBLE_LEN = 16, 32, 64


# --------------------------------------------------------------------------- ids
def id_hex(h: str) -> bytes:
    b = bytes.fromhex(h)
    if len(b) != ID_LEN:
        raise ValueError(f"id must be 32 hex digits, got {h!r}")
    return b


def fresh_id() -> bytes:
    """Random id with a non-zero first byte (the all-zero id is reserved as 'no id')."""
    while True:
        b = os.urandom(ID_LEN)
        if any(b):
            return b


def derived_id(*parts: bytes) -> bytes:
    """Deterministic id from byte strings (used for attribute ids that are functions of
    an anchor id plus parameters, e.g. the typed-leaf attribute: src/leaf.rs:51-61)."""
    return blake3(b"".join(struct.pack("<I", len(p)) + p for p in parts))[:ID_LEN]


# --------------------------------------------------------------------------- value schemas
def v_genid(i: bytes) -> bytes:
    assert len(i) == ID_LEN
    return bytes(16) + i


def r_genid(v: bytes) -> bytes:
    return bytes(v[16:32])


def v_shortstring(s: str) -> bytes:
    b = s.encode("utf-8")
    if len(b) > VALUE_LEN or b"\x00" in b:
        raise ValueError(f"short string must be <= 32 bytes without NUL: {s!r}")
    return b + bytes(VALUE_LEN - len(b))


def r_shortstring(v: bytes) -> str:
    return bytes(v).rstrip(b"\x00").decode("utf-8")


def v_u256(n: int) -> bytes:
    return int(n).to_bytes(32, "big", signed=False)


def r_u256(v: bytes) -> int:
    return int.from_bytes(bytes(v), "big", signed=False)


def v_i256(n: int) -> bytes:
    return int(n).to_bytes(32, "big", signed=True)


def r_i256(v: bytes) -> int:
    return int.from_bytes(bytes(v), "big", signed=True)


def v_f64(x: float) -> bytes:
    return struct.pack("<d", float(x)) + bytes(24)


def r_f64(v: bytes) -> float:
    return struct.unpack("<d", bytes(v[:8]))[0]


def v_bool(b: bool) -> bytes:
    return bytes(31) + (b"\x01" if b else b"\x00")


def r_bool(v: bytes) -> bool:
    return bytes(v)[31] != 0


def v_handle(h: bytes) -> bytes:
    assert len(h) == VALUE_LEN
    return bytes(h)


# --------------------------------------------------------------------------- sets
def _canon(arr: np.ndarray) -> np.ndarray:
    """Sort rows lexicographically and drop duplicates."""
    if arr.shape[0] <= 1:
        return np.ascontiguousarray(arr)
    keys = np.ascontiguousarray(arr).view(">u8").reshape(arr.shape[0], 8)
    order = np.lexsort(keys[:, ::-1].T)
    s = arr[order]
    keep = np.ones(s.shape[0], dtype=bool)
    keep[1:] = np.any(s[1:] != s[:-1], axis=1)
    return np.ascontiguousarray(s[keep])


class TribleSet:
    """Immutable canonical set of tribles."""

    __slots__ = ("data", "_by_attr", "_by_entity")

    def __init__(self, data: np.ndarray | None = None, _canonical: bool = False):
        if data is None:
            data = np.zeros((0, TRIBLE_LEN), dtype=np.uint8)
        data = np.asarray(data, dtype=np.uint8).reshape(-1, TRIBLE_LEN)
        self.data = data if _canonical else _canon(data)
        self._by_attr = None
        self._by_entity = None

    # construction ---------------------------------------------------------
    @staticmethod
    def from_tribles(tribles: Iterable[bytes]) -> "TribleSet":
        buf = b"".join(tribles)
        if len(buf) % TRIBLE_LEN:
            raise ValueError("trible bytes are not a multiple of 64")
        return TribleSet(np.frombuffer(buf, dtype=np.uint8).reshape(-1, TRIBLE_LEN).copy())

    @staticmethod
    def from_archive(blob) -> "TribleSet":
        a = np.frombuffer(blob, dtype=np.uint8)
        if a.size % TRIBLE_LEN:
            raise ValueError("archive length is not a multiple of 64")
        return TribleSet(a.reshape(-1, TRIBLE_LEN).copy())

    def archive(self) -> bytes:
        return self.data.tobytes()

    def __len__(self) -> int:
        return int(self.data.shape[0])

    def __or__(self, other: "TribleSet") -> "TribleSet":
        if len(other) == 0:
            return self
        if len(self) == 0:
            return other
        return TribleSet(np.concatenate([self.data, other.data], axis=0))

    @staticmethod
    def union(sets: Iterable["TribleSet"]) -> "TribleSet":
        arrs = [s.data for s in sets if len(s)]
        if not arrs:
            return TribleSet()
        return TribleSet(np.concatenate(arrs, axis=0))

    def __eq__(self, other) -> bool:
        return isinstance(other, TribleSet) and self.data.shape == other.data.shape and bool(
            np.array_equal(self.data, other.data))

    def __iter__(self) -> Iterator[tuple[bytes, bytes, bytes]]:
        for row in self.data:
            b = row.tobytes()
            yield b[:16], b[16:32], b[32:]

    # indexes ----------------------------------------------------------------
    def _attr_index(self):
        if self._by_attr is None:
            idx: dict[bytes, np.ndarray] = {}
            if len(self):
                a = np.ascontiguousarray(self.data[:, 16:32]).view(">u8").reshape(-1, 2)
                order = np.lexsort((a[:, 1], a[:, 0]))
                sa = a[order]
                brk = np.flatnonzero(np.any(sa[1:] != sa[:-1], axis=1)) + 1
                starts = np.concatenate([[0], brk])
                ends = np.concatenate([brk, [len(order)]])
                for s, e in zip(starts, ends):
                    idx[self.data[order[s], 16:32].tobytes()] = order[s:e]
            self._by_attr = idx
        return self._by_attr

    def _entity_index(self):
        if self._by_entity is None:
            idx: dict[bytes, np.ndarray] = {}
            if len(self):
                # rows are sorted by entity first
                e = np.ascontiguousarray(self.data[:, :16]).view(">u8").reshape(-1, 2)
                brk = np.flatnonzero(np.any(e[1:] != e[:-1], axis=1)) + 1
                starts = np.concatenate([[0], brk])
                ends = np.concatenate([brk, [len(self)]])
                for s, en in zip(starts, ends):
                    idx[self.data[s, :16].tobytes()] = np.arange(s, en)
            self._by_entity = idx
        return self._by_entity

    # queries ----------------------------------------------------------------
    def with_attr(self, attr: bytes) -> list[tuple[bytes, bytes]]:
        """All ``(entity, value)`` pairs that carry ``attr``."""
        rows = self._attr_index().get(attr)
        if rows is None:
            return []
        out = []
        for r in rows:
            b = self.data[r].tobytes()
            out.append((b[:16], b[32:]))
        return out

    def of_entity(self, entity: bytes) -> list[tuple[bytes, bytes]]:
        """All ``(attribute, value)`` pairs of ``entity``."""
        rows = self._entity_index().get(entity)
        if rows is None:
            return []
        out = []
        for r in rows:
            b = self.data[r].tobytes()
            out.append((b[16:32], b[32:]))
        return out

    def values(self, entity: bytes, attr: bytes) -> list[bytes]:
        return [v for a, v in self.of_entity(entity) if a == attr]

    def one(self, entity: bytes, attr: bytes) -> bytes:
        """Exactly one value, else an error (selection is exact-cardinality: src/selection.rs:173-257)."""
        vs = self.values(entity, attr)
        if len(vs) != 1:
            raise LookupError(f"entity {entity.hex()} has {len(vs)} values for attribute {attr.hex()}, expected 1")
        return vs[0]

    def maybe(self, entity: bytes, attr: bytes) -> bytes | None:
        vs = self.values(entity, attr)
        if len(vs) > 1:
            raise LookupError(f"entity {entity.hex()} has {len(vs)} values for attribute {attr.hex()}, expected <= 1")
        return vs[0] if vs else None

    def entities_where(self, attr: bytes, value: bytes) -> list[bytes]:
        return [e for e, v in self.with_attr(attr) if v == value]

    def find(self, pattern: list[tuple]) -> list[dict]:
        """Conjunctive query.  ``pattern`` is a list of ``(e, a, v)`` where ``a`` is a constant id and
        ``e``/``v`` are constants (bytes) or variable names (str).  Returns variable bindings."""
        results: list[dict] = [{}]
        for e, a, v in pattern:
            nxt = []
            pairs = self.with_attr(a)
            for b in results:
                ev = b.get(e, None) if isinstance(e, str) else e
                vv = b.get(v, None) if isinstance(v, str) else v
                for pe, pv in pairs:
                    if ev is not None and pe != ev:
                        continue
                    if vv is not None:
                        want = vv if len(vv) == VALUE_LEN else v_genid(vv)
                        if pv != want:
                            continue
                    nb = dict(b)
                    if isinstance(e, str) and ev is None:
                        nb[e] = pe
                    if isinstance(v, str) and vv is None:
                        nb[v] = pv
                    nxt.append(nb)
            results = nxt
            if not results:
                break
        return results


class TribleBuilder:
    """Mutable accumulator; ``entity()`` mirrors the reference's ``entity!{ _ @ a: v }``."""

    def __init__(self):
        self._rows: list[bytes] = []

    def add(self, e: bytes, a: bytes, v: bytes) -> None:
        if len(e) != ID_LEN or len(a) != ID_LEN or len(v) != VALUE_LEN:
            raise ValueError("trible fields must be 16/16/32 bytes")
        self._rows.append(e + a + v)

    def entity(self, pairs: list[tuple[bytes, bytes]], id: bytes | None = None) -> bytes:
        """Add an entity.  Without ``id`` the id is derived from the sorted attribute/value pairs
        (content-derived: src/ingest.rs:156-176); with ``id`` the pairs are attached to that id
        (non-identity labels: src/ingest.rs:195-203)."""
        if id is None:
            id = content_id(pairs)
        for a, v in pairs:
            self.add(id, a, v)
        return id

    def extend(self, ts: TribleSet) -> None:
        self._rows.append(ts.data.tobytes())

    def build(self) -> TribleSet:
        buf = b"".join(self._rows)
        return TribleSet(np.frombuffer(buf, dtype=np.uint8).reshape(-1, TRIBLE_LEN).copy()) if buf else TribleSet()

    def __len__(self):
        return sum(len(r) for r in self._rows) // TRIBLE_LEN


def content_id(pairs: list[tuple[bytes, bytes]]) -> bytes:
    body = b"".join(a + v for a, v in sorted(pairs))
    i = blake3(b"entity\x00" + body)[:ID_LEN]
    return i if any(i) else b"\x01" + i[1:]

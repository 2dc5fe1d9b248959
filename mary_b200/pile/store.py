"""Blob stores: the on-disk ``Pile`` (native, mmap'd, append-only) and an in-memory twin for tests.

The reference uses the external TribleSpace ``Pile`` (src/persist.rs:744-799) and a
``MemoryBlobStore`` fixture in its unit tests (src/leaf.rs:687-770); both roles are covered here
behind one small interface: ``put(bytes) -> handle``, ``get(handle) -> memoryview``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from .hashing import blake3

KIND_BLOB, KIND_BRANCH = 1, 2


class PileError(RuntimeError):
    pass


@dataclass
class Record:
    index: int
    kind: int
    offset: int
    length: int
    timestamp_ns: int
    hash: bytes
    branch: bytes


def _as_buffer(data):
    """Return (ctypes-passable object, length, keepalive)."""
    if isinstance(data, bytes):
        return data, len(data), data
    arr = np.frombuffer(memoryview(data).cast("B"), dtype=np.uint8)
    return ctypes.c_void_p(arr.ctypes.data), arr.size, arr


class MemoryBlobStore:
    """Dict-backed store with the same interface as :class:`Pile`."""

    def __init__(self):
        self._blobs: dict[bytes, bytes] = {}
        self._branches: list[tuple[bytes, bytes]] = []
        self.bytes_put = 0
        self.bytes_dedup = 0

    def put(self, data) -> bytes:
        b = bytes(memoryview(data).cast("B"))
        h = blake3(b)
        if h in self._blobs:
            self.bytes_dedup += len(b)
        else:
            self._blobs[h] = b
            self.bytes_put += len(b)
        return h

    def get(self, handle: bytes) -> memoryview:
        try:
            return memoryview(self._blobs[bytes(handle)])
        except KeyError:
            raise PileError(f"blob {bytes(handle).hex()} is not in the store") from None

    def has(self, handle: bytes) -> bool:
        return bytes(handle) in self._blobs

    def put_branch(self, branch_id: bytes, payload: bytes) -> None:
        self._branches.append((bytes(branch_id), bytes(payload)))

    def branch_records(self):
        return list(self._branches)

    def flush(self):
        pass

    def refresh(self):
        pass

    def close(self):
        pass


class Pile:
    """Append-only content-addressed file.  Blobs come back as zero-copy views of the mapping, whose
    file offsets are 256-byte aligned."""

    def __init__(self, path: str, create: bool = True, validate: bool = True):
        from .. import _native
        self._lib = _native.core()
        self.path = str(path)
        self._h = self._lib.pile_open(self.path.encode(), 1 if create else 0, 1 if validate else 0)
        if not self._h:
            raise PileError(f"cannot open pile {self.path}")
        err = self._lib.pile_error(self._h).decode()
        if err:
            self._lib.pile_close(self._h)
            self._h = None
            raise PileError(f"{self.path}: {err}; the file is left untouched — run Pile.amputate(path) to cut the torn tail")
        self._base = self._lib.pile_base(self._h)

    @staticmethod
    def open(path: str, create: bool = True, validate: bool = True) -> "Pile":
        return Pile(path, create, validate)

    @staticmethod
    def amputate(path: str) -> int:
        """Explicit repair of a torn tail; returns the number of bytes cut."""
        from .. import _native
        n = _native.core().pile_amputate(str(path).encode())
        if n < 0:
            raise PileError(f"cannot amputate {path}")
        return int(n)

    # -- blob interface
    def put(self, data) -> bytes:
        buf, n, keep = _as_buffer(data)
        out = (ctypes.c_uint8 * 32)()
        idx = self._lib.pile_put(self._h, KIND_BLOB, buf, n, None, out)
        if idx < 0:
            raise PileError(f"{self.path}: put failed: {self._lib.pile_error(self._h).decode()}")
        return bytes(out)

    def get(self, handle: bytes) -> memoryview:
        ptr = ctypes.c_void_p()
        n = ctypes.c_uint64()
        rc = self._lib.pile_get(self._h, bytes(handle), ctypes.byref(ptr), ctypes.byref(n))
        if rc == -1:
            raise PileError(f"blob {bytes(handle).hex()} is not in {self.path}")
        if rc == -2:
            raise PileError(f"blob {bytes(handle).hex()} in {self.path} fails its BLAKE3 check")
        if n.value == 0:
            return memoryview(b"")
        arr = (ctypes.c_uint8 * n.value).from_address(ptr.value)
        mv = memoryview(arr).cast("B")
        return mv.toreadonly()

    def address(self, handle: bytes) -> tuple[int, int]:
        """(host address, length) of a blob inside the mapping — for pinned registration / direct H2D."""
        ptr = ctypes.c_void_p()
        n = ctypes.c_uint64()
        if self._lib.pile_get(self._h, bytes(handle), ctypes.byref(ptr), ctypes.byref(n)) != 0:
            raise PileError(f"blob {bytes(handle).hex()} is not readable in {self.path}")
        return int(ptr.value or 0), int(n.value)

    def has(self, handle: bytes) -> bool:
        ptr = ctypes.c_void_p()
        n = ctypes.c_uint64()
        return self._lib.pile_get(self._h, bytes(handle), ctypes.byref(ptr), ctypes.byref(n)) == 0

    def release(self, handle: bytes) -> None:
        """Drop the page-cache pages of a blob after its bytes were copied elsewhere
        (src/models/inkling/pile.rs:119-207)."""
        a, n = self.address(handle)
        self._lib.pile_release(self._h, ctypes.c_void_p(a), n)

    # -- branch records
    def put_branch(self, branch_id: bytes, payload: bytes) -> None:
        out = (ctypes.c_uint8 * 32)()
        if self._lib.pile_put(self._h, KIND_BRANCH, payload, len(payload), bytes(branch_id), out) < 0:
            raise PileError(f"{self.path}: branch update failed: {self._lib.pile_error(self._h).decode()}")

    def records(self):
        kind, off, ln, ts = ctypes.c_uint32(), ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        h, br = (ctypes.c_uint8 * 32)(), (ctypes.c_uint8 * 16)()
        for i in range(self._lib.pile_count(self._h)):
            self._lib.pile_record(self._h, i, ctypes.byref(kind), ctypes.byref(off), ctypes.byref(ln),
                                  ctypes.byref(ts), h, br)
            yield Record(i, kind.value, off.value, ln.value, ts.value, bytes(h), bytes(br))

    def branch_records(self):
        out = []
        for r in self.records():
            if r.kind == KIND_BRANCH:
                data = (ctypes.c_uint8 * r.length).from_address(self._base + r.offset)
                out.append((r.branch, bytes(data)))
        return out

    # -- maintenance
    def refresh(self) -> None:
        if self._lib.pile_refresh(self._h) != 0:
            raise PileError(f"{self.path}: {self._lib.pile_error(self._h).decode()}")

    def flush(self) -> None:
        self._lib.pile_flush(self._h)

    @property
    def size(self) -> int:
        return int(self._lib.pile_size(self._h))

    def stats(self) -> dict:
        a, b = ctypes.c_uint64(), ctypes.c_uint64()
        self._lib.pile_stats(self._h, ctypes.byref(a), ctypes.byref(b))
        return {"bytes_put": a.value, "bytes_dedup": b.value, "records": int(self._lib.pile_count(self._h))}

    def close(self) -> None:
        if self._h:
            self._lib.pile_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

"""BLAKE3-256: native (``_core.so``) with a pure-Python twin used to cross-check it in tests."""
from __future__ import annotations

import ctypes
import struct

_IV = (0x6A09E667, 0xBB67AE85, 0x3C6EF372, 0xA54FF53A, 0x510E527F, 0x9B05688C, 0x1F83D9AB, 0x5BE0CD19)
_PERM = (2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8)
_M = 0xFFFFFFFF
CHUNK_START, CHUNK_END, PARENT, ROOT = 1, 2, 4, 8


def _rotr(x, n):
    return ((x >> n) | (x << (32 - n))) & _M


def _compress(cv, m, counter, block_len, flags):
    s = list(cv) + list(_IV[:4]) + [counter & _M, (counter >> 32) & _M, block_len, flags]
    m = list(m)

    def g(a, b, c, d, mx, my):
        s[a] = (s[a] + s[b] + mx) & _M; s[d] = _rotr(s[d] ^ s[a], 16)
        s[c] = (s[c] + s[d]) & _M;      s[b] = _rotr(s[b] ^ s[c], 12)
        s[a] = (s[a] + s[b] + my) & _M; s[d] = _rotr(s[d] ^ s[a], 8)
        s[c] = (s[c] + s[d]) & _M;      s[b] = _rotr(s[b] ^ s[c], 7)

    for r in range(7):
        g(0, 4, 8, 12, m[0], m[1]); g(1, 5, 9, 13, m[2], m[3])
        g(2, 6, 10, 14, m[4], m[5]); g(3, 7, 11, 15, m[6], m[7])
        g(0, 5, 10, 15, m[8], m[9]); g(1, 6, 11, 12, m[10], m[11])
        g(2, 7, 8, 13, m[12], m[13]); g(3, 4, 9, 14, m[14], m[15])
        if r < 6:
            m = [m[p] for p in _PERM]
    return [s[i] ^ s[i + 8] for i in range(8)] + [s[i + 8] ^ cv[i] for i in range(8)]


def _words(block: bytes):
    return struct.unpack("<16I", block.ljust(64, b"\x00"))


def _chunk_output(data: bytes, index: int):
    cv = list(_IV)
    nblocks = max(1, (len(data) + 63) // 64)
    for b in range(nblocks):
        blk = data[b * 64:(b + 1) * 64]
        flags = CHUNK_START if b == 0 else 0
        if b + 1 == nblocks:
            return cv, _words(blk), index, len(blk), flags | CHUNK_END
        cv = _compress(cv, _words(blk), index, 64, flags)[:8]


def _subtree(data: bytes, chunk0: int):
    if len(data) <= 1024:
        return _chunk_output(data, chunk0)
    chunks = (len(data) + 1023) // 1024
    left = 1
    while left * 2 < chunks:
        left *= 2
    l = _compress(*_subtree(data[:left * 1024], chunk0))[:8]
    r = _compress(*_subtree(data[left * 1024:], chunk0 + left))[:8]
    return list(_IV), tuple(l + r), 0, 64, PARENT


def blake3_py(data: bytes) -> bytes:
    """Pure-Python BLAKE3-256 (slow; the oracle for the native implementation)."""
    cv, m, _ctr, blen, flags = _subtree(bytes(data), 0)
    out = _compress(cv, m, 0, blen, flags | ROOT)
    return struct.pack("<8I", *out[:8])


def blake3(data) -> bytes:
    """BLAKE3-256 of a bytes-like object (native)."""
    from .. import _native
    lib = _native.core()
    out = (ctypes.c_uint8 * 32)()
    if isinstance(data, (bytes, bytearray)):
        buf = (ctypes.c_char * len(data)).from_buffer_copy(data) if isinstance(data, bytearray) else data
        lib.pile_hash(buf, len(data), out)
    else:
        mv = memoryview(data).cast("B")
        if mv.readonly:
            import numpy as np
            arr = np.frombuffer(mv, dtype=np.uint8)
            lib.pile_hash(ctypes.c_void_p(arr.ctypes.data), arr.size, out)
        else:
            lib.pile_hash((ctypes.c_char * len(mv)).from_buffer(mv), len(mv), out)
    return bytes(out)

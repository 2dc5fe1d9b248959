"""ctypes handles to the in-tree native libraries (``_core.so`` and ``_kernels.so``)."""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_lock = threading.Lock()
_core = None
_kernels = None


def core() -> ctypes.CDLL:
    """Host runtime library; compiled on first use when it is missing (g++ only, a few seconds)."""
    global _core
    with _lock:
        if _core is None:
            p = _ROOT / "_core.so"
            if not p.exists():
                from . import _build
                _build.build_core()
            _core = ctypes.CDLL(str(p))
            _declare_core(_core)
        return _core


def kernels() -> ctypes.CDLL:
    """CUDA kernel library.  Raises when it has not been built: a GPU run must never fall back silently."""
    global _kernels
    with _lock:
        if _kernels is None:
            p = _ROOT / "_kernels.so"
            if not p.exists():
                raise RuntimeError(
                    f"{p} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                    "(nvcc, sm_100a) before using the CUDA ops")
            _kernels = ctypes.CDLL(str(p))
        return _kernels


def kernels_available() -> bool:
    return (_ROOT / "_kernels.so").exists()


def _declare_core(lib):
    c = ctypes
    lib.pile_open.restype = c.c_void_p
    lib.pile_open.argtypes = [c.c_char_p, c.c_int, c.c_int]
    lib.pile_error.restype = c.c_char_p
    lib.pile_error.argtypes = [c.c_void_p]
    lib.pile_close.argtypes = [c.c_void_p]
    lib.pile_refresh.argtypes = [c.c_void_p]
    lib.pile_hash.argtypes = [c.c_void_p, c.c_uint64, c.c_void_p]
    lib.pile_put.restype = c.c_int64
    lib.pile_put.argtypes = [c.c_void_p, c.c_uint32, c.c_void_p, c.c_uint64, c.c_void_p, c.c_void_p]
    lib.pile_get.argtypes = [c.c_void_p, c.c_void_p, c.POINTER(c.c_void_p), c.POINTER(c.c_uint64)]
    lib.pile_count.restype = c.c_int64
    lib.pile_count.argtypes = [c.c_void_p]
    lib.pile_size.restype = c.c_uint64
    lib.pile_size.argtypes = [c.c_void_p]
    lib.pile_record.argtypes = [c.c_void_p, c.c_int64, c.POINTER(c.c_uint32), c.POINTER(c.c_uint64),
                                c.POINTER(c.c_uint64), c.POINTER(c.c_uint64), c.c_void_p, c.c_void_p]
    lib.pile_base.restype = c.c_void_p
    lib.pile_base.argtypes = [c.c_void_p]
    lib.pile_stats.argtypes = [c.c_void_p, c.POINTER(c.c_uint64), c.POINTER(c.c_uint64)]
    lib.pile_flush.argtypes = [c.c_void_p]
    lib.pile_amputate.restype = c.c_int64
    lib.pile_amputate.argtypes = [c.c_char_p]
    lib.pile_release.argtypes = [c.c_void_p, c.c_void_p, c.c_uint64]

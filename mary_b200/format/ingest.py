"""Import: checkpoint files -> ``(name, array, shape)`` -> leaves + modules + a model root.

Reference: src/ingest.rs:89-262.  Non-float tensors are skipped (:101-109); ``LeafDtype`` chooses the
stored element (F32 or F16, :27-31) — BF16 is added here because the serving paths run in bf16."""
from __future__ import annotations

from pathlib import Path
from typing import Iterable, Iterator

import numpy as np

from ..pile.trible import TribleBuilder
from .leaf import Elem
from .model import build_model_root, put_tensor


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def _as_elem(arr: np.ndarray, dtype: str):
    if dtype == "f32":
        return np.ascontiguousarray(arr, dtype=np.float32), Elem.F32
    if dtype == "f16":
        return np.ascontiguousarray(arr, dtype=np.float32).astype(np.float16), Elem.F16
    if dtype == "bf16":
        return f32_to_bf16_bits(arr), Elem.BF16
    raise ValueError(f"unknown leaf dtype {dtype!r} (f32, f16, bf16)")


def ingest_tensors(store, tb: TribleBuilder, tensors: Iterable[tuple[str, np.ndarray]], dtype: str = "f32") -> list[bytes]:
    """Write every ``(name, float array)``; returns the module ids."""
    members = []
    for name, arr in tensors:
        a, elem = _as_elem(arr, dtype)
        members.append(put_tensor(store, tb, name, a, elem))
    return members


def iter_checkpoint(path: str | Path) -> Iterator[tuple[str, np.ndarray]]:
    """Yield ``(name, f32 array)`` from a file or directory; format priority safetensors > gguf > pickle
    (src/formats/mod.rs:44-95)."""
    from .formats import detect_format, iter_gguf, iter_pickle
    from .safetensors import SafeTensors
    fmt, files = detect_format(path)
    for f in files:
        if fmt == "safetensors":
            st = SafeTensors(f)
            for k in st.keys():
                a = st.f32(k)
                if a is not None:
                    yield k, a
        elif fmt == "gguf":
            yield from iter_gguf(f)
        elif fmt == "pickle":
            yield from iter_pickle(f)


def ingest_members(store, tb: TribleBuilder, path: str | Path, dtype: str = "f32", name_filter=None) -> list[bytes]:
    it = iter_checkpoint(path)
    if name_filter is not None:
        it = ((n, a) for n, a in it if name_filter(n))
    return ingest_tensors(store, tb, it, dtype)


def ingest_model(store, tb: TribleBuilder, path: str | Path, name: str | None = None, source: str | None = None,
                 dtype: str = "f32", name_filter=None) -> bytes:
    members = ingest_members(store, tb, path, dtype, name_filter)
    if not members:
        raise ValueError(f"{path}: no float tensors found")
    return build_model_root(store, tb, members, name=name, source=source,
                            quantization=None if dtype == "f32" else dtype)

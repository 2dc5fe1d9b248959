"""``WeightLoader``: one interface over checkpoint files and piles.

Reference: src/nn/weight_loader.rs:257-629 — ``SingleFile/MultiShard`` (import only), ``Pile``
(materialised keymap), ``Typed`` (zero-copy leaf views), ``Aliased`` (zero-copy into device memory).
Here the pile variant hands out zero-copy host views of the mapping, and ``to_device`` copies a leaf to the
GPU through a pinned staging ring (the mapping is page-cache memory, so the copy engine cannot read it
directly unless the range is registered)."""
from __future__ import annotations

import numpy as np

from ..format.leaf import Elem, Leaf
from ..format.safetensors import SafeTensors
from ..format.selection import SelectedModelIndex


class WeightLoader:
    def __init__(self, index: SelectedModelIndex | None = None, files: list[SafeTensors] | None = None):
        self.index, self.files = index, files or []
        self.bytes_read = 0
        self._file_of = {k: f for f in self.files for k in f.keys()}

    @staticmethod
    def from_pile(index: SelectedModelIndex) -> "WeightLoader":
        return WeightLoader(index=index)

    @staticmethod
    def from_files(paths) -> "WeightLoader":
        return WeightLoader(files=[SafeTensors(p) for p in paths])

    def names(self) -> list[str]:
        return self.index.names() if self.index is not None else sorted(self._file_of)

    def has_weight(self, name: str) -> bool:
        return self.index.has(name) if self.index is not None else name in self._file_of

    def leaf(self, name: str) -> Leaf:
        if self.index is None:
            raise LookupError("leaf views exist only for pile-backed loaders")
        return self.index.leaf(name)

    def load_host_f32(self, name: str) -> np.ndarray:
        if self.index is not None:
            l = self.index.leaf(name)
            self.bytes_read += len(l.payload)
            return l.to_f32()
        a = self._file_of[name].f32(name)
        if a is None:
            raise TypeError(f"{name}: not a float tensor")
        self.bytes_read += a.nbytes
        return a

    view_f32 = load_host_f32

    def load_tensor(self, name: str, dtype=None, device=None):
        """torch tensor of ``name``; BF16/F16/F32 leaves keep their stored bits when ``dtype`` matches."""
        import torch
        if self.index is not None:
            l = self.index.leaf(name)
            self.bytes_read += len(l.payload)
            if l.elem in (Elem.F32, Elem.F16, Elem.BF16):
                t = l.torch()
            else:
                t = torch.from_numpy(l.to_f32())
        else:
            t = torch.from_numpy(self.load_host_f32(name))
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        if device is not None and str(device) != "cpu":
            t = to_device(t, device)
        elif not t.is_contiguous() or t.data_ptr() % 16:
            t = t.clone()
        return t

    def load_f32(self, name: str, device=None):
        import torch
        return self.load_tensor(name, torch.float32, device)


_STAGE = {}


def to_device(t, device):
    """Host tensor (possibly a read-only view of a mapped pile) -> device, through a pinned staging buffer."""
    import torch
    n = t.numel() * t.element_size()
    key = str(device)
    st = _STAGE.get(key)
    if st is None or st.numel() < n:
        st = torch.empty(max(n, 64 << 20), dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        _STAGE[key] = st
    flat = t.contiguous().view(torch.uint8).reshape(-1)
    st[:n].copy_(flat)
    out = torch.empty(t.shape, dtype=t.dtype, device=device)
    out.view(torch.uint8).reshape(-1).copy_(st[:n], non_blocking=False)
    return out

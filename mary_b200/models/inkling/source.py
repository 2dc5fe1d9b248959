"""``Weights``: the one door through which a serving process reads a model pile — tensors, packed experts, documents — with
residency and byte counters, an admission gate before anything is copied, and ONE registration of the pile mapping for direct
host-to-device copies.

Reference: ``Weights`` facade (``tensor / stored / held / expert_packed / document / copy_share``, residency and byte counters,
src/models/inkling/source.rs:52-446), the startup copy with its admission gate (src/models/inkling/pile.rs:1192-1650),
``Aliases``: one registration of the pile mapping with bind statistics (src/models/inkling/fp4gemm.rs:493-840), release of the
source pages after the copy (pile.rs:119-207).

On a B200 the weights are served from HBM, so the reference's "anonymous RAM copy of this node's share" becomes the device
copy of this rank's share.  The copy engine cannot read page-cache memory unless the range is registered; instead of staging
every tensor through a pinned bounce buffer, :meth:`register` pins the whole pile mapping once (``cudaHostRegister``, read-only
mapping) and every later copy is a direct DMA from the mapping.  Where registration is refused (no CUDA device, or the
platform rejects read-only registrations) the loader falls back to the staging path and the counters say so."""
from __future__ import annotations

import ctypes
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from ...format import jsonfacts
from ...format.leaf import Elem
from ...format.persist import read_model_pile
from ...format.selection import SelectedModelIndex
from ...nn.weight_loader import to_device
from ...runtime.budget import AdmissionError

CUDA_HOST_REGISTER_READ_ONLY = 0x08


@dataclass
class IoStats:
    tensors: int = 0
    bytes_requested: int = 0
    bytes_direct: int = 0            # copied straight from the registered mapping
    bytes_staged: int = 0            # copied through the pinned bounce buffer
    bytes_released: int = 0          # page-cache pages handed back after the copy
    seconds: float = 0.0
    held: dict = field(default_factory=dict)     # name -> bytes resident on the device


class Weights:
    def __init__(self, pile, facts=None, index: SelectedModelIndex | None = None):
        self.pile = pile
        self.facts = read_model_pile(pile) if facts is None else facts
        self.index = index or SelectedModelIndex.from_snapshot(pile, self.facts)
        self.stats = IoStats()
        self.registered = False
        self._reg = None

    @staticmethod
    def open(pile) -> "Weights":
        return Weights(pile)

    # ---- what the pile holds
    def names(self) -> list[str]:
        return self.index.names()

    def has(self, name: str) -> bool:
        return self.index.has(name)

    def document(self, name: str):
        return jsonfacts.load_document(self.pile, self.facts, name)

    def stored(self, name: str) -> int:
        """Bytes of the tensor as stored in the pile."""
        return len(self.index.leaf(name).payload)

    def held(self, name: str) -> int:
        """Bytes of the tensor resident on the device through this facade (0 when it was never copied)."""
        return self.stats.held.get(name, 0)

    # ---- registration: one pinned registration of the whole mapping
    def register(self) -> bool:
        """Pin the pile mapping for direct DMA.  Returns whether the registration holds; never raises for a refusal."""
        if self.registered or not torch.cuda.is_available():
            return self.registered
        base, size = int(self.pile._base or 0), int(self.pile.size())
        if not base or not size:
            return False
        try:
            rt = torch.cuda.cudart()
            rc = rt.cudaHostRegister(base, size, CUDA_HOST_REGISTER_READ_ONLY)
            ok = int(rc) == 0 if not hasattr(rc, "value") else rc.value == 0
        except Exception:
            ok = False
        self.registered, self._reg = ok, (base, size) if ok else None
        return ok

    def unregister(self) -> None:
        if self.registered and self._reg:
            try:
                torch.cuda.cudart().cudaHostUnregister(self._reg[0])
            except Exception:
                pass
        self.registered, self._reg = False, None

    # ---- copies
    def _to_device(self, host: torch.Tensor, device, name: str):
        n = host.numel() * host.element_size()
        self.stats.bytes_requested += n
        t0 = time.perf_counter()
        if str(device) == "cpu":
            out = host.clone()
        elif self.registered:
            out = torch.empty(host.shape, dtype=host.dtype, device=device)
            out.copy_(host, non_blocking=True)             # the source is registered (pinned) memory: a direct DMA
            self.stats.bytes_direct += n
        else:
            out = to_device(host, device)
            self.stats.bytes_staged += n
        self.stats.seconds += time.perf_counter() - t0
        self.stats.tensors += 1
        self.stats.held[name] = self.stats.held.get(name, 0) + n
        return out

    def tensor(self, name: str, device="cpu", dtype=None):
        """A dense tensor by name (stored bits kept when ``dtype`` matches the stored element)."""
        leaf = self.index.leaf(name)
        host = leaf.torch() if leaf.elem in (Elem.BF16, Elem.F32, Elem.F16, Elem.I32, Elem.I64, Elem.U8) else torch.from_numpy(leaf.to_f32())
        out = self._to_device(host, device, name)
        return out if dtype is None or out.dtype == dtype else out.to(dtype)

    def expert_packed(self, name: str, device="cpu"):
        """An NVFP4 expert matrix ``(codes [rows, k/2], scales [rows, k/16], scale2)`` straight from its blob."""
        codes, scales, s2 = self.index.leaf(name).fp4_parts()
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            c, s = torch.from_numpy(codes), torch.from_numpy(scales)
        return self._to_device(c, device, name), self._to_device(s, device, name + "#scales"), s2

    def release(self, name: str) -> None:
        """Hand the page-cache pages of a tensor back to the kernel once its bytes live on the device (pile.rs:119-207)."""
        leaf = self.index.leaf(name)
        try:
            self.pile.release(leaf.handle)
            self.stats.bytes_released += len(leaf.payload)
        except Exception:
            pass

    # ---- admission
    def share_bytes(self, names) -> int:
        return sum(self.stored(n) for n in names)

    def admit(self, names, other_bytes: int, capacity: int, headroom: float = 0.03) -> int:
        """Refuse a share that cannot fit BEFORE the first copy: the stored bytes of ``names`` plus ``other_bytes`` (activations,
        KV cache, workspaces) against ``capacity``.  Returns the share's bytes."""
        want = self.share_bytes(names)
        if want + other_bytes > capacity * (1.0 - headroom):
            g = 1 << 30
            raise AdmissionError(f"this rank's share is {want / g:.2f} GiB of weights + {other_bytes / g:.2f} GiB of cache and activations = "
                                 f"{(want + other_bytes) / g:.2f} GiB, and the device offers {capacity / g:.2f} GiB")
        return want

    def io_table(self) -> str:
        s = self.stats
        g = 1 << 30
        rate = s.bytes_requested / s.seconds / g if s.seconds else 0.0
        return (f"weights: {s.tensors} tensors, {s.bytes_requested / g:.2f} GiB requested ({s.bytes_direct / g:.2f} direct from the "
                f"{'registered' if self.registered else 'unregistered'} mapping, {s.bytes_staged / g:.2f} staged), {s.bytes_released / g:.2f} GiB "
                f"of source pages released, {rate:.2f} GiB/s")

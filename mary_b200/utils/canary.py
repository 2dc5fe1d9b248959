"""Guard bands around the output buffers of the package's kernels: the stand-in for a memory sanitizer on machines where the
sanitizer tools are closed.

With ``MARY_CANARY=1`` every output that the op wrappers allocate (``ops.cuda``, ``ops.cuda_moe``, ``ops.train_ops``) sits between
two bands of ``GUARD`` bytes filled with a pattern; ``check_all()`` synchronises and verifies every band allocated since the last
check, naming the first buffer whose neighbourhood a kernel wrote outside its extent (a write past the end, before the start, or
— for row-pitched outputs — into the bytes between rows, which the caller verifies with ``Guarded.rows_intact``).  Off by default:
allocation is then plain ``torch.empty``.

The reference relies on wgpu's bounds-checked buffer accesses for the same class of error (every binding is range-checked by the
API); raw CUDA pointers have no such net."""
from __future__ import annotations

import math

import torch

GUARD = 512            # bytes on each side, a multiple of the 256-byte allocation granule
PATTERN = 0xA5

_live: list["Guarded"] = []
_enabled: bool | None = None


def enabled() -> bool:
    global _enabled
    if _enabled is None:
        from . import flags
        _enabled = bool(flags.get("MARY_CANARY"))
    return _enabled


def set_enabled(on: bool) -> None:
    global _enabled
    _enabled = bool(on)


class Guarded:
    """A tensor of ``shape`` whose storage has ``GUARD`` pattern bytes before and after it."""

    def __init__(self, shape, dtype, device, what: str = ""):
        n = int(math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        body = (n + 15) // 16 * 16
        self.raw = torch.empty(GUARD + body + GUARD, dtype=torch.uint8, device=device)
        self.raw[:GUARD].fill_(PATTERN)
        self.raw[GUARD + n:].fill_(PATTERN)
        self.n, self.what = n, what
        self.tensor = self.raw[GUARD:GUARD + n].view(dtype).view(*shape)

    def intact(self) -> bool:
        head, tail = self.raw[:GUARD], self.raw[GUARD + self.n:]
        return bool((head == PATTERN).all().item()) and bool((tail == PATTERN).all().item())


def empty(*shape, dtype=torch.float32, device="cpu", what: str = "") -> torch.Tensor:
    """``torch.empty`` or, with the canaries on, a guarded buffer remembered for ``check_all``."""
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    if not enabled():
        return torch.empty(*shape, dtype=dtype, device=device)
    g = Guarded(shape, dtype, device, what)
    _live.append(g)
    if len(_live) > 4096:                      # long runs: check and forget the oldest half
        check_all(keep=2048)
    return g.tensor


def check_all(keep: int = 0) -> int:
    """Verify the guard bands of every buffer handed out since the last check; returns how many were checked."""
    if not _live:
        return 0
    if _live[0].raw.is_cuda:
        torch.cuda.synchronize()
    n = len(_live) - keep
    for g in _live[:n]:
        if not g.intact():
            raise RuntimeError(f"a kernel wrote outside an output buffer ({g.what or 'unnamed'}, {g.n} bytes)")
    del _live[:n]
    return n

"""Fail loudly: an exception on ANY thread ends the process (src/models/inkling/fatal.rs:57-140 — a panic hook that aborts,
plus a diagnosis line for allocation refusals), so a serving rank never lingers half-dead while its peers wait on it."""
from __future__ import annotations

import os
import sys
import threading
import traceback

_armed = False


def _diagnose(exc: BaseException) -> str:
    s = f"{type(exc).__name__}: {exc}"
    if "out of memory" in s.lower():
        try:
            import torch
            free, total = torch.cuda.mem_get_info()
            s += f"\n  device memory: {free / 2**30:.2f} GiB free of {total / 2**30:.2f} GiB — see mary_b200.runtime.budget for the bill"
        except Exception:
            pass
    return s


def arm(exit_code: int = 70) -> None:
    """Install hooks for the main thread and for worker threads."""
    global _armed
    if _armed:
        return
    _armed = True

    def die(exc_type, exc, tb):
        traceback.print_exception(exc_type, exc, tb, file=sys.stderr)
        sys.stderr.write("fatal: " + _diagnose(exc) + "\n")
        sys.stderr.flush()
        os._exit(exit_code)

    sys.excepthook = die
    threading.excepthook = lambda a: die(a.exc_type, a.exc_value, a.exc_traceback)

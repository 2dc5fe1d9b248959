"""Per-kernel timing without a profiler: CUDA events between consecutive launches on one stream.

Every launcher wrapper in ``mary_b200.ops.cuda`` ends in ``check(rc, name)``; while a ``Tracer`` is active that call
also records a CUDA event tagged with the op name.  Launches on one stream run in order, so the time between two
consecutive events is the device time of the later op (plus whatever plain torch work ran in between, reported under
the op that follows it).  The reference has no tracing framework, only ``Instant`` buckets and a ``stage_sync!`` macro
that synchronises per stage (src/bin/inkling_forward.rs:1318-1352,4128-4155); this gives the same per-stage table with
one synchronisation at the end."""
from __future__ import annotations

from collections import defaultdict

import torch


class nvtx_range:
    """``with nvtx_range("layer 3"):`` — an NVTX range when ``MARY_NVTX=1`` (for Nsight timelines), nothing otherwise."""

    def __init__(self, name: str):
        from . import flags
        self.name, self.on = name, bool(flags.get("MARY_NVTX")) and torch.cuda.is_available()

    def __enter__(self):
        if self.on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *a):
        if self.on:
            torch.cuda.nvtx.range_pop()


class Tracer:
    def __init__(self):
        self.events: list[tuple[str, torch.cuda.Event]] = []

    def __enter__(self):
        from ..ops import cuda as K
        self._K = K
        K.TRACE = self
        self.mark("start")
        return self

    def __exit__(self, *a):
        self.mark("end")
        self._K.TRACE = None

    def mark(self, name: str):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append((name, e))

    def table(self) -> list[tuple[str, int, float]]:
        """``(op, calls, total ms)`` sorted by time."""
        torch.cuda.synchronize()
        agg: dict[str, list] = defaultdict(lambda: [0, 0.0])
        for (_, a), (name, b) in zip(self.events[:-1], self.events[1:]):
            agg[name][0] += 1
            agg[name][1] += a.elapsed_time(b)
        return sorted(((k, v[0], v[1]) for k, v in agg.items()), key=lambda r: -r[2])

    def report(self) -> str:
        rows = self.table()
        total = sum(r[2] for r in rows) or 1.0
        out = [f"{'op':<28}{'calls':>8}{'ms':>12}{'share':>9}"]
        out += [f"{n:<28}{c:>8}{ms:>12.3f}{100 * ms / total:>8.1f}%" for n, c, ms in rows]
        out.append(f"{'total':<28}{'':>8}{total:>12.3f}")
        return "\n".join(out)

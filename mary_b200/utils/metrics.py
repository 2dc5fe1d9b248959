"""Run metrics as JSON lines plus a human summary: tokens/s, TTFT, TPOT percentiles, speculative acceptance with a Wilson
interval (the reference prints per-run reports only: src/bin/inkling_forward.rs:1144-1162,6037-6400)."""
from __future__ import annotations

import json
import math
import time


def wilson(successes: int, n: int, z: float = 1.96) -> tuple[float, float]:
    if n == 0:
        return 0.0, 1.0
    p = successes / n
    d = 1 + z * z / n
    c = p + z * z / (2 * n)
    h = z * math.sqrt(p * (1 - p) / n + z * z / (4 * n * n))
    return (c - h) / d, (c + h) / d


def percentile(xs, q: float) -> float:
    xs = sorted(xs)
    if not xs:
        return float("nan")
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


class MetricsLog:
    def __init__(self, path: str | None = None):
        self.path, self.rows = path, []
        self._f = open(path, "a") if path else None

    def emit(self, kind: str, **kw):
        row = {"t": time.time(), "kind": kind, **kw}
        self.rows.append(row)
        if self._f:
            self._f.write(json.dumps(row) + "\n")
            self._f.flush()

    def summary(self) -> dict:
        steps = [r for r in self.rows if r["kind"] == "step"]
        toks = sum(r.get("tokens_out", 0) for r in steps)
        secs = sum(r.get("seconds", 0.0) for r in steps)
        ttft = [r["ttft_s"] for r in self.rows if r["kind"] == "request" and "ttft_s" in r]
        acc = sum(r.get("accepted", 0) for r in steps)
        drafted = sum(r.get("drafted", 0) for r in steps)
        lo, hi = wilson(acc, drafted)
        return {"tokens": toks, "tokens_per_s": toks / secs if secs else 0.0, "ttft_p50_s": percentile(ttft, 0.5),
                "ttft_p99_s": percentile(ttft, 0.99), "tpot_p50_s": percentile([r["seconds"] for r in steps], 0.5),
                "acceptance": acc / drafted if drafted else None, "acceptance_wilson95": (lo, hi) if drafted else None}

"""Rank health on the host: heartbeats through a key-value store, graceful leave, and a guard that turns a missing peer into an
exception BEFORE the next launch (the reference has only "socket EOF = peer done" and a cohort id on the wire,
src/bin/inkling_forward.rs:747-751,1221-1263).

Device-side waits on peer flags are bounded and report through the status word; this module is the host half: a rank that raised,
exited or never joined stops beating, its peers see the stale entry at their next ``guard()`` and stop issuing kernels or
collectives that would wait for it.  The store is anything with ``set(key, bytes)`` / ``get(key) -> bytes``: a
``torch.distributed`` store (``TCPStore``, ``FileStore``, ``HashStore``) in production, a dict in tests.  Nothing here touches a
GPU; failures are injected on the host (stop beating, leave, corrupt a header)."""
from __future__ import annotations

import struct
import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, ranks, reason: str):
        super().__init__(f"rank(s) {sorted(ranks)} {reason}")
        self.ranks = sorted(ranks)


class DictStore:
    """In-process stand-in for a distributed store (tests; single-process runs)."""

    def __init__(self):
        self._d, self._lock = {}, threading.Lock()

    def set(self, k, v):
        with self._lock:
            self._d[k] = bytes(v)

    def get(self, k):
        with self._lock:
            return self._d[k]


def _try_get(store, key):
    try:
        if hasattr(store, "check") and not store.check([key]):      # torch stores block in get(); ask first
            return None
        return bytes(store.get(key))
    except KeyError:
        return None


class Heartbeat:
    """``start()`` beats every ``interval`` seconds from a daemon thread; ``stale()`` lists peers whose last beat is older than
    ``timeout`` (or that never beat once ``grace`` seconds have passed since this rank started); ``leave()`` marks an orderly
    departure between steps, which peers report as "left" rather than "stopped answering"."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.2, timeout: float = 1.0, grace: float = 5.0, clock=time.monotonic,
                 prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.grace, self.clock, self.prefix = interval, timeout, grace, clock, prefix
        self._stop = threading.Event()
        self._thread = None
        self._t0 = clock()
        self.seq = 0

    def beat(self) -> None:
        self.seq += 1
        self.store.set(f"{self.prefix}/{self.rank}", struct.pack("<dq", self.clock(), self.seq))

    def start(self) -> "Heartbeat":
        self.beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            self.beat()

    def stop(self) -> None:
        """Stop beating WITHOUT saying goodbye (what a crashed rank looks like)."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def leave(self) -> None:
        self.stop()
        self.store.set(f"{self.prefix}/{self.rank}", struct.pack("<dq", -1.0, self.seq))

    def status(self) -> dict:
        """``{rank: "ok" | "left" | "stale" | "absent"}`` for every peer."""
        now, out = self.clock(), {}
        for r in range(self.world):
            if r == self.rank:
                continue
            raw = _try_get(self.store, f"{self.prefix}/{r}")
            if raw is None:
                out[r] = "absent" if now - self._t0 > self.grace else "ok"
                continue
            t, _ = struct.unpack("<dq", raw)
            out[r] = "left" if t < 0 else ("stale" if now - t > self.timeout else "ok")
        return out

    def guard(self) -> None:
        """Call between steps, before launching anything that waits on a peer."""
        st = self.status()
        for kind, reason in (("left", "left the job"), ("stale", "stopped answering"), ("absent", "never joined")):
            bad = [r for r, s in st.items() if s == kind]
            if bad:
                raise RankFailure(bad, reason)


WIRE_HEADER = struct.Struct("<qqq")        # rows, first position, cohort id — the 24-byte header of a pipeline message


def pack_header(rows: int, pos0: int, cohort: int) -> bytes:
    return WIRE_HEADER.pack(rows, pos0, cohort)


def check_header(raw: bytes, expect_cohort: int, max_rows: int) -> tuple[int, int]:
    """A desynchronised pipeline (an answer for another cohort, a corrupt length) fails loudly here instead of silently feeding
    the wrong rows to the next stage."""
    if len(raw) != WIRE_HEADER.size:
        raise RankFailure([], f"sent a {len(raw)}-byte header, expected {WIRE_HEADER.size}")
    rows, pos0, cohort = WIRE_HEADER.unpack(raw)
    if cohort != expect_cohort:
        raise RankFailure([], f"answered for cohort {cohort} while cohort {expect_cohort} was due (pipeline out of step)")
    if not 0 <= rows <= max_rows or pos0 < 0:
        raise RankFailure([], f"sent an impossible header rows={rows} pos0={pos0}")
    return rows, pos0

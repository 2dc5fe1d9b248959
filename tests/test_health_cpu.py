"""Failure detection on the host: a rank that stops beating, leaves, or never joins is seen by its peers before their next launch;
a pipeline message for the wrong cohort or with a corrupt length fails loudly.  No GPU is involved."""
import threading
import time

import pytest

from mary_b200.parallel.health import DictStore, Heartbeat, RankFailure, check_header, pack_header


def test_peers_notice_a_silent_rank_a_leaver_and_an_absentee():
    store = DictStore()
    now = [100.0]
    hb = [Heartbeat(store, r, 4, timeout=1.0, grace=2.0, clock=lambda: now[0]) for r in range(4)]
    for h in hb[:3]:
        h.beat()                                   # rank 3 never joins
    hb[0].guard()                                  # inside the grace period an absent rank is not yet a failure
    now[0] += 0.5
    hb[0].beat(), hb[1].beat()                     # rank 2 goes silent
    now[0] += 0.8
    assert hb[0].status() == {1: "ok", 2: "stale", 3: "ok"}
    with pytest.raises(RankFailure) as e:
        hb[0].guard()
    assert e.value.ranks == [2] and "stopped answering" in str(e.value)
    hb[2].beat()
    hb[1].leave()
    with pytest.raises(RankFailure, match="left the job"):
        hb[0].guard()
    now[0] += 2.0
    hb[0].beat(), hb[2].beat()
    assert hb[2].status()[3] == "absent"


def test_threads_as_ranks_detect_a_rank_that_raises_between_steps():
    store = DictStore()
    world, seen = 3, {}

    def rank(r):
        hb = Heartbeat(store, r, world, interval=0.02, timeout=1.0, grace=5.0).start()
        try:
            for step in range(600):
                hb.guard()
                if r == 1 and step == 3:
                    raise RuntimeError("injected host failure")            # dies without saying goodbye
                time.sleep(0.01)
        except RankFailure as ex:
            seen[r] = ex.ranks
        except RuntimeError:
            pass
        finally:
            hb.stop()
    ts = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    assert set(seen) == {0, 2} and all(1 in v for v in seen.values()), seen


def test_torch_store_backend_and_wire_header_checks():
    dist = pytest.importorskip("torch.distributed")
    store = dist.HashStore()
    a, b = Heartbeat(store, 0, 2, timeout=0.2, grace=0.0), Heartbeat(store, 1, 2, timeout=0.2, grace=0.0)
    a.beat(), b.beat()
    a.guard()
    time.sleep(0.3)
    a.beat()
    with pytest.raises(RankFailure):
        a.guard()
    raw = pack_header(48, 4096, 2)
    assert len(raw) == 24 and check_header(raw, 2, 128) == (48, 4096)
    with pytest.raises(RankFailure, match="cohort 2 while cohort 1"):
        check_header(raw, 1, 128)
    with pytest.raises(RankFailure, match="impossible"):
        check_header(pack_header(1 << 40, 0, 1), 1, 128)
    with pytest.raises(RankFailure, match="header"):
        check_header(raw[:20], 2, 128)

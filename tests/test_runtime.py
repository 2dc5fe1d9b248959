import numpy as np
import pytest
import torch

from mary_b200.models.gemma4 import Gemma4Model, tiny_config
from mary_b200.models.gemma4.weights import init_random_
from mary_b200.runtime.engine import Engine
from mary_b200.runtime.kv_cache import OutOfPages, PageAllocator, PagedKVCache


def test_page_allocator_extend_truncate_release():
    a = PageAllocator(8, 16)
    assert a.extend(1, 17) == 17 and a.pages(1) == [0, 1] and a.free_pages == 6
    a.extend(2, 16)
    assert a.pages(2) == [2]
    a.extend(1, 15)
    assert a.pages(1) == [0, 1] and a.seq_len(1) == 32
    a.extend(1, 1)
    assert a.pages(1) == [0, 1, 3]
    a.truncate(1, 32)                         # speculative row rejected: the page goes back
    assert a.pages(1) == [0, 1] and a.free_pages == 5
    with pytest.raises(OutOfPages):
        a.extend(3, 16 * 6)
    assert a.seq_len(3) == -1                 # a failed extend leaves no trace
    a.release(1)
    assert a.free_pages == 7
    t, l = a.page_table([2], 4)
    assert t.tolist() == [[2, -1, -1, -1]] and l.tolist() == [16]


def _engine(max_seqs=4, prefill_chunk=2048, pages=64):
    torch.manual_seed(0)
    cfg = tiny_config()
    m = Gemma4Model(cfg)
    init_random_(m, 0)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], pages, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    return Engine(m, cache, max_tokens=256, max_seqs=max_seqs, prefill_chunk=prefill_chunk)


def test_continuous_batching_matches_isolated_runs():
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 4096, n).tolist() for n in (5, 33, 17)]
    alone = [_engine().generate([p], 6)[0] for p in prompts]
    together = _engine().generate(prompts, 6)
    assert together == alone                  # neighbours in the batch do not contaminate each other


def test_chunked_prefill_matches_whole_prefill():
    p = np.random.default_rng(1).integers(0, 4096, 50).tolist()
    assert _engine(prefill_chunk=16).generate([p], 5) == _engine().generate([p], 5)


def test_admission_waits_for_pages_and_all_finish():
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 4096, 40).tolist() for _ in range(6)]
    e = _engine(max_seqs=8, pages=12)         # room for about three sequences at a time
    outs = e.generate(prompts, 4)
    assert all(len(o) == 4 for o in outs)
    assert e.cache.alloc.free_pages == 12     # everything was released
    assert outs == [_engine().generate([p], 4)[0] for p in prompts]


def test_speculative_rows_commit_and_rollback_leave_no_trace():
    """Feed a correct draft and a wrong draft: accepted tokens equal plain greedy, and the cache afterwards is
    identical to a run without speculation (rejected rows leave no trace)."""
    p = np.random.default_rng(3).integers(0, 4096, 20).tolist()
    plain = _engine().generate([p], 6)[0]
    e = _engine()
    rid = e.add_request(p, 6)
    e.step()                                  # prefill -> first token
    assert e.outputs[rid] == plain[:1]
    good_then_bad = np.asarray([plain[1], (plain[2] + 1) % 4096], dtype=np.int32)
    e.lib.sched_set_drafts(e.h, rid, good_then_bad.ctypes.data, 2)
    e.step()
    assert e.outputs[rid] == plain[:3] and e.accepted_hist == [1]
    assert e.cache.alloc.seq_len(rid) == len(p) + 2          # pending + one accepted draft kept, one row dropped
    e.run()
    assert e.outputs[rid][:6] == plain


def test_admission_reserves_the_pages_a_running_request_can_grow_to():
    """Two requests that each fit the pool alone but not together: the second one must wait until the first has finished,
    instead of both being admitted and the decode loop finding the pool empty."""
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, 4096, 20).tolist() for _ in range(2)]
    # 20 prompt + 70 new + 8 speculative rows = 98 tokens = 7 pages each; the pool holds 10
    e = _engine(max_seqs=4, pages=10)
    rids = [e.add_request(p, 70) for p in prompts]
    e.step()
    assert e.lib.sched_num_running(e.h) == 1 and e.lib.sched_num_waiting(e.h) == 1
    e.run()
    assert all(len(e.outputs[r]) >= 70 for r in rids)
    assert e.cache.alloc.free_pages == 10


def test_empty_prompt_and_oversized_requests_are_refused_at_submission():
    e = _engine(pages=8)
    with pytest.raises(ValueError):
        e.add_request([], 4)
    with pytest.raises(ValueError):
        e.add_request([1, 2, 3], 16 * 8)      # more pages than the pool holds
    assert e.generate([[5, 6, 7]], 3)[0] is not None


def test_spec_decoder_refuses_a_step_that_could_leave_its_page_table():
    from mary_b200.models.moe import MoEDecoder, init_random_ as moe_init, tiny_moe_config
    from mary_b200.runtime.spec_decode import SpecDecoder
    cfg = tiny_moe_config("gqa")
    m = MoEDecoder(cfg, dtype=torch.float32)
    moe_init(m, 0)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 16, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    dec = SpecDecoder(m, cache, 2, spec_k=0, max_len=48, device="cpu", use_graph=False)
    dec.set_context([40, 40], [1, 2])
    for _ in range(6):
        dec.step()
    with pytest.raises(RuntimeError, match="refused"):
        for _ in range(4):
            dec.step()

"""Host-side checks of the runtime's batch description."""
import pytest


def test_debug_checks_refuse_inconsistent_batches(monkeypatch):
    import numpy as np
    from mary_b200.runtime.batch import BatchMeta, check_batch
    table = np.array([[0, 1], [2, 3]], dtype=np.int32)
    check_batch([1, 1], [17, 3], table, 16, num_pages=4)
    with pytest.raises(ValueError, match="cannot hold"):
        check_batch([1, 1], [40, 3], table, 16)
    with pytest.raises(ValueError, match="outside the cache"):
        check_batch([1, 1], [17, 3], table, 16, num_pages=2)
    with pytest.raises(ValueError, match="two positions"):
        check_batch([1, 1], [17, 3], np.array([[0, 1], [1, 3]], dtype=np.int32), 16)
    with pytest.raises(ValueError, match="inconsistent"):
        check_batch([5], [3], table[:1], 16)
    monkeypatch.setenv("MARY_DEBUG_CHECKS", "1")
    from mary_b200.utils import flags
    flags.reset()                                     # flags are read once per process
    with pytest.raises(ValueError):
        BatchMeta.build([1, 1], [17, 3], np.array([[0, 1], [1, 3]], dtype=np.int32), 16)
    BatchMeta.build([1, 1], [17, 3], table, 16)
    monkeypatch.delenv("MARY_DEBUG_CHECKS")
    flags.reset()


def test_flags_are_typed_and_refuse_malformed_values(monkeypatch):
    from mary_b200.utils import flags
    monkeypatch.setenv("MARY_BENCH_LIMIT_S", "12")
    monkeypatch.setenv("MARY_PDL", "yes")
    flags.reset()
    assert flags.get("MARY_BENCH_LIMIT_S") == 12 and flags.get("MARY_PDL") is True
    monkeypatch.setenv("MARY_BENCH_LIMIT_S", "soon")
    flags.reset()
    with pytest.raises(ValueError, match="MARY_BENCH_LIMIT_S"):
        flags.get("MARY_BENCH_LIMIT_S")
    with pytest.raises(KeyError):
        flags.get("MARY_NOT_DECLARED")
    monkeypatch.delenv("MARY_BENCH_LIMIT_S"), monkeypatch.delenv("MARY_PDL")
    flags.reset()
    assert any(name == "MARY_MOE_FUSED" for name, *_ in flags.table())


def test_pool_policy_and_prefill_admission():
    from mary_b200.models.moe import k3_class_config
    from mary_b200.runtime import budget
    from mary_b200.runtime.pool import CleanupPolicy, Pool, choose_memory_config
    assert choose_memory_config() == "default" and Pool(CleanupPolicy.STAGE).line().startswith("pool: policy stage")
    c = k3_class_config()
    small, big = budget.prefill_activation_bytes(c, 512), budget.prefill_activation_bytes(c, 8192)
    assert small < big and budget.largest_buffer(c, 8192) < big
    n = budget.longest_sequence(c, 8 << 30)
    assert budget.prefill_activation_bytes(c, n) <= (8 << 30) < budget.prefill_activation_bytes(c, n + 1)
    with pytest.raises(budget.AdmissionError, match="longest chunk"):
        budget.check_prefill(c, 65536, 4 << 30)
    assert budget.check_prefill(c, 512, 8 << 30) == small


def test_engine_emits_metrics_rows(tmp_path):
    import json
    import torch
    from mary_b200.models.gemma4 import Gemma4Model, tiny_config
    from mary_b200.models.gemma4.weights import init_random_
    from mary_b200.runtime.engine import Engine
    from mary_b200.runtime.kv_cache import PagedKVCache
    from mary_b200.utils.metrics import MetricsLog
    torch.manual_seed(0)
    m = Gemma4Model(tiny_config())
    init_random_(m, 0)
    spec = m.kv_spec()
    cache = PagedKVCache(spec["num_layers"], 32, 16, spec["kv_heads"], spec["head_dim"], dtype=torch.float32)
    log = MetricsLog(str(tmp_path / "m.jsonl"))
    e = Engine(m, cache, max_tokens=128, max_seqs=4, metrics=log)
    e.generate([[1, 2, 3], [4, 5, 6, 7]], 3)
    rows = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert sum(r["kind"] == "request" for r in rows) == 2 and sum(r["kind"] == "step" for r in rows) >= 3
    s = log.summary()
    assert s["tokens"] >= 6 and s["ttft_p50_s"] > 0


def test_every_gate_passes_and_every_mutant_is_caught(capsys):
    from mary_b200 import gates
    assert gates.run("all") == 0
    assert gates.run("all", mutate=True) == 0
    out = capsys.readouterr().out
    assert out.count("PASS") == len(gates.GATES) and out.count("mutant caught") == len(gates.GATES)
    assert gates.run("no-such-gate") == 2

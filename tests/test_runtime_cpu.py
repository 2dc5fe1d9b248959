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
    with pytest.raises(ValueError):
        BatchMeta.build([1, 1], [17, 3], np.array([[0, 1], [1, 3]], dtype=np.int32), 16)
    BatchMeta.build([1, 1], [17, 3], table, 16)

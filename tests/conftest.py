import os
import sys
from pathlib import Path

import pytest

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch
    has_gpu = torch.cuda.is_available()
    ngpu = torch.cuda.device_count() if has_gpu else 0
    for it in items:
        if "gpu" in it.keywords and not has_gpu:
            it.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in it.keywords and ngpu < 2:
            it.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture
def tmp_pile(tmp_path):
    from mary_b200.pile import Pile, signing_key_file
    p = Pile.open(str(tmp_path / "t.pile"))
    key = signing_key_file(str(tmp_path / "key"))
    yield p, key
    p.close()

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs more than one CUDA device")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
        ngpu = torch.cuda.device_count() if have else 0
    except Exception:
        have, ngpu = False, 0
    skip = pytest.mark.skip(reason="no CUDA device")
    skipm = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for it in items:
        if "gpu" in it.keywords and not have:
            it.add_marker(skip)
        if "multigpu" in it.keywords and ngpu < 2:
            it.add_marker(skipm)

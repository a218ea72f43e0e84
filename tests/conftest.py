import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu: needs >= 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        skip = pytest.mark.skip(reason="needs >= 2 GPUs")
        for it in items:
            if "multigpu" in it.keywords and n < 2:
                it.add_marker(skip)
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords or "multigpu" in it.keywords:
            it.add_marker(skip)

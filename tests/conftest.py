import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a real B200 (run with -m gpu on the GPU box)")
    config.addinivalue_line("markers", "multigpu: needs two or more GPUs")


def pytest_collection_modifyitems(config, items):
    import torch_musa_b200 as bw

    if bw.is_available():
        n = bw.device_count()
        skip_multi = pytest.mark.skip(reason="needs >= 2 GPUs")
        for item in items:
            if "multigpu" in item.keywords and n < 2:
                item.add_marker(skip_multi)
        return
    skip = pytest.mark.skip(reason="no blackwell device on this host")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def bw():
    import torch_musa_b200

    return torch_musa_b200


@pytest.fixture
def dev():
    import torch

    return torch.device("blackwell:0")

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def guard_words_are_intact():
    """After every test that ran on the GPU: no kernel stored outside a workspace, a scratch area or a cache pool
    (abacus_b200/kernels/guards.py)."""
    yield
    guards = sys.modules.get("abacus_b200.kernels.guards")
    if guards is not None and guards._buffers:
        import torch
        if torch.cuda.is_available():
            guards.assert_intact()


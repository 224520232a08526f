import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def tune():
    """Set launch-shape knobs of the library for one test: ``tune("CHUNK_ROWS", 64)``.  Every knob
    goes back to its start-up value afterwards."""
    from quick_ssm_b200 import _lib

    def _set(name, value):
        _lib.tune_set(name, int(value))

    yield _set
    _lib.tune_reset()

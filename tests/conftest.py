import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    """Tests marked gpu need a CUDA device and the built library: skip them (instead of failing at the
    first call) on a box that has neither, e.g. a plain `pytest` on a CPU-only machine."""
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    have_lib = os.path.exists(os.path.join(ROOT, "rwkvstic_b200", "libb200rwkv.so"))
    if have_gpu and have_lib:
        return
    why = "no CUDA device" if not have_gpu else "rwkvstic_b200/libb200rwkv.so is not built"
    skip = pytest.mark.skip(reason=f"needs a GPU run: {why}")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name), allow_pickle=False)
    return load

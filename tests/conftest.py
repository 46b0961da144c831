import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def emulated_ops(monkeypatch):
    """Replace the CUDA kernels by the slow torch emulation of tests/emu_ops.py,
    so that the engine's host logic can run where there is no GPU."""
    import emu_ops
    from rust_inference_b200 import ops
    for name in emu_ops.__all__:
        monkeypatch.setattr(ops, name, getattr(emu_ops, name))
    return emu_ops

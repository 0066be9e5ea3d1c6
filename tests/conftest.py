"""Shared pytest configuration.

Tests marked ``gpu`` need a real B200; everything else runs on the
host-simulated backend (no GPU) and on CPU ``gloo`` ranks.
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a real B200 GPU (run with -m gpu on a GPU box)")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    has_gpu = _has_gpu()
    skip_gpu = pytest.mark.skip(reason="needs a B200 GPU")
    for item in items:
        if "gpu" in item.keywords and not has_gpu:
            item.add_marker(skip_gpu)
    # The allocator tests count segments of the process-wide caching allocator: they run before tests that leave
    # device tensors behind for the life of the process (TorchScript keeps the constants of frozen modules in its
    # global compilation unit).
    first = [i for i in items if i.fspath.basename == "test_runtime.py"]
    rest = [i for i in items if i.fspath.basename != "test_runtime.py"]
    items[:] = first + rest


@pytest.fixture(scope="session")
def b200():
    import torch
    import catch_b200  # noqa: F401

    return torch.b200


@pytest.fixture(scope="session")
def dev():
    import catch_b200  # noqa: F401

    return "blackwell"

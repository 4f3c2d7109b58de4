import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _engine_device_follows_the_marker(request, monkeypatch):
    """Several CPU test modules pin ``VERL_ENGINE_DEVICE=cpu`` in ``os.environ`` when they are imported, and pytest imports
    every module of the directory at collection, whatever ``-m`` selects. A test marked ``gpu`` therefore drops the pin
    for its own duration (and for the child processes it starts), so its engines are built on the CUDA device."""
    if request.node.get_closest_marker("gpu") is not None:
        monkeypatch.delenv("VERL_ENGINE_DEVICE", raising=False)
        monkeypatch.delenv("VERL_PLATFORM", raising=False)
    yield

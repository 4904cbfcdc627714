"""Shared fixtures: the two tiny configurations, model folders with random weights in temporary
folders, and the plain implementation's logits for them."""
from __future__ import annotations

import os
import sys

import pytest

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    """Without a GPU the gpu-marked tests are skipped rather than failed."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


from tiny_models import TINY  # noqa: E402


@pytest.fixture(scope="session", params=sorted(TINY))
def tiny(request, tmp_path_factory):
    """A tiny model folder: (name, folder, settings)."""
    from tiny_models import make_folder
    name = request.param
    folder = make_folder(name, str(tmp_path_factory.mktemp(f"tiny_{name}")))
    return name, folder, TINY[name]

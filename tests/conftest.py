"""Shared pytest configuration: the ``gpu`` marker and repository paths."""

from __future__ import annotations

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


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


@pytest.fixture(scope="session")
def golden_small():
    import torch
    return torch.load(os.path.join(GOLDEN, "small.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_config1():
    import torch
    return torch.load(os.path.join(GOLDEN, "config1.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_sampled():
    import torch
    return torch.load(os.path.join(GOLDEN, "sampled.pt"), weights_only=False)

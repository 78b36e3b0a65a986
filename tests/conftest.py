"""Shared fixtures.  Tests marked ``gpu`` need a CUDA device and the compiled kernels; all others run on
the CPU."""
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


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a temporary folder."""
    from tiny_models import write_tiny

    root = tmp_path_factory.mktemp("tiny_models")
    return {w: write_tiny(str(root / w), w) for w in ("a", "b", "c", "d", "e")}

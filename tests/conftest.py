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
    config.addinivalue_line("markers", "expects_a_recorded_index: the test itself reads the bounds-checked build's record")


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


@pytest.fixture(autouse=True)
def no_index_outside_its_array(request):
    """When the kernels are built with their index checks (FMS_B200_DEBUG_BOUNDS=1), every GPU test also fails if a
    kernel computed an index outside its array (the access was skipped and recorded)."""
    yield
    if "gpu" not in request.keywords:
        return
    from fms_b200.kernels import build

    if build.DEBUG_BOUNDS and "expects_a_recorded_index" not in request.keywords:
        assert build.bounds_violations() == []

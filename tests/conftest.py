"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


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
def oracle():
    from oracle.binding import Oracle, build

    build(reference=os.path.isdir("/root/reference"))
    return Oracle()


@pytest.fixture(scope="session")
def ref_floor():
    from oracle.binding import RefFloor

    if not RefFloor.available():
        pytest.skip("oracle/_ref/libhyle_ref_floor.so was not built (reference tree absent)")
    return RefFloor()


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "ref_floor.npz")
    return np.load(path)

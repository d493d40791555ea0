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


def reference_tree() -> str:
    """Where the reference project is mounted (absent on a GPU box): $HYLE_REF, else the default mount."""
    from oracle.binding import reference_root

    return reference_root()


GUARD_BYTES = 4096
GUARD_PATTERN = 0xA5


class GuardedOutputs:
    """Places every output tensor between two bands of a known byte pattern.

    The payload starts 4096 bytes into a private buffer and the trailing band starts at the
    payload's last byte + 1, so a kernel that writes even one element before the start or past a
    ragged tail changes a band.  `check()` compares every band with the pattern."""

    def __init__(self):
        self.buffers = []

    def allocate(self, shape, dtype, device):
        import torch

        count = 1
        for extent in shape:
            count *= int(extent)
        payload = count * torch.empty(0, dtype=dtype).element_size()
        raw = torch.full((2 * GUARD_BYTES + payload,), GUARD_PATTERN, dtype=torch.uint8, device=device)
        self.buffers.append((raw, payload))
        return raw[GUARD_BYTES:GUARD_BYTES + payload].view(dtype).reshape(shape)

    def guarded(self, shape, dtype, device="cuda"):
        """An output tensor for entry points called with explicit outputs."""
        return self.allocate(tuple(shape) if not isinstance(shape, int) else (shape,), dtype, device)

    def check(self):
        import torch

        torch.cuda.synchronize()
        for raw, payload in self.buffers:
            front = raw[:GUARD_BYTES]
            back = raw[GUARD_BYTES + payload:]
            assert bool((front == GUARD_PATTERN).all()), "a kernel wrote BEFORE the start of an output tensor"
            assert bool((back == GUARD_PATTERN).all()), "a kernel wrote PAST the end of an output tensor"
        self.buffers.clear()


@pytest.fixture(autouse=True)
def guard_bands(request):
    """Every `-m gpu` test: outputs the operators allocate sit between guard bands that are checked
    when the test ends (the stand-in for a memory checker on machines where none may run)."""
    if "gpu" not in request.keywords:
        yield None
        return
    import torch

    if not torch.cuda.is_available():
        yield None
        return
    from hyle_b200 import ops

    guards = GuardedOutputs()
    previous = ops.set_output_allocator(guards.allocate)
    try:
        yield guards
        guards.check()
    finally:
        ops.set_output_allocator(previous)


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle, build

    build(reference=os.path.isdir(reference_tree()))
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

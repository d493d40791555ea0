"""The C++23 provider adapter (hyle_b200/provider) against the REFERENCE's own runtime.

`tests/provider/cold_path_test.cc` registers the adapter with `make_custom_provider`, creates a
reference `Context` and calls the reference's `compute::prepare` for every operator of the path: the
provider must be selected for its domain and decline (Status::Unimplemented) outside it.  The program
links the reference's compute core compiled in place from the reference tree, so it is built only
where that tree is mounted; elsewhere the prebuilt binary (oracle/_ref/provider, which travels) is run.
"""
import os
import subprocess

import pytest

from oracle.binding import make_environment, reference_root

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROVIDER_TESTS = os.path.join(ROOT, "tests", "provider")
BINARIES = os.path.join(ROOT, "oracle", "_ref", "provider")


def build_provider_tests():
    """Compile both test programs where the reference tree is mounted; returns False elsewhere."""
    from hyle_b200.build import build

    build()  # the programs link libhyle_b200.so
    if not os.path.isdir(os.path.join(reference_root(), "include", "hyle")):
        return False
    made = subprocess.run(["make", "-C", PROVIDER_TESTS, "-j", "8"], capture_output=True, text=True, timeout=1800,
                          env=make_environment())
    assert made.returncode == 0, made.stdout[-3000:] + made.stderr[-3000:]
    return True


def test_adapter_is_selected_by_the_reference_runtime():
    build_provider_tests()
    binary = os.path.join(BINARIES, "b200_cold_path_test")
    if not os.path.exists(binary):
        pytest.skip("reference tree absent and no prebuilt oracle/_ref/provider/b200_cold_path_test")
    run = subprocess.run([binary], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "0 failure(s)" in run.stdout
    assert run.stdout.count("ok  ") >= 49 and "FAIL" not in run.stdout


def test_hot_path_program_is_built_with_the_cold_one():
    """The GPU half (tests/test_provider_hot_path.py) runs a prebuilt program: make sure it exists
    wherever the cold one could be built, and that without a GPU it says so instead of failing."""
    if not build_provider_tests():
        pytest.skip("reference tree absent: nothing to build here")
    binary = os.path.join(BINARIES, "b200_hot_path_test")
    assert os.path.exists(binary)
    import torch

    if not torch.cuda.is_available():
        run = subprocess.run([binary], capture_output=True, text=True, timeout=120)
        assert run.returncode == 77 and "needs a GPU" in run.stdout


def test_region_provider_claims_the_fused_recipes_under_graph_compile():
    """`tests/provider/region_test.cc`, CPU half: graph::compile of the reference with the region provider
    claims Binary{kAdd} -> RmsNorm, Unary{kSilu} -> Binary{kMultiply} and Softmax -> Cast + TopK{1} as three
    regions lowered to the provider's custom operators, and declines five near misses."""
    build_provider_tests()
    binary = os.path.join(BINARIES, "b200_region_test")
    if not os.path.exists(binary):
        pytest.skip("reference tree absent and no prebuilt oracle/_ref/provider/b200_region_test")
    run = subprocess.run([binary], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "0 failure(s)" in run.stdout and "FAIL" not in run.stdout
    for line in ("three regions are claimed", "runs as b200-add-rms-norm", "runs as b200-activation-multiply",
                 "runs as b200-greedy-head", "TopK{count=2}: not claimed", "residual sum nobody else reads"):
        assert line in run.stdout

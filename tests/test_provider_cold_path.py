"""The C++23 provider adapter (hyle_b200/provider) against the REFERENCE's own runtime.

`cold_path_test.cc` registers the adapter with `make_custom_provider`, creates a reference
`Context` and calls the reference's `compute::prepare` for every operator of the path: the provider
must be selected for its domain and decline (Status::Unimplemented) outside it.  The program links
the reference's compute core compiled in place from the reference tree, so it is built only where
that tree is mounted; elsewhere the prebuilt binary (baseline/_ref, which travels) is run.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "baseline", "_ref", "b200_cold_path_test")
REFERENCE = "/root/reference"


def test_adapter_is_selected_by_the_reference_runtime():
    from hyle_b200.build import build

    build()  # the test binary links libhyle_b200.so for the host-side workspace query
    if os.path.isdir(os.path.join(REFERENCE, "include", "hyle")):
        made = subprocess.run(["make", "-C", os.path.join(ROOT, "hyle_b200", "provider"), "-j", "8"],
                              capture_output=True, text=True, timeout=1200)
        assert made.returncode == 0, made.stdout[-3000:] + made.stderr[-3000:]
    if not os.path.exists(BINARY):
        pytest.skip("reference tree absent and no prebuilt baseline/_ref/b200_cold_path_test")
    run = subprocess.run([BINARY], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "0 failure(s)" in run.stdout
    assert run.stdout.count("ok  ") >= 49 and "FAIL" not in run.stdout

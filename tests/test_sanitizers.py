"""Host code under AddressSanitizer + UndefinedBehaviorSanitizer.

A device memory checker is not available to these tests, and the reference itself instruments host code
only (cmake/HyleSanitizers.cmake:1-10: HYLE_SANITIZER=asan|tsan|ubsan; device code is not instrumented).
The same is done here for the two host-side parts: the CPU checker (oracle/hyle_oracle.c, against its
golden vectors) and the provider adapter (hyle_b200/provider/*.h under the reference's own runtime, the
programs of tests/provider/).  Device-side writes are covered by the guard bands of tests/conftest.py.
"""
import os
import subprocess
import sys

import pytest

from oracle.binding import ORACLE_DIR, make_environment, reference_root

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARIES = os.path.join(ROOT, "oracle", "_ref", "provider")
REPORTS = ("AddressSanitizer", "runtime error:", "LeakSanitizer")


def asan_runtime():
    found = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True)
    path = found.stdout.strip()
    if found.returncode != 0 or not os.path.isabs(path) or not os.path.exists(path):
        pytest.skip("no ASan runtime beside gcc")
    return path


def test_oracle_golden_vectors_under_asan_and_ubsan():
    runtime = asan_runtime()
    made = subprocess.run(["make", "-C", ORACLE_DIR, "sanitize"], capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stdout[-3000:] + made.stderr[-3000:]
    library = os.path.join(ORACLE_DIR, "_san", "libhyle_oracle_san.so")
    program = ("import sys, pytest, oracle.binding as b; assert b.ORACLE_LIB.endswith('_san.so'), b.ORACLE_LIB; "
               "sys.exit(pytest.main(['-q', '-x', '-p', 'no:cacheprovider', 'tests/test_oracle.py']))")
    # Python itself is not instrumented, so leaks are not reported; every access of the checker is.
    environment = dict(os.environ, LD_PRELOAD=runtime, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0",
                       UBSAN_OPTIONS="print_stacktrace=1", HYLE_ORACLE_LIB=library)
    run = subprocess.run([sys.executable, "-c", program], capture_output=True, text=True, timeout=900, cwd=ROOT,
                         env=environment)
    text = run.stdout + run.stderr
    assert run.returncode == 0, text[-4000:]
    assert " passed" in run.stdout and not any(word in text for word in REPORTS), text[-4000:]


@pytest.mark.parametrize("program, marker", [("b200_cold_path_test_san", "0 failure(s)"),
                                             ("b200_region_test_san", "0 failure(s)")])
def test_adapter_programs_under_asan_and_ubsan(program, marker):
    """The cold path (propose / prepare / decline for every operator) and graph::compile with the region
    provider, adapter code instrumented, leak check on."""
    asan_runtime()
    from hyle_b200.build import build

    build()
    if os.path.isdir(os.path.join(reference_root(), "include", "hyle")):
        made = subprocess.run(["make", "-C", os.path.join(ROOT, "tests", "provider"), "-j", "8", "sanitize"],
                              capture_output=True, text=True, timeout=1800, env=make_environment())
        assert made.returncode == 0, made.stdout[-3000:] + made.stderr[-3000:]
    binary = os.path.join(BINARIES, program)
    if not os.path.exists(binary):
        pytest.skip("reference tree absent and no prebuilt " + program)
    run = subprocess.run([binary], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="print_stacktrace=1",
                                  CUDA_VISIBLE_DEVICES=""))  # the CPU halves only: no device work under ASan
    text = run.stdout + run.stderr
    assert run.returncode == 0, text[-4000:]
    assert marker in run.stdout and "FAIL" not in run.stdout
    assert not any(word in text for word in REPORTS), text[-4000:]

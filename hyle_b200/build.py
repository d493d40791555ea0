"""Compile the sm_100a kernel library in-tree (``hyle_b200/libhyle_b200.so``).

nvcc cross-compiles without a GPU.  Run as ``python -m hyle_b200.build``.
"""
from __future__ import annotations

import os
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PACKAGE_DIR, "csrc")
LIBRARY_PATH = os.path.join(PACKAGE_DIR, "libhyle_b200.so")


def build(verbose: bool = False, ptxas_verbose: bool = False) -> str:
    """Run the Makefile in ``csrc``; returns the path of the built library."""
    command = ["make", "-C", CSRC_DIR, "-j", str(os.cpu_count() or 4)]
    if ptxas_verbose:
        command.append("PTXAS_V=1")
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout)
        sys.stderr.write(result.stderr)
    if result.returncode != 0:
        raise RuntimeError("building libhyle_b200.so failed (see compiler output above)")
    if not os.path.exists(LIBRARY_PATH):
        raise RuntimeError(f"make succeeded but {LIBRARY_PATH} is missing")
    return LIBRARY_PATH


if __name__ == "__main__":
    print(build(verbose=True, ptxas_verbose="--ptxas-v" in sys.argv))

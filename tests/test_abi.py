"""The C-ABI library builds for sm_100a, loads without a GPU and exports what the header declares."""
import ctypes
import os
import re

import pytest

from hyle_b200 import abi
from hyle_b200.build import LIBRARY_PATH, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hyle_b200.h")


@pytest.fixture(scope="module")
def library():
    build()
    return abi.load()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"HYLE_B200_API\s+[\w\s\*]*?\b(hyle_b200_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert len(names) >= 16
    assert names == sorted(abi.SIGNATURES), "binding and include/hyle_b200.h list different entry points"


def test_library_exports_every_declared_symbol(library):
    raw = ctypes.CDLL(LIBRARY_PATH)
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"


def test_version_strings_and_pure_host_queries(library):
    assert library.hyle_b200_abi_version() == abi.ABI_VERSION
    assert library.hyle_b200_result_string(0) == b"ok"
    assert b"invalid" in library.hyle_b200_result_string(abi.INVALID_VALUE)
    assert b"not supported" in library.hyle_b200_result_string(abi.NOT_SUPPORTED)
    assert library.hyle_b200_sum_squares_workspace_bytes(0) >= 64 + 8 * 148
    # one f64 per tile of 8192 values on top of the fixed part
    grown = library.hyle_b200_sum_squares_workspace_bytes(1 << 31) - library.hyle_b200_sum_squares_workspace_bytes(0)
    assert (1 << 31) // 8192 * 8 <= grown <= (1 << 31) // 8192 * 8 * 1.02


def test_argument_errors_are_reported_before_any_launch(library):
    """Null pointers and bad counts return cudaErrorInvalidValue without touching a device."""
    L = library
    assert L.hyle_b200_binary(None, 0, 0, None, None, None, 16, 16) == abi.INVALID_VALUE
    assert L.hyle_b200_binary(None, 0, 0, 1 << 20, 1 << 20, 1 << 20, 16, 5) == abi.INVALID_VALUE  # 16 % 5
    assert L.hyle_b200_binary(None, 9, 0, 1 << 20, 1 << 20, 1 << 20, 16, 16) == abi.INVALID_VALUE  # kind
    assert L.hyle_b200_reduce_rows_f32(None, 7, 1 << 20, 1 << 20, 4, 4) == abi.INVALID_VALUE
    assert L.hyle_b200_q8_0_encode(None, abi.BF16, 1 << 20, 33, 1 << 20, None) == abi.INVALID_VALUE  # not /32
    assert L.hyle_b200_q8_0_roundtrip_bf16(None, 1 << 20, 64, 1 << 20, 1 << 20, 1 << 20, None, 1 << 20, 8) == abi.INVALID_VALUE
    assert L.hyle_b200_logits_reduce_f32(None, None, 4, 4, None, None, None, None, None, 0, None) == abi.INVALID_VALUE
    assert L.hyle_b200_workspace_clear(None, None, 64) == abi.INVALID_VALUE
    assert L.hyle_b200_workspace_clear(None, None, 0) == abi.OK
    # empty work is a successful no-op
    assert L.hyle_b200_binary(None, 0, 0, None, None, None, 0, 1) == abi.OK
    assert L.hyle_b200_swiglu_bf16(None, None, None, None, 0, 0, 0, 0) == abi.OK


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(abi, "_library", None)
    monkeypatch.setattr(abi, "LIBRARY_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(abi.LibraryMissing):
        abi.load()


def test_ops_refuse_cpu_tensors(library):
    import torch
    from hyle_b200 import ops

    with pytest.raises(ValueError):
        ops.add(torch.zeros(4), torch.zeros(4))

"""ctypes binding of the C ABI declared in ``include/hyle_b200.h``.

This module is plumbing: it loads ``libhyle_b200.so`` and declares argument types.  It never
falls back to another implementation; a missing library is an ImportError-like failure at the
first call (``load()``), so GPU code paths cannot silently run on something else.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIBRARY_PATH

# enum hyle_b200_dtype
F32, BF16, F16, E4M3, E5M2, BOOL, I32 = 0, 1, 2, 3, 4, 5, 6
# enum hyle_b200_binary_kind
BINARY_ADD, BINARY_MULTIPLY, BINARY_SUBTRACT, BINARY_DIVIDE, BINARY_MINIMUM, BINARY_MAXIMUM = 0, 1, 2, 3, 4, 5
# enum hyle_b200_unary_kind
GATE_SILU, GATE_GELU, GATE_GELU_TANH = 0, 1, 2  # hyle_b200_gate_kind
(UNARY_ABS, UNARY_NEG, UNARY_EXP, UNARY_LOG, UNARY_SQRT, UNARY_RSQRT, UNARY_TANH, UNARY_SIGMOID, UNARY_RELU,
 UNARY_GELU, UNARY_GELU_TANH, UNARY_SILU, UNARY_SOFTPLUS) = range(13)
# enum hyle_b200_reduce_kind
REDUCE_SUM, REDUCE_MEAN, REDUCE_MINIMUM, REDUCE_MAXIMUM = 0, 1, 2, 3
# enum hyle_b200_softmax_kind
SOFTMAX, LOG_SOFTMAX = 0, 1
# enum hyle_b200_result
OK, INVALID_VALUE, NOT_SUPPORTED, STATIC_SCRATCH_EXCEEDED, IO_ERROR = 0, 1, 801, 100001, 100002
STATIC_MAX_VALUES = 1 << 31
# enum hyle_b200_status_bits
STATUS_INVALID_Q8_INPUT = 1
STATUS_EXCHANGE_TIMEOUT = 2
STATUS_INVALID_FP8_INPUT = 4
STATUS_INVALID_CATEGORICAL_ROW = 8
STATUS_SCAN_OVERFLOW = 16
STATUS_STREAM_WAIT_TIMEOUT = 32
EXCHANGE_MAX_RANKS, EXCHANGE_MAILBOX_BYTES, EXCHANGE_HANDLE_BYTES = 8, 256, 64

ABI_VERSION = 20

_p = ctypes.c_void_p
_u64 = ctypes.c_uint64
_i = ctypes.c_int
_f = ctypes.c_float
_u32 = ctypes.c_uint32

# name -> (restype, argtypes); the complete export list of include/hyle_b200.h
SIGNATURES = {
    "hyle_b200_abi_version": (_i, []),
    "hyle_b200_result_string": (ctypes.c_char_p, [_i]),
    "hyle_b200_binary": (_i, [_p, _i, _i, _p, _p, _p, _u64, _u64]),
    "hyle_b200_unary": (_i, [_p, _i, _i, _p, _p, _u64]),
    "hyle_b200_reduce_rows_f32": (_i, [_p, _i, _p, _p, _u64, _u64]),
    "hyle_b200_add_bias_row_sum_max_f32": (_i, [_p, _p, _p, _p, _p, _p, _u64, _u64]),
    "hyle_b200_rms_norm_bf16": (_i, [_p, _p, _p, _i, _p, _u64, _u64, _f]),
    "hyle_b200_add_rms_norm_bf16": (_i, [_p, _p, _p, _p, _i, _p, _p, _u64, _u64, _f]),
    "hyle_b200_layer_norm_bf16": (_i, [_p, _p, _p, _p, _p, _u64, _u64, _f]),
    "hyle_b200_swiglu_bf16": (_i, [_p, _p, _p, _p, _u64, _u64, _u64, _u64]),
    "hyle_b200_gated_activation": (_i, [_p, _i, _i, _i, _p, _p, _p, _u64, _u64, _u64, _u64]),
    "hyle_b200_logits_workspace_bytes": (_u64, [_u64, _u64]),
    "hyle_b200_logits_reduce_f32": (_i, [_p, _p, _u64, _u64, _p, _p, _p, _p, _p, _u64, _p]),
    "hyle_b200_logits_reduce_f32_tuned": (_i, [_p, _p, _u64, _u64, _p, _p, _p, _p, _p, _u64, _p, _p]),
    "hyle_b200_logits_stream_plan": (_i, [_u64, _u64, _p, _p]),
    "hyle_b200_logits_stream_task": (_i, [_u64, _u32, _u32, _u64, _p, _p, _p]),
    "hyle_b200_softmax_f32": (_i, [_p, _i, _p, _p, _u64, _u64, _p, _u64, _p]),
    "hyle_b200_workspace_clear": (_i, [_p, _p, _u64]),
    "hyle_b200_select": (_i, [_p, _i, _p, _p, _p, _p, _u64, _u64, _u64]),
    "hyle_b200_cast": (_i, [_p, _i, _i, _p, _p, _u64]),
    "hyle_b200_masked_softmax_f16": (_i, [_p, _p, _p, _u64, _f, _p, _u64, _u64]),
    "hyle_b200_reduce_rows_extremum": (_i, [_p, _i, _i, _p, _p, _u64, _u64]),
    "hyle_b200_selfcheck_q8_0_scale": (_i, [_p, _p]),
    "hyle_b200_rms_norm": (_i, [_p, _i, _p, _p, _i, _p, _u64, _u64, _f]),
    "hyle_b200_additive_masked_softmax_f16": (_i, [_p, _p, _p, _u64, _f, _p, _u64, _u64]),
    "hyle_b200_cast_f32_to_bf16": (_i, [_p, _p, _p, _u64]),
    "hyle_b200_q8_0_encode": (_i, [_p, _i, _p, _u64, _p, _p]),
    "hyle_b200_fp8_e4m3_encode": (_i, [_p, _i, _p, _u64, _f, _p, _p]),
    "hyle_b200_strided_cast": (_i, [_p, _i, _i, _p, _p, _u32, _p, _p]),
    "hyle_b200_strided_scatter": (_i, [_p, _i, _p, _p, _u32, _p, _p]),
    "hyle_b200_scan": (_i, [_p, _i, _p, _p, _u64, _u64, _i, _p]),
    "hyle_b200_paged_append": (_i, [_p, _p, _p, _p, _u32, _u32, _u32, _u32, _u64]),
    "hyle_b200_paged_append_device_lengths": (_i, [_p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32, _u64, _u32, _p]),
    "hyle_b200_q8_0_decode_bf16": (_i, [_p, _p, _u64, _p]),
    "hyle_b200_sum_squares_workspace_bytes": (_u64, [_u64]),
    "hyle_b200_sum_squares_bf16": (_i, [_p, _p, _u64, _p, _p, _u64]),
    "hyle_b200_q8_0_roundtrip_bf16": (_i, [_p, _p, _u64, _p, _p, _p, _p, _p, _u64]),
    "hyle_b200_q8_0_roundtrip_bf16_static": (_i, [_p, _p, _u64, _p, _p, _p, _p]),
    "hyle_b200_q8_0_roundtrip_bf16_exchange": (_i, [_p, _p, _u64, _p, _p, _p, _p, _p, _u64,
                                                     ctypes.POINTER(_p), _u32, _u32, _u32, _u32]),
    "hyle_b200_exchange_create": (_i, [ctypes.POINTER(_p), ctypes.c_char_p]),
    "hyle_b200_exchange_open": (_i, [ctypes.c_char_p, ctypes.POINTER(_p)]),
    "hyle_b200_exchange_close": (_i, [_p]),
    "hyle_b200_exchange_destroy": (_i, [_p]),
    "hyle_b200_file_stream_open": (_i, [ctypes.c_char_p, _u64, _u64, _p, ctypes.POINTER(_p)]),
    "hyle_b200_file_stream_read_group": (_i, [_p, _p, _p, _u32]),
    "hyle_b200_file_stream_next": (_i, [_p, _p, ctypes.POINTER(_p), ctypes.POINTER(_u64), ctypes.POINTER(_u64)]),
    "hyle_b200_file_stream_get_report": (_i, [_p, _p]),
    "hyle_b200_file_stream_close": (_i, [_p]),
    "hyle_b200_q8_0_decode_file_bf16": (_i, [_p, ctypes.c_char_p, _u64, _u64, _p, _p, _p]),
    "hyle_b200_random_bits": (_i, [_p, _p, _u64, _u32, _p]),
    "hyle_b200_categorical": (_i, [_p, _i, _p, _p, _u64, _u64, _p, _p, _p]),
}



class StreamTuning(ctypes.Structure):
    """hyle_b200_stream_tuning: zero fields mean "choose"."""
    _fields_ = [("chunk_vectors", ctypes.c_int32), ("window_rows", _u32), ("help_after_polls", _u32),
                ("ctas_per_sm", ctypes.c_int32)]


class FileStreamOptions(ctypes.Structure):
    """hyle_b200_file_stream_options: zero fields take the defaults (8 MiB chunks, 4 slots)."""
    _fields_ = [("chunk_bytes", _u64), ("slots", _u32), ("readers", _u32), ("chunk_granule", _u64)]


class FileRange(ctypes.Structure):
    """hyle_b200_file_range."""
    _fields_ = [("file_offset", _u64), ("bytes", _u64), ("destination", ctypes.c_void_p)]


class FileStreamReport(ctypes.Structure):
    """hyle_b200_file_stream_report."""
    _fields_ = [(name, _u64) for name in ("bytes_read", "bytes_copied", "io_calls", "copies", "staging_bytes", "device_bytes",
                                           "chunk_bytes", "chunks")]


class StreamPlan(ctypes.Structure):
    """hyle_b200_stream_plan."""
    _fields_ = [("chunk_vectors", ctypes.c_int32), ("chunks_per_row", _u32), ("chunk_values", _u32),
                ("window_rows", _u32), ("fixed_tasks_per_cta", _u32), ("ctas_per_sm", ctypes.c_int32),
                ("grid", _u32), ("help_after_polls", _u32)]


_library = None


class LibraryMissing(RuntimeError):
    """libhyle_b200.so is not built; there is no other implementation to fall back to."""


def load() -> ctypes.CDLL:
    """Load the kernel library once and declare every entry point's signature."""
    global _library
    if _library is not None:
        return _library
    if not os.path.exists(LIBRARY_PATH):
        raise LibraryMissing(
            f"{LIBRARY_PATH} not found: build it with `python -m hyle_b200.build` "
            "(there is no CPU or framework fallback for these operators)")
    library = ctypes.CDLL(LIBRARY_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(library, name)  # AttributeError if the export is missing
        function.restype = restype
        function.argtypes = argtypes
    version = library.hyle_b200_abi_version()
    if version != ABI_VERSION:
        raise RuntimeError(f"libhyle_b200.so has ABI version {version}, binding expects {ABI_VERSION}")
    _library = library
    return library


class KernelError(RuntimeError):
    def __init__(self, function: str, code: int):
        self.code = code
        text = load().hyle_b200_result_string(code).decode()
        super().__init__(f"{function} failed: {code} ({text})")


def check(function: str, code: int) -> None:
    if code != OK:
        raise KernelError(function, code)

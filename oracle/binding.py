"""ctypes binding of the CPU checker libraries -- TEST INFRASTRUCTURE.

``Oracle``   oracle/libhyle_oracle.so, the from-scratch restatement (hyle_oracle.c), numpy in/out.
``RefFloor`` oracle/_ref/libhyle_ref_floor.so, the reference's own scalar floor compiled from the
             reference tree (ref_floor_shim.cc); present only where it was built.
Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
# HYLE_ORACLE_LIB: another build of the same file (the sanitizer build of tests/test_sanitizers.py).
ORACLE_LIB = os.environ.get("HYLE_ORACLE_LIB") or os.path.join(ORACLE_DIR, "libhyle_oracle.so")
REF_LIB = os.path.join(ORACLE_DIR, "_ref", "libhyle_ref_floor.so")
REF_PAGED_LIB = os.path.join(ORACLE_DIR, "_ref", "libhyle_ref_paged.so")

F32, BF16, F16 = 0, 1, 2
ADD, MULTIPLY, SUBTRACT, DIVIDE, NUMBER_MINIMUM, NUMBER_MAXIMUM = 0, 1, 2, 3, 4, 5  # Binary kinds
E4M3, E5M2, BOOL, I32 = 3, 4, 5, 6  # storage types of Cast, after F32, BF16, F16
CAST_WORD = {0: np.float32, 1: np.uint16, 2: np.uint16, 3: np.uint8, 4: np.uint8, 5: np.uint8, 6: np.int32}
(ABS, NEG, EXP, LOG, SQRT, RSQRT, TANH, SIGMOID, RELU, GELU, GELU_TANH, SILU, SOFTPLUS) = range(13)  # Unary kinds
SUM, MEAN, MINIMUM, MAXIMUM = 0, 1, 2, 3

_vp, _u64, _i, _f = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_float


def reference_root() -> str:
    """Where the reference project's source tree is mounted: ``$HYLE_REF``, else the build machine's
    mount point.  The one place that default is written; every Makefile takes HYLE_REF from here."""
    return os.environ.get("HYLE_REF", "/root/reference")


def make_environment() -> dict:
    """The environment for the Makefiles that compile reference sources in place."""
    return dict(os.environ, HYLE_REF=reference_root())


def build(reference: bool = True) -> None:
    """Compile the checker (and the reference floor when the reference tree is mounted)."""
    target = "all" if reference else "libhyle_oracle.so"
    result = subprocess.run(["make", "-C", ORACLE_DIR, target], capture_output=True, text=True,
                            env=make_environment())
    if result.returncode != 0:
        raise RuntimeError("building the oracle failed:\n" + result.stdout + result.stderr)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_LIB):
            build(reference=False)
        self.lib = ctypes.CDLL(ORACLE_LIB)
        L = self.lib
        L.hyle_oracle_max_threads.restype = _i
        L.hyle_oracle_bf16_to_f32.restype = _f
        L.hyle_oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.hyle_oracle_f32_to_bf16.restype = ctypes.c_uint16
        L.hyle_oracle_f32_to_bf16.argtypes = [_f]
        L.hyle_oracle_f16_to_f32.restype = _f
        L.hyle_oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.hyle_oracle_f32_to_f16.restype = ctypes.c_uint16
        L.hyle_oracle_f32_to_f16.argtypes = [_f]
        L.hyle_oracle_binary.argtypes = [_i, _i, _vp, _vp, _vp, _u64, _u64]
        L.hyle_oracle_unary.argtypes = [_i, _i, _vp, _vp, _u64]
        L.hyle_oracle_cast.argtypes = [_i, _i, _vp, _vp, _u64]
        L.hyle_oracle_cast.restype = _i
        L.hyle_oracle_random_bits.argtypes = [_vp, _u64, ctypes.c_uint32, _vp]
        L.hyle_oracle_categorical.argtypes = [_i, _vp, _vp, _u64, _u64, _vp, _vp, _vp]
        L.hyle_oracle_categorical.restype = _u64
        L.hyle_oracle_fp8_e4m3_encode.argtypes = [_i, _vp, _u64, _f, _vp]
        L.hyle_oracle_fp8_e4m3_encode.restype = ctypes.c_uint32
        _u32 = ctypes.c_uint32
        L.hyle_oracle_paged_append.argtypes = [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _u64]
        L.hyle_oracle_paged_append.restype = None
        L.hyle_oracle_scan_f32.argtypes = [_vp, _vp, _u64, _u64, _i]
        L.hyle_oracle_scan_f32.restype = None
        L.hyle_oracle_scan_i32.argtypes = [_vp, _vp, _u64, _u64, _i]
        L.hyle_oracle_scan_i32.restype = _u32
        L.hyle_oracle_paged_append_device_lengths.argtypes = [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u64, _u32, _u32]
        L.hyle_oracle_paged_append_device_lengths.restype = _u32
        for name in ("e4m3", "e5m2"):
            getattr(L, f"hyle_oracle_f32_to_{name}").argtypes = [_f]
            getattr(L, f"hyle_oracle_f32_to_{name}").restype = ctypes.c_uint8
            getattr(L, f"hyle_oracle_{name}_to_f32").argtypes = [ctypes.c_uint8]
            getattr(L, f"hyle_oracle_{name}_to_f32").restype = _f
        L.hyle_oracle_layer_norm_bf16.argtypes = [_vp, _vp, _vp, _vp, _vp, _u64, _u64, _f]
        L.hyle_oracle_reduce_rows_f32.argtypes = [_i, _vp, _vp, _u64, _u64]
        L.hyle_oracle_row_sum_f64.argtypes = [_vp, _vp, _vp, _u64, _u64]
        L.hyle_oracle_rms_norm_bf16.argtypes = [_vp, _vp, _i, _vp, _vp, _u64, _u64, _f]
        L.hyle_oracle_rms_norm.argtypes = [_i, _vp, _vp, _i, _vp, _vp, _u64, _u64, _f]
        L.hyle_oracle_add_rms_norm_bf16.argtypes = [_vp, _vp, _vp, _i, _vp, _vp, _vp, _u64, _u64, _f]
        L.hyle_oracle_swiglu_bf16.argtypes = [_vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64]
        L.hyle_oracle_gated_activation.argtypes = [_i, _i, _i, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64]
        L.hyle_oracle_softmax_f32.argtypes = [_i, _vp, _vp, _u64, _u64]
        L.hyle_oracle_argmax_f32.argtypes = [_vp, _vp, _vp, _u64, _u64]
        L.hyle_oracle_logits_reduce_f32.argtypes = [_vp, _u64, _u64, _vp, _vp, _vp, _vp, _vp]
        L.hyle_oracle_cast_f32_to_bf16.argtypes = [_vp, _vp, _u64]
        L.hyle_oracle_q8_0_encode.restype = _i
        L.hyle_oracle_q8_0_encode.argtypes = [_i, _vp, _u64, _vp]
        L.hyle_oracle_q8_0_decode_bf16.argtypes = [_vp, _u64, _vp]
        L.hyle_oracle_sum_squares_bf16.restype = ctypes.c_double
        L.hyle_oracle_sum_squares_bf16.argtypes = [_vp, _u64]
        L.hyle_oracle_q8_0_roundtrip_bf16.restype = _i
        L.hyle_oracle_q8_0_roundtrip_bf16.argtypes = [_vp, _u64, _vp, _vp, _vp]

    # bf16 / f16 arrays are numpy uint16 storage words throughout.
    def set_threads(self, n: int) -> None:
        self.lib.hyle_oracle_set_threads(int(n))

    def max_threads(self) -> int:
        return self.lib.hyle_oracle_max_threads()

    def f32_to_bf16(self, x):
        x = _c(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.lib.hyle_oracle_cast_f32_to_bf16(_ptr(x), _ptr(out), x.size)
        return out

    def bf16_to_f32(self, x):
        return (_c(x, np.uint16).astype(np.uint32) << 16).view(np.float32)

    def f32_to_f16_scalar(self, v: float) -> int:
        return self.lib.hyle_oracle_f32_to_f16(float(v))

    def f16_to_f32_scalar(self, h: int) -> float:
        return self.lib.hyle_oracle_f16_to_f32(int(h))

    def f32_to_bf16_scalar(self, v: float) -> int:
        return self.lib.hyle_oracle_f32_to_bf16(float(v))

    def binary(self, kind, dtype, lhs, rhs):
        np_dtype = np.float32 if dtype == F32 else np.uint16
        lhs, rhs = _c(lhs, np_dtype), _c(rhs, np_dtype)
        out = np.empty_like(lhs)
        self.lib.hyle_oracle_binary(kind, dtype, _ptr(lhs), _ptr(rhs), _ptr(out), lhs.size, max(rhs.size, 1))
        return out

    def unary(self, kind, dtype, x):
        np_dtype = np.float32 if dtype == F32 else np.uint16
        x = _c(x, np_dtype)
        out = np.empty_like(x)
        self.lib.hyle_oracle_unary(kind, dtype, _ptr(x), _ptr(out), x.size)
        return out

    def cast(self, src, dst, x):
        """Cast between storage types; x and the result are arrays of the storage words."""
        x = _c(x, CAST_WORD[src])
        out = np.empty(x.shape, CAST_WORD[dst])
        if self.lib.hyle_oracle_cast(src, dst, _ptr(x), _ptr(out), x.size) != 0:
            raise ValueError(f"no Cast from {src} to {dst} on the CPU route")
        return out

    def fp8_e4m3_encode(self, dtype, x, scale):
        x = _c(x, np.float32 if dtype == F32 else np.uint16)
        out = np.empty(x.shape, np.uint8)
        status = self.lib.hyle_oracle_fp8_e4m3_encode(dtype, _ptr(x), x.size, scale, _ptr(out))
        return out, int(status)

    def scan(self, x, exclusive=False):
        """(prefix sums along the last axis, status): f32 summed left to right in float; i32 exact, with
        status 16 and an untouched (zero) result when a prefix leaves the int32 range."""
        x = np.ascontiguousarray(x)
        cols = x.shape[-1]
        rows = x.size // cols if cols else 0
        out = np.zeros_like(x)
        if x.dtype == np.float32:
            self.lib.hyle_oracle_scan_f32(_ptr(x), _ptr(out), rows, cols, int(exclusive))
            return out, 0
        assert x.dtype == np.int32
        return out, int(self.lib.hyle_oracle_scan_i32(_ptr(x), _ptr(out), rows, cols, int(exclusive)))

    def paged_append(self, arena, new_rows, words, page_rows):
        """Returns the arena [pages * page_rows, row bytes] (uint8) after the episode ``words`` (uint32)."""
        arena = np.array(arena, dtype=np.uint8, order="C", copy=True)
        new_rows = _c(new_rows, np.uint8) if new_rows is not None else np.zeros((0, arena.shape[1]), np.uint8)
        words = _c(words, np.uint32)
        self.lib.hyle_oracle_paged_append(_ptr(arena), _ptr(new_rows), _ptr(words), page_rows, arena.shape[0] // page_rows,
                                          new_rows.shape[0], (words.size - 4) // 8, arena.shape[1])
        return arena

    def paged_append_device_lengths(self, arena, new_rows, words, query_lengths, kv_lengths, page_rows, status=0):
        """(arena after the episode, status word after it) for the device-lengths records ``words``."""
        arena = np.array(arena, dtype=np.uint8, order="C", copy=True)
        new_rows, words = _c(new_rows, np.uint8), _c(words, np.uint32)
        q, kv = _c(query_lengths, np.int32), _c(kv_lengths, np.int32)
        status = self.lib.hyle_oracle_paged_append_device_lengths(
            _ptr(arena), _ptr(new_rows), _ptr(words), _ptr(q), _ptr(kv), page_rows, arena.shape[0] // page_rows,
            new_rows.shape[0], (words.size - 4) // 8, arena.shape[1], q.size, status)
        return arena, int(status)

    def random_bits(self, identities, words):
        identities = _c(identities, np.uint32)
        rows = identities.shape[0]
        out = np.empty((rows, words), np.uint32)
        self.lib.hyle_oracle_random_bits(_ptr(identities), rows, words, _ptr(out))
        return out

    def categorical(self, dtype, logits, identities):
        """(index i32[rows], log p f32[rows], uniform f64[rows], invalid rows)"""
        logits = _c(logits, np.float32 if dtype == F32 else np.uint16)
        identities = _c(identities, np.uint32)
        rows, cols = logits.shape
        index, logp, uniform = np.empty(rows, np.int32), np.empty(rows, np.float32), np.empty(rows, np.float64)
        invalid = self.lib.hyle_oracle_categorical(dtype, _ptr(logits), _ptr(identities), rows, cols, _ptr(index), _ptr(logp), _ptr(uniform))
        return index, logp, uniform, int(invalid)

    def masked_softmax_f16(self, x16, mask, scale):
        """Softmax{scale, Boolean mask} on f16 rows (src/compute_provider_native/transformer.cc:44-57): f32 value times
        scale, -inf where the mask byte is 0, the pinned f32 softmax, one rounding to f16.  Returns (f16 words, f32)."""
        x16 = _c(x16, np.uint16)
        values = x16.view(np.float16).astype(np.float32) * np.float32(scale)
        mask = np.asarray(mask)
        if mask.dtype == np.float16:
            # MaskKind::kAdditive: the addend joins after the scaling, each step rounded to f32
            # (src/compute_provider_cuda/reduction_kernel.cu:131-146)
            with np.errstate(all="ignore"):
                values = (values + np.broadcast_to(mask.astype(np.float32), values.shape)).astype(np.float32)
        else:
            values = np.where(np.broadcast_to(mask != 0, values.shape), values, np.float32(-np.inf)).astype(np.float32)
        shape = values.shape
        y = self.softmax(values.reshape(-1, shape[-1])).reshape(shape)
        with np.errstate(all="ignore"):
            return y.astype(np.float16).view(np.uint16), y

    def reduce_rows(self, kind, x):
        x = _c(x, np.float32)
        rows, cols = x.shape
        out = np.empty(rows, np.float32)
        self.lib.hyle_oracle_reduce_rows_f32(kind, _ptr(x), _ptr(out), rows, cols)
        return out

    def reduce_rows_narrow(self, kind, dtype, words):
        """Minimum / Maximum of bf16 or f16 rows in the rows' type (src/compute_provider_native/reduction.cc:203-223):
        the f32 reduction on the exactly converted values; an extremum is one of them, so it converts back unchanged
        (NaN becomes the canonical quiet NaN of the type)."""
        words = _c(words, np.uint16)
        return self.cast(F32, dtype, self.reduce_rows(kind, self.cast(dtype, F32, words).view(np.float32)))

    def row_sum_f64(self, x):
        x = _c(x, np.float32)
        rows, cols = x.shape
        s, a = np.empty(rows, np.float64), np.empty(rows, np.float64)
        self.lib.hyle_oracle_row_sum_f64(_ptr(x), _ptr(s), _ptr(a), rows, cols)
        return s, a

    @staticmethod
    def _weight(weight):
        if weight is None:
            return None, BF16
        if weight.dtype == np.float32:
            return np.ascontiguousarray(weight), F32
        return _c(weight, np.uint16), BF16

    def rms_norm(self, x, weight, eps):
        x = _c(x, np.uint16)
        rows, hidden = x.shape
        w, wdt = self._weight(weight)
        y, y32 = np.empty_like(x), np.empty(x.shape, np.float32)
        self.lib.hyle_oracle_rms_norm_bf16(_ptr(x), _ptr(w), wdt, _ptr(y), _ptr(y32), rows, hidden, eps)
        return y, y32

    def rms_norm_stored(self, dtype, x, weight, weight_dtype, eps):
        """RmsNorm on rows stored as `dtype` (F32 / F16 / BF16; 16-bit words for the narrow ones); the weight,
        if any, is stored as `weight_dtype`.  Returns (stored result, f32 before the rounding)."""
        x = _c(x, np.float32 if dtype == F32 else np.uint16)
        rows, hidden = x.shape
        w = None if weight is None else _c(weight, np.float32 if weight_dtype == F32 else np.uint16)
        y, y32 = np.empty_like(x), np.empty(x.shape, np.float32)
        self.lib.hyle_oracle_rms_norm(dtype, _ptr(x), _ptr(w), weight_dtype, _ptr(y), _ptr(y32), rows, hidden, eps)
        return y, y32

    def layer_norm(self, x, scale, bias, eps):
        x = _c(x, np.uint16)
        rows, hidden = x.shape
        scale = None if scale is None else _c(scale, np.uint16)
        bias = None if bias is None else _c(bias, np.uint16)
        y, y32 = np.empty_like(x), np.empty(x.shape, np.float32)
        self.lib.hyle_oracle_layer_norm_bf16(_ptr(x), _ptr(scale), _ptr(bias), _ptr(y), _ptr(y32), rows, hidden, eps)
        return y, y32

    def add_rms_norm(self, x, residual, weight, eps):
        x, residual = _c(x, np.uint16), _c(residual, np.uint16)
        rows, hidden = x.shape
        w, wdt = self._weight(weight)
        y, y32, h = np.empty_like(x), np.empty(x.shape, np.float32), np.empty_like(x)
        self.lib.hyle_oracle_add_rms_norm_bf16(_ptr(x), _ptr(residual), _ptr(w), wdt, _ptr(y), _ptr(y32),
                                               _ptr(h), rows, hidden, eps)
        return y, y32, h

    def swiglu(self, gate, up, cols=None, gate_stride=None, up_stride=None):
        gate, up = _c(gate, np.uint16), _c(up, np.uint16)
        rows = gate.shape[0]
        cols = gate.shape[1] if cols is None else cols
        gate_stride = cols if gate_stride is None else gate_stride
        up_stride = cols if up_stride is None else up_stride
        out, out32 = np.empty((rows, cols), np.uint16), np.empty((rows, cols), np.float32)
        self.lib.hyle_oracle_swiglu_bf16(_ptr(gate), _ptr(up), _ptr(out), _ptr(out32), rows, cols,
                                         gate_stride, up_stride)
        return out, out32

    def gated_activation(self, activation, dtype, gate, up, round_gate=False):
        """(storage words, unrounded f32) of GatedActivation{activation} on bf16 / f16 words [rows, cols]."""
        gate, up = _c(gate, np.uint16), _c(up, np.uint16)
        rows, cols = gate.shape
        out, out32 = np.empty((rows, cols), np.uint16), np.empty((rows, cols), np.float32)
        self.lib.hyle_oracle_gated_activation(activation, dtype, int(round_gate), _ptr(gate), _ptr(up), _ptr(out),
                                              _ptr(out32), rows, cols, cols, cols)
        return out, out32

    def softmax(self, x, log=False):
        x = _c(x, np.float32)
        rows, cols = x.shape
        out = np.empty_like(x)
        self.lib.hyle_oracle_softmax_f32(1 if log else 0, _ptr(x), _ptr(out), rows, cols)
        return out

    def argmax(self, x):
        x = _c(x, np.float32)
        rows, cols = x.shape
        index, value = np.empty(rows, np.int32), np.empty(rows, np.float32)
        self.lib.hyle_oracle_argmax_f32(_ptr(x), _ptr(index), _ptr(value), rows, cols)
        return index, value

    def logits_reduce(self, x, want_probs=True):
        x = _c(x, np.float32)
        rows, cols = x.shape
        lse = np.empty(rows, np.float32)
        index, value = np.empty(rows, np.int32), np.empty(rows, np.float32)
        probs = np.empty(x.shape, np.uint16) if want_probs else None
        probs32 = np.empty(x.shape, np.float32) if want_probs else None
        self.lib.hyle_oracle_logits_reduce_f32(_ptr(x), rows, cols, _ptr(lse), _ptr(probs), _ptr(probs32),
                                               _ptr(index), _ptr(value))
        return lse, probs, probs32, index, value

    def q8_0_encode(self, dtype, x):
        np_dtype = np.float32 if dtype == F32 else np.uint16
        x = _c(x, np_dtype)
        out = np.empty(x.size // 32 * 34, np.uint8)
        invalid = self.lib.hyle_oracle_q8_0_encode(dtype, _ptr(x), x.size, _ptr(out))
        return out, bool(invalid)

    def q8_0_decode(self, blocks, count):
        blocks = _c(blocks, np.uint8)
        out = np.empty(count, np.uint16)
        self.lib.hyle_oracle_q8_0_decode_bf16(_ptr(blocks), count, _ptr(out))
        return out

    def sum_squares(self, x):
        x = _c(x, np.uint16)
        return self.lib.hyle_oracle_sum_squares_bf16(_ptr(x), x.size)

    def q8_0_roundtrip(self, x, blocks=None, decoded=None):
        x = _c(x, np.uint16)
        if blocks is None:
            blocks = np.empty(x.size // 32 * 34, np.uint8)
        if decoded is None:
            decoded = np.empty(x.size, np.uint16)
        total = ctypes.c_double()
        invalid = self.lib.hyle_oracle_q8_0_roundtrip_bf16(_ptr(x), x.size, _ptr(blocks), _ptr(decoded),
                                                           ctypes.byref(total))
        return blocks, decoded, total.value, bool(invalid)


class RefFloor:
    """The reference's own scalar floor (when oracle/_ref was built from the reference tree)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_LIB)

    def __init__(self):
        self.lib = ctypes.CDLL(REF_LIB)
        L = self.lib
        L.hyle_ref_f32_to_bf16.restype = ctypes.c_uint16
        L.hyle_ref_f32_to_bf16.argtypes = [_f]
        L.hyle_ref_bf16_to_f32.restype = _f
        L.hyle_ref_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.hyle_ref_f32_to_f16.restype = ctypes.c_uint16
        L.hyle_ref_f32_to_f16.argtypes = [_f]
        L.hyle_ref_f16_to_f32.restype = _f
        L.hyle_ref_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.hyle_ref_swiglu_bf16.argtypes = [_vp, _vp, _vp, _u64, _u64, _u64, _u64]
        L.hyle_ref_rms_norm_bf16.argtypes = [_vp, _vp, _vp, _u64, _u64, _f]
        L.hyle_ref_softmax_f32.argtypes = [_i, _vp, _vp, _u64, _u64]
        L.hyle_ref_argmax_f32.argtypes = [_vp, _vp, _vp, _u64, _u64]
        L.hyle_ref_activation_f32.argtypes = [_i, _vp, _vp, _u64]
        L.hyle_ref_random_word.argtypes = [_vp, _u64]
        L.hyle_ref_random_word.restype = ctypes.c_uint32
        for name in ("e4m3", "e5m2"):
            getattr(L, f"hyle_ref_f32_to_{name}").argtypes = [_f]
            getattr(L, f"hyle_ref_f32_to_{name}").restype = ctypes.c_uint8
            getattr(L, f"hyle_ref_{name}_to_f32").argtypes = [ctypes.c_uint8]
            getattr(L, f"hyle_ref_{name}_to_f32").restype = _f
        L.hyle_ref_layer_norm_bf16.argtypes = [_vp, _vp, _vp, _vp, _u64, _u64, _f]
        L.hyle_ref_activation_f32.restype = _i

    def set_threads(self, n: int) -> None:
        self.lib.hyle_ref_set_threads(int(n))

    def activation(self, kind, x):
        """sigmoid / relu / gelu / gelu_tanh / silu (UnaryKind numbers 7..11) by the reference's scalar floor."""
        x = _c(x, np.float32)
        out = np.empty_like(x)
        if self.lib.hyle_ref_activation_f32(kind, _ptr(x), _ptr(out), x.size) != 0:
            raise ValueError(f"no reference floor for unary kind {kind}")
        return out

    def swiglu(self, gate, up):
        gate, up = _c(gate, np.uint16), _c(up, np.uint16)
        rows, cols = gate.shape
        out = np.empty_like(gate)
        self.lib.hyle_ref_swiglu_bf16(_ptr(gate), _ptr(up), _ptr(out), rows, cols, cols, cols)
        return out

    def rms_norm(self, x, weight, eps):
        x = _c(x, np.uint16)
        rows, hidden = x.shape
        weight = None if weight is None else _c(weight, np.uint16)
        y = np.empty_like(x)
        self.lib.hyle_ref_rms_norm_bf16(_ptr(x), _ptr(weight), _ptr(y), rows, hidden, eps)
        return y

    def layer_norm(self, x, scale, bias, eps):
        x = _c(x, np.uint16)
        rows, hidden = x.shape
        scale = None if scale is None else _c(scale, np.uint16)
        bias = None if bias is None else _c(bias, np.uint16)
        y = np.empty_like(x)
        self.lib.hyle_ref_layer_norm_bf16(_ptr(x), _ptr(scale), _ptr(bias), _ptr(y), rows, hidden, eps)
        return y

    def softmax(self, x, log=False):
        x = _c(x, np.float32)
        rows, cols = x.shape
        out = np.empty_like(x)
        self.lib.hyle_ref_softmax_f32(1 if log else 0, _ptr(x), _ptr(out), rows, cols)
        return out

    def argmax(self, x):
        x = _c(x, np.float32)
        rows, cols = x.shape
        index, value = np.empty(rows, np.int32), np.empty(rows, np.float32)
        self.lib.hyle_ref_argmax_f32(_ptr(x), _ptr(index), _ptr(value), rows, cols)
        return index, value


class RefPaged:
    """The reference's own paged-append CUDA kernel (oracle/_ref/libhyle_ref_paged.so, built from the
    reference tree behind ref_paged_shim.cu).  Takes DEVICE pointers; only GPU parity tests use it."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_PAGED_LIB)

    def __init__(self):
        self.lib = ctypes.CDLL(REF_PAGED_LIB)
        _u32 = ctypes.c_uint32
        self.lib.hyle_ref_paged_append.argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u64]
        self.lib.hyle_ref_paged_append.restype = _i
        self.lib.hyle_ref_paged_append_device_lengths.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u64,
                                                                  _u32, _vp]
        self.lib.hyle_ref_paged_append_device_lengths.restype = _i

    def paged_append(self, stream, arena_ptr, rows_ptr, metadata_ptr, page_rows, physical_pages, input_rows, capacity,
                     row_bytes) -> int:
        return self.lib.hyle_ref_paged_append(stream, arena_ptr, rows_ptr, metadata_ptr, page_rows, physical_pages,
                                              input_rows, capacity, row_bytes)

    def paged_append_device_lengths(self, stream, arena_ptr, rows_ptr, metadata_ptr, query_ptr, kv_ptr, page_rows,
                                    physical_pages, input_rows, capacity, row_bytes, requests, status_ptr) -> int:
        return self.lib.hyle_ref_paged_append_device_lengths(stream, arena_ptr, rows_ptr, metadata_ptr, query_ptr, kv_ptr,
                                                             page_rows, physical_pages, input_rows, capacity, row_bytes,
                                                             requests, status_ptr)

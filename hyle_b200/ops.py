"""Operators of the B200 provider on torch CUDA tensors.

torch is used here for device memory and the current stream only; every operator is one call
through the C ABI (``include/hyle_b200.h``) into hand-written sm_100a kernels.  Names follow the
reference's operator schema (include/hyle/compute/operation.h): Binary, Reduce, RmsNorm,
GatedActivation, Softmax, TopK, Cast, CacheEncode.  There is no fallback: a missing library or a
CPU tensor raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import numpy as np
import torch

from . import abi

_DTYPE = {torch.float32: abi.F32, torch.bfloat16: abi.BF16, torch.float16: abi.F16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _device_tensor(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this provider has no CPU route)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be dense row-major")
    return t


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _torch_empty(shape, dtype, device) -> torch.Tensor:
    return torch.empty(shape, dtype=dtype, device=device)


_allocate_output = _torch_empty


def set_output_allocator(allocate=None):
    """Route every output tensor the operators create through ``allocate(shape, dtype, device)``.

    For callers that own the device pool (and for tests that place each output between guard bytes).
    ``None`` restores ``torch.empty``.  Returns the previous allocator."""
    global _allocate_output
    previous = _allocate_output
    _allocate_output = _torch_empty if allocate is None else allocate
    return previous


def _new(shape, dtype, device) -> torch.Tensor:
    if isinstance(shape, int):
        shape = (shape,)
    return _allocate_output(tuple(shape), dtype, device)


def new_output(shape, dtype, device="cuda") -> torch.Tensor:
    """An uninitialised tensor from the output allocator (see :func:`set_output_allocator`), for entry
    points called with explicit outputs."""
    return _new(shape, dtype, device)


def _new_like(t: torch.Tensor) -> torch.Tensor:
    return _allocate_output(tuple(t.shape), t.dtype, t.device)


def binary(kind: int, lhs: torch.Tensor, rhs: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Binary{kind}; ``rhs`` has lhs's shape or lhs's trailing axes (NumPy broadcast)."""
    _device_tensor(lhs, "lhs"), _device_tensor(rhs, "rhs")
    if lhs.dtype != rhs.dtype or lhs.dtype not in _DTYPE:
        raise ValueError("lhs and rhs must share one of f32 / bf16 / f16")
    if tuple(lhs.shape[lhs.dim() - rhs.dim():]) != tuple(rhs.shape):
        raise ValueError("rhs must equal lhs's shape or its trailing axes")
    if out is None:
        out = _new_like(lhs)
    abi.check("hyle_b200_binary", abi.load().hyle_b200_binary(
        _stream(), kind, _DTYPE[lhs.dtype], lhs.data_ptr(), rhs.data_ptr(), out.data_ptr(),
        lhs.numel(), max(rhs.numel(), 1) if lhs.numel() else 1))
    return out


def add(lhs, rhs, out=None):
    return binary(abi.BINARY_ADD, lhs, rhs, out)


def multiply(lhs, rhs, out=None):
    return binary(abi.BINARY_MULTIPLY, lhs, rhs, out)


def subtract(lhs, rhs, out=None):
    return binary(abi.BINARY_SUBTRACT, lhs, rhs, out)


def divide(lhs, rhs, out=None):
    return binary(abi.BINARY_DIVIDE, lhs, rhs, out)


def minimum(lhs, rhs, out=None):
    """Number minimum: a NaN operand yields the other one; min(+0, -0) = -0 in either order."""
    return binary(abi.BINARY_MINIMUM, lhs, rhs, out)


def maximum(lhs, rhs, out=None):
    """Number maximum: a NaN operand yields the other one; max(+0, -0) = +0 in either order."""
    return binary(abi.BINARY_MAXIMUM, lhs, rhs, out)


def unary(kind: int, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Unary{kind} (``abi.UNARY_*``) on a dense f32 / bf16 / f16 tensor."""
    _device_tensor(x, "x")
    if x.dtype not in _DTYPE:
        raise ValueError("x must be f32 / bf16 / f16")
    if out is None:
        out = _new_like(x)
    abi.check("hyle_b200_unary", abi.load().hyle_b200_unary(
        _stream(), kind, _DTYPE[x.dtype], x.data_ptr(), out.data_ptr(), x.numel()))
    return out


def reduce_rows(kind: int, x: torch.Tensor) -> torch.Tensor:
    """Reduce{kind, axes={-1}} of an f32 tensor, or its Minimum / Maximum for a bf16 or f16 tensor (result in
    the tensor's type); output drops the last axis."""
    _device_tensor(x, "x")
    narrow = x.dtype in (torch.bfloat16, torch.float16) and kind in (abi.REDUCE_MINIMUM, abi.REDUCE_MAXIMUM)
    if not (x.dtype == torch.float32 or narrow) or x.dim() < 1 or not x.is_contiguous():
        raise ValueError("reduce_rows takes a dense f32 tensor of rank >= 1 (bf16 / f16 for Minimum and Maximum)")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else int(torch.Size(x.shape[:-1]).numel())
    out = _new(x.shape[:-1], x.dtype, x.device)
    if narrow:
        abi.check("hyle_b200_reduce_rows_extremum", abi.load().hyle_b200_reduce_rows_extremum(
            _stream(), kind, _DTYPE[x.dtype], x.data_ptr(), out.data_ptr(), rows, cols))
        return out
    abi.check("hyle_b200_reduce_rows_f32", abi.load().hyle_b200_reduce_rows_f32(
        _stream(), kind, x.data_ptr(), out.data_ptr(), rows, cols))
    return out


def add_bias_row_sum_max(a: torch.Tensor, bias: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """C = A + bias (broadcast over rows), per-row sum and per-row max of C, fused."""
    _device_tensor(a, "a"), _device_tensor(bias, "bias")
    if a.dtype != torch.float32 or bias.dtype != torch.float32 or a.dim() != 2 or bias.shape != a.shape[1:]:
        raise ValueError("a must be f32 [rows, cols] and bias f32 [cols]")
    rows, cols = a.shape
    c = _new_like(a)
    row_sum = _new(rows, torch.float32, a.device)
    row_max = _new(rows, torch.float32, a.device)
    abi.check("hyle_b200_add_bias_row_sum_max_f32", abi.load().hyle_b200_add_bias_row_sum_max_f32(
        _stream(), a.data_ptr(), bias.data_ptr(), c.data_ptr(), row_sum.data_ptr(), row_max.data_ptr(),
        rows, cols))
    return c, row_sum, row_max


def _weight_args(weight: Optional[torch.Tensor], hidden: int):
    if weight is None:
        return None, abi.BF16
    _device_tensor(weight, "weight")
    if weight.numel() != hidden or weight.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("weight must be bf16 or f32 with `hidden` elements")
    return weight.data_ptr(), _DTYPE[weight.dtype]


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], epsilon: float,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RmsNorm{epsilon, accumulation=f32} over the last axis of a bf16, f16 or f32 tensor; the weight has x's
    type or is f32."""
    _device_tensor(x, "x")
    if x.dtype not in _DTYPE or not x.is_contiguous():
        raise ValueError("rms_norm takes a dense bf16, f16 or f32 tensor")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    if x.dtype == torch.bfloat16:
        w_ptr, w_dtype = _weight_args(weight, hidden)
    elif weight is None:
        w_ptr, w_dtype = None, _DTYPE[x.dtype]
    else:
        _device_tensor(weight, "weight")
        if weight.numel() != hidden or weight.dtype not in (x.dtype, torch.float32) or not weight.is_contiguous():
            raise ValueError("weight must have x's type or be f32, with `hidden` elements")
        w_ptr, w_dtype = weight.data_ptr(), _DTYPE[weight.dtype]
    if out is None:
        out = _new_like(x)
    abi.check("hyle_b200_rms_norm", abi.load().hyle_b200_rms_norm(
        _stream(), _DTYPE[x.dtype], x.data_ptr(), w_ptr, w_dtype, out.data_ptr(), rows, hidden, epsilon))
    return out


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: Optional[torch.Tensor],
                 epsilon: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """h = x + residual (bf16, one rounding); y = RmsNorm(h).  Returns (y, h)."""
    _device_tensor(x, "x"), _device_tensor(residual, "residual")
    if x.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16 or x.shape != residual.shape:
        raise ValueError("x and residual must be bf16 tensors of one shape")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    w_ptr, w_dtype = _weight_args(weight, hidden)
    y, h = _new_like(x), _new_like(x)
    abi.check("hyle_b200_add_rms_norm_bf16", abi.load().hyle_b200_add_rms_norm_bf16(
        _stream(), x.data_ptr(), residual.data_ptr(), w_ptr, w_dtype, y.data_ptr(), h.data_ptr(),
        rows, hidden, epsilon))
    return y, h


def layer_norm(x: torch.Tensor, scale: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float = 1e-5,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm over the last axis of a bf16 tensor; bf16 ``scale`` and ``bias`` of [hidden], both or neither."""
    _device_tensor(x, "x")
    if x.dtype != torch.bfloat16 or (scale is None) != (bias is None):
        raise ValueError("layer_norm takes bf16 x and bf16 scale and bias (both or neither)")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    if out is None:
        out = _new_like(x)
    abi.check("hyle_b200_layer_norm_bf16", abi.load().hyle_b200_layer_norm_bf16(
        _stream(), x.data_ptr(), _ptr(scale), _ptr(bias), out.data_ptr(), rows, hidden, eps))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """GatedActivation{kSilu, kSeparate}: silu(gate) * up on bf16 tensors of one shape."""
    _device_tensor(gate, "gate"), _device_tensor(up, "up")
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or gate.shape != up.shape:
        raise ValueError("gate and up must be bf16 tensors of one shape")
    cols = gate.shape[-1]
    rows = gate.numel() // cols if cols else 0
    out = _new_like(gate)
    abi.check("hyle_b200_swiglu_bf16", abi.load().hyle_b200_swiglu_bf16(
        _stream(), gate.data_ptr(), up.data_ptr(), out.data_ptr(), rows, cols, cols, cols))
    return out


def gated_activation(gate: torch.Tensor, up: torch.Tensor, activation: int = abi.GATE_SILU,
                     round_gate: bool = False) -> torch.Tensor:
    """GatedActivation{activation, kSeparate} on bf16 / f16 tensors of one shape; with ``round_gate`` the
    result of Unary{activation} followed by Binary{kMultiply} (the activated gate rounded to storage first)."""
    _device_tensor(gate, "gate"), _device_tensor(up, "up")
    if gate.dtype not in (torch.bfloat16, torch.float16) or up.dtype != gate.dtype or gate.shape != up.shape:
        raise ValueError("gate and up must be bf16 or f16 tensors of one shape")
    cols = gate.shape[-1]
    rows = gate.numel() // cols if cols else 0
    out = _new_like(gate)
    abi.check("hyle_b200_gated_activation", abi.load().hyle_b200_gated_activation(
        _stream(), activation, _DTYPE[gate.dtype], int(round_gate), gate.data_ptr(), up.data_ptr(), out.data_ptr(),
        rows, cols, cols, cols))
    return out


def swiglu_packed(packed: torch.Tensor) -> torch.Tensor:
    """GatedActivation{kSilu, kPackedHalves}: the last axis holds [gate | up]."""
    _device_tensor(packed, "packed")
    if packed.dtype != torch.bfloat16 or packed.shape[-1] % 2:
        raise ValueError("packed must be bf16 with an even last axis")
    cols = packed.shape[-1] // 2
    rows = packed.numel() // (2 * cols) if cols else 0
    out = _new(packed.shape[:-1] + (cols,), torch.bfloat16, packed.device)
    abi.check("hyle_b200_swiglu_bf16", abi.load().hyle_b200_swiglu_bf16(
        _stream(), packed.data_ptr(), packed.data_ptr() + 2 * cols, out.data_ptr(), rows, cols,
        2 * cols, 2 * cols))
    return out


def make_logits_workspace(device, rows: int, cols: int) -> torch.Tensor:
    """Zero-filled scratch for `logits_reduce` / `softmax` on batches of 64 rows or more (the
    streaming kernel); reusable by any number of stream-ordered calls of at most this shape."""
    return torch.zeros(abi.load().hyle_b200_logits_workspace_bytes(rows, cols), dtype=torch.uint8, device=device)


def logits_reduce(logits: torch.Tensor, want_probs: bool = True, want_lse: bool = True,
                  want_argmax: bool = True, workspace: Optional[torch.Tensor] = None,
                  status: Optional[torch.Tensor] = None, tuning: Optional[abi.StreamTuning] = None):
    """Fused log-sum-exp, softmax->bf16 and argmax of f32 [rows, cols] logits.

    Returns (lse f32[rows], probs bf16[rows, cols], index i32[rows], value f32[rows]); entries not
    asked for are None.  With a `workspace` (`make_logits_workspace`) large batches take the
    streaming kernel; without one every batch takes the cluster kernel.  ``status`` (one int32 word)
    receives abi.STATUS_STREAM_WAIT_TIMEOUT if the streaming kernel could not complete a row;
    ``tuning`` overrides its schedule (sweeps, tests of the rare paths).
    """
    _device_tensor(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("logits must be f32 [rows, cols]")
    rows, cols = logits.shape
    dev = logits.device
    lse = _new(rows, torch.float32, dev) if want_lse else None
    probs = _new((rows, cols), torch.bfloat16, dev) if want_probs else None
    index = _new(rows, torch.int32, dev) if want_argmax else None
    value = _new(rows, torch.float32, dev) if want_argmax else None
    arguments = (_stream(), logits.data_ptr(), rows, cols, _ptr(lse), _ptr(probs), _ptr(index), _ptr(value),
                 _ptr(workspace), 0 if workspace is None else workspace.numel(), _ptr(status))
    if tuning is None:
        abi.check("hyle_b200_logits_reduce_f32", abi.load().hyle_b200_logits_reduce_f32(*arguments))
    else:
        abi.check("hyle_b200_logits_reduce_f32_tuned",
                  abi.load().hyle_b200_logits_reduce_f32_tuned(*arguments, ctypes.addressof(tuning)))
    return lse, probs, index, value


def logits_stream_plan(rows: int, cols: int, tuning: Optional[abi.StreamTuning] = None) -> Optional[abi.StreamPlan]:
    """The streaming kernel's schedule for a shape (host arithmetic), or None when the shape takes the cluster kernel."""
    plan = abi.StreamPlan()
    code = abi.load().hyle_b200_logits_stream_plan(rows, cols, None if tuning is None else ctypes.addressof(tuning),
                                                   ctypes.addressof(plan))
    if code == abi.NOT_SUPPORTED:
        return None
    abi.check("hyle_b200_logits_stream_plan", code)
    return plan


def argmax(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """TopK{count=1}: (index i32[rows], value f32[rows]); lowest index on ties, NaN last."""
    _, _, index, value = logits_reduce(logits, want_probs=False, want_lse=False)
    return index, value


def softmax(x: torch.Tensor, log: bool = False, out: Optional[torch.Tensor] = None,
            workspace: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax{axis=-1, kSoftmax|kLogSoftmax} on f32 rows, f32 output."""
    _device_tensor(x, "x")
    if x.dtype != torch.float32:
        raise ValueError("softmax takes f32 input")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if out is None:
        out = _new_like(x)
    abi.check("hyle_b200_softmax_f32", abi.load().hyle_b200_softmax_f32(
        _stream(), abi.LOG_SOFTMAX if log else abi.SOFTMAX, x.data_ptr(), out.data_ptr(), rows, cols,
        _ptr(workspace), 0 if workspace is None else workspace.numel(), _ptr(status)))
    return out


_CAST_TORCH = {abi.F32: torch.float32, abi.BF16: torch.bfloat16, abi.F16: torch.float16, abi.E4M3: torch.uint8,
               abi.E5M2: torch.uint8, abi.BOOL: torch.uint8, abi.I32: torch.int32}
_CAST_DTYPE = {torch.float32: abi.F32, torch.bfloat16: abi.BF16, torch.float16: abi.F16, torch.int32: abi.I32,
               torch.uint8: abi.BOOL, torch.bool: abi.BOOL}


def cast(x: torch.Tensor, source: int, destination: int) -> torch.Tensor:
    """Cast between storage types (``abi.F32`` ... ``abi.I32``).  The 8-bit floating formats and bool
    travel as uint8 tensors of their storage bytes."""
    _device_tensor(x, "x")
    if x.dtype != _CAST_TORCH[source]:
        raise ValueError(f"source type {source} is carried by {_CAST_TORCH[source]}, got {x.dtype}")
    out = _new(x.shape, _CAST_TORCH[destination], x.device)
    abi.check("hyle_b200_cast", abi.load().hyle_b200_cast(
        _stream(), source, destination, x.data_ptr(), out.data_ptr(), x.numel()))
    return out


def fp8_e4m3_encode(x: torch.Tensor, scale: float, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """CacheEncode{float8(scale)}: uint8 E4M3 codes of x / scale; a non-finite value gives 0 and a status bit."""
    _device_tensor(x, "x")
    if x.dtype not in _DTYPE:
        raise ValueError("x must be f32 / bf16 / f16")
    out = _new(x.shape, torch.uint8, x.device)
    abi.check("hyle_b200_fp8_e4m3_encode", abi.load().hyle_b200_fp8_e4m3_encode(
        _stream(), _DTYPE[x.dtype], x.data_ptr(), x.numel(), scale, out.data_ptr(), _ptr(status)))
    return out


def strided_cast(x: torch.Tensor, dtype: Optional[int] = None) -> torch.Tensor:
    """Dense copy of ANY view ``x`` (slices, permutations, broadcasts), cast to the library dtype ``dtype``
    (abi.F32 ...) or kept as it is.  8-bit float codes travel as uint8 with ``source`` / ``dtype`` given as
    library dtypes through :func:`strided_cast_raw`."""
    source = _CAST_DTYPE[x.dtype]
    return strided_cast_raw(x, source, source if dtype is None else dtype)


def strided_cast_raw(x: torch.Tensor, source: int, destination: int) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor (this provider has no CPU route)")
    if x.dim() > 8:
        raise ValueError("views of rank <= 8")
    if x.element_size() != torch.empty(0, dtype=_CAST_TORCH[source]).element_size():
        raise ValueError("the view's element size does not match the source type")
    out = _new(x.shape, _CAST_TORCH[destination], x.device)
    dims = (ctypes.c_int64 * max(1, x.dim()))(*x.shape)
    strides = (ctypes.c_int64 * max(1, x.dim()))(*[s * x.element_size() for s in x.stride()])
    abi.check("hyle_b200_strided_cast", abi.load().hyle_b200_strided_cast(
        _stream(), source, destination, x.data_ptr(), out.data_ptr(), x.dim(), dims, strides))
    return out


def strided_scatter(dense: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Place the dense tensor ``dense`` into ``out``, ANY view of the same shape and element size that does not
    overlap itself (a slice of a larger tensor, a permuted layout); bytes of ``out``'s storage outside the view
    are left alone.  Returns ``out``."""
    _device_tensor(dense, "dense")
    if not out.is_cuda or out.device != dense.device:
        raise ValueError("out must be a CUDA tensor on dense's device")
    if not dense.is_contiguous() or tuple(dense.shape) != tuple(out.shape) or dense.element_size() != out.element_size():
        raise ValueError("dense must be contiguous and have out's shape and element size")
    if out.dim() > 8:
        raise ValueError("views of rank <= 8")
    dtype = {4: abi.F32, 2: abi.BF16, 1: abi.BOOL}.get(out.element_size())
    if dtype is None:
        raise ValueError("elements of 1, 2 or 4 bytes")
    dims = (ctypes.c_int64 * max(1, out.dim()))(*out.shape)
    strides = (ctypes.c_int64 * max(1, out.dim()))(*[s * out.element_size() for s in out.stride()])
    abi.check("hyle_b200_strided_scatter", abi.load().hyle_b200_strided_scatter(
        _stream(), dtype, dense.data_ptr(), out.data_ptr(), out.dim(), dims, strides))
    return out


def scan(x: torch.Tensor, exclusive: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Scan{axis=-1, exclusive}: prefix sums along the last axis of a dense f32 / i32 tensor.  For i32 a
    ``status`` word is required: abi.STATUS_SCAN_OVERFLOW is set there, and the result left unwritten, when
    a prefix does not fit int32."""
    _device_tensor(x, "x")
    if x.dtype not in (torch.float32, torch.int32) or not x.is_contiguous() or x.dim() < 1:
        raise ValueError("scan takes a dense f32 / i32 tensor")
    if x.dtype == torch.int32 and status is None:
        raise ValueError("the i32 scan reports overflow through a status word")
    out = _new_like(x)
    cols = x.shape[-1]
    abi.check("hyle_b200_scan", abi.load().hyle_b200_scan(
        _stream(), abi.F32 if x.dtype == torch.float32 else abi.I32, x.data_ptr(), out.data_ptr(),
        x.numel() // cols if cols else 0, cols, int(exclusive), _ptr(status)))
    return out


def paged_append_metadata(instructions, capacity: int, device=None) -> torch.Tensor:
    """Pack an episode for :func:`paged_append`: int32 words {active_count, 0, 0, 0} followed by
    ``capacity`` instructions of {source_kind, source_page, source_row, destination_page,
    destination_row, rows, 0, 0} (include/hyle/compute/detail/paged_append_wire.h:11-25).
    ``instructions`` is a sequence of 6-tuples in that order; unused slots are zero."""
    if len(instructions) > capacity:
        raise ValueError("more instructions than the episode's capacity")
    words = np.zeros(4 + 8 * capacity, dtype=np.uint32)
    words[0] = len(instructions)
    for slot, fields in enumerate(instructions):
        if len(fields) != 6:
            raise ValueError("an instruction has six fields")
        words[4 + 8 * slot: 4 + 8 * slot + 6] = [int(f) & 0xFFFFFFFF for f in fields]
    packed = torch.from_numpy(words.view(np.int32))
    return packed.to(device) if device is not None else packed


def paged_append(arena: torch.Tensor, new_rows: Optional[torch.Tensor], metadata: torch.Tensor, page_rows: int,
                 capacity: Optional[int] = None) -> torch.Tensor:
    """Move rows into the pages of ``arena`` [physical_pages * page_rows, row...] in place, as the device
    resident episode ``metadata`` says (see :func:`paged_append_metadata`); ``new_rows`` [input_rows, row...]
    holds the packed rows of source kind 0 and may be None.  Malformed instructions are skipped, a
    malformed episode does nothing (src/compute_backend_cuda/cuda_paged_append.cu:16-45)."""
    _device_tensor(arena, "arena")
    _device_tensor(metadata, "metadata")
    if not arena.is_contiguous() or arena.dim() < 2 or arena.shape[0] % page_rows:
        raise ValueError("arena must be contiguous [physical_pages * page_rows, row...]")
    if metadata.dtype != torch.int32 or metadata.dim() != 1 or (metadata.numel() - 4) % 8 or metadata.numel() < 4:
        raise ValueError("metadata must be int32 words: 4 of header + 8 per instruction")
    row_bytes = arena[0].numel() * arena.element_size()
    input_rows = 0
    if new_rows is not None:
        _device_tensor(new_rows, "new_rows")
        if not new_rows.is_contiguous() or new_rows.numel() == 0 or new_rows[0].numel() * new_rows.element_size() != row_bytes:
            raise ValueError("new_rows must be contiguous rows of the arena's row size")
        input_rows = new_rows.shape[0]
    if capacity is None:
        capacity = (metadata.numel() - 4) // 8
    elif capacity > (metadata.numel() - 4) // 8:
        raise ValueError("capacity exceeds the metadata buffer")
    abi.check("hyle_b200_paged_append", abi.load().hyle_b200_paged_append(
        _stream(), arena.data_ptr(), _ptr(new_rows), metadata.data_ptr(), page_rows, arena.shape[0] // page_rows,
        input_rows, capacity, row_bytes))
    return arena


def paged_append_device_lengths(arena: torch.Tensor, new_rows: torch.Tensor, metadata: torch.Tensor,
                                query_lengths: torch.Tensor, kv_lengths: torch.Tensor, page_rows: int,
                                status: torch.Tensor) -> torch.Tensor:
    """Paged append whose row ranges are derived on the device from ``query_lengths`` / ``kv_lengths``
    (int32 [requests]); ``metadata`` is int32 words: 4 of header, then 8 per record (directory, request
    bounds, dirty pages: include/hyle/compute/detail/device_lengths_paged_append_wire.h:8-24).
    ``status`` (one int32 word) follows the reference's device status protocol: 0 = ok, 1 = a page
    record out of range, 4 = inconsistent episode or lengths; nothing is done when it is not 0 on entry."""
    for name, t in (("arena", arena), ("new_rows", new_rows), ("metadata", metadata), ("query_lengths", query_lengths),
                    ("kv_lengths", kv_lengths), ("status", status)):
        _device_tensor(t, name)
    if not arena.is_contiguous() or arena.dim() < 2 or arena.shape[0] % page_rows:
        raise ValueError("arena must be contiguous [physical_pages * page_rows, row...]")
    row_bytes = arena[0].numel() * arena.element_size()
    if not new_rows.is_contiguous() or new_rows.numel() == 0 or new_rows[0].numel() * new_rows.element_size() != row_bytes:
        raise ValueError("new_rows must be contiguous rows of the arena's row size")
    if metadata.dtype != torch.int32 or metadata.dim() != 1 or (metadata.numel() - 4) % 8 or metadata.numel() < 4:
        raise ValueError("metadata must be int32 words: 4 of header + 8 per record")
    if query_lengths.dtype != torch.int32 or kv_lengths.dtype != torch.int32 or query_lengths.shape != kv_lengths.shape:
        raise ValueError("lengths must be int32 tensors of one shape")
    if status.dtype != torch.int32 or status.numel() != 1:
        raise ValueError("status is one int32 word")
    abi.check("hyle_b200_paged_append_device_lengths", abi.load().hyle_b200_paged_append_device_lengths(
        _stream(), arena.data_ptr(), new_rows.data_ptr(), metadata.data_ptr(), query_lengths.data_ptr(),
        kv_lengths.data_ptr(), page_rows, arena.shape[0] // page_rows, new_rows.shape[0], (metadata.numel() - 4) // 8,
        row_bytes, query_lengths.numel(), status.data_ptr()))
    return arena


def cast_f32_to_bf16(x: torch.Tensor) -> torch.Tensor:
    _device_tensor(x, "x")
    if x.dtype != torch.float32:
        raise ValueError("cast_f32_to_bf16 takes f32 input")
    out = _new(x.shape, torch.bfloat16, x.device)
    abi.check("hyle_b200_cast_f32_to_bf16", abi.load().hyle_b200_cast_f32_to_bf16(
        _stream(), x.data_ptr(), out.data_ptr(), x.numel()))
    return out


def q8_0_bytes(count: int) -> int:
    """Size of the Q8_0 carrier for ``count`` values: 34 bytes per block of 32."""
    if count % 32:
        raise ValueError("Q8_0 needs a multiple of 32 values")
    return count // 32 * 34


def q8_0_encode(x: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """CacheEncode{q8_0}: returns the U8 carrier [..., cols/32*34]."""
    _device_tensor(x, "x")
    if x.dtype not in _DTYPE or x.shape[-1] % 32:
        raise ValueError("q8_0_encode takes f32/bf16/f16 with a last axis that is a multiple of 32")
    out = _new(x.shape[:-1] + (x.shape[-1] // 32 * 34,), torch.uint8, x.device)
    abi.check("hyle_b200_q8_0_encode", abi.load().hyle_b200_q8_0_encode(
        _stream(), _DTYPE[x.dtype], x.data_ptr(), x.numel(), out.data_ptr(), _ptr(status)))
    return out


def q8_0_decode(blocks: torch.Tensor, count: int) -> torch.Tensor:
    _device_tensor(blocks, "blocks")
    if blocks.dtype != torch.uint8 or blocks.numel() != q8_0_bytes(count):
        raise ValueError("blocks must be the U8 carrier of `count` values")
    out = _new(count, torch.bfloat16, blocks.device)
    abi.check("hyle_b200_q8_0_decode_bf16", abi.load().hyle_b200_q8_0_decode_bf16(
        _stream(), blocks.data_ptr(), count, out.data_ptr()))
    return out


def q8_0_decode_file(path: str, count: int, file_offset: int = 0, out: Optional[torch.Tensor] = None,
                     chunk_bytes: int = 0, slots: int = 0, device="cuda"):
    """Decode the Q8_0 bank of ``count`` values stored at ``file_offset`` of ``path`` into a bf16 device tensor,
    streaming the file through pinned staging chunks while the decode kernel runs.  Returns (tensor, report)."""
    if count % 32:
        raise ValueError("Q8_0 needs a multiple of 32 values")
    if out is None:
        out = _new(count, torch.bfloat16, device)
    options = abi.FileStreamOptions(chunk_bytes, slots, 0, 0)
    report = abi.FileStreamReport()
    abi.check("hyle_b200_q8_0_decode_file_bf16", abi.load().hyle_b200_q8_0_decode_file_bf16(
        _stream(), os.fsencode(path), file_offset, count, out.data_ptr(), ctypes.addressof(options), ctypes.addressof(report)))
    return out, report


class FileStream:
    """Chunks of a file range, resident on the device in file order (`hyle_b200_file_stream_*`).

    Iterating yields (device pointer, bytes, offset in the range); a chunk is valid until the next one is asked for."""

    def __init__(self, path: str, nbytes: int, file_offset: int = 0, chunk_bytes: int = 0, slots: int = 0, granule: int = 0):
        self._handle = ctypes.c_void_p()
        options = abi.FileStreamOptions(chunk_bytes, slots, 0, granule)
        abi.check("hyle_b200_file_stream_open", abi.load().hyle_b200_file_stream_open(
            os.fsencode(path), file_offset, nbytes, ctypes.addressof(options), ctypes.byref(self._handle)))

    def __iter__(self):
        lib = abi.load()
        while True:
            pointer, size, offset = ctypes.c_void_p(), ctypes.c_uint64(), ctypes.c_uint64()
            abi.check("hyle_b200_file_stream_next", lib.hyle_b200_file_stream_next(
                self._handle, _stream(), ctypes.byref(pointer), ctypes.byref(size), ctypes.byref(offset)))
            if size.value == 0:
                return
            yield pointer.value, size.value, offset.value

    def read_group(self, ranges) -> None:
        """Copy byte ranges of the file into device tensors: ``ranges`` = [(file offset, tensor or (pointer, bytes))].
        Only for a stream opened with ``nbytes == 0``.  The current stream waits for the group's last copy."""
        table = (abi.FileRange * len(ranges))()
        for entry, (offset, target) in zip(table, ranges):
            if isinstance(target, torch.Tensor):
                _device_tensor(target, "destination")
                if not target.is_contiguous():
                    raise ValueError("destinations must be dense")
                pointer, size = target.data_ptr(), target.numel() * target.element_size()
            else:
                pointer, size = target
            entry.file_offset, entry.bytes, entry.destination = offset, size, pointer
        abi.check("hyle_b200_file_stream_read_group", abi.load().hyle_b200_file_stream_read_group(
            self._handle, _stream(), ctypes.addressof(table) if len(ranges) else None, len(ranges)))

    def report(self) -> abi.FileStreamReport:
        report = abi.FileStreamReport()
        abi.check("hyle_b200_file_stream_get_report", abi.load().hyle_b200_file_stream_get_report(self._handle, ctypes.addressof(report)))
        return report

    def close(self) -> None:
        if self._handle:
            abi.load().hyle_b200_file_stream_close(self._handle)
            self._handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def make_workspace(device, count: int = 0) -> torch.Tensor:
    """Zero-filled scratch for sum_squares / q8_0_roundtrip of up to ``count`` values; reusable
    across stream-ordered calls."""
    return torch.zeros(abi.load().hyle_b200_sum_squares_workspace_bytes(count), dtype=torch.uint8, device=device)


def sum_squares(x: torch.Tensor, workspace: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sum of squares of a bf16 tensor as a device f64 scalar."""
    _device_tensor(x, "x")
    if x.dtype != torch.bfloat16:
        raise ValueError("sum_squares takes bf16 input")
    if out is None:
        out = _new(1, torch.float64, x.device)
    abi.check("hyle_b200_sum_squares_bf16", abi.load().hyle_b200_sum_squares_bf16(
        _stream(), x.data_ptr(), x.numel(), out.data_ptr(), workspace.data_ptr(), workspace.numel()))
    return out


def q8_0_roundtrip(x: torch.Tensor, workspace: torch.Tensor, blocks: Optional[torch.Tensor] = None,
                   decoded: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None,
                   status: Optional[torch.Tensor] = None):
    """One pass: Q8_0 blocks, decoded bf16 and sum of squares of a bf16 tensor."""
    _device_tensor(x, "x")
    if x.dtype != torch.bfloat16 or x.numel() % 32:
        raise ValueError("q8_0_roundtrip takes bf16 input with a multiple of 32 values")
    if blocks is None:
        blocks = _new(q8_0_bytes(x.numel()), torch.uint8, x.device)
    if decoded is None:
        decoded = _new_like(x)
    if sum_out is None:
        sum_out = _new(1, torch.float64, x.device)
    abi.check("hyle_b200_q8_0_roundtrip_bf16", abi.load().hyle_b200_q8_0_roundtrip_bf16(
        _stream(), x.data_ptr(), x.numel(), blocks.data_ptr(), decoded.data_ptr(), sum_out.data_ptr(),
        _ptr(status), workspace.data_ptr(), workspace.numel()))
    return blocks, decoded, sum_out


def q8_0_roundtrip_static(x: torch.Tensor, blocks: Optional[torch.Tensor] = None,
                          decoded: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None,
                          status: Optional[torch.Tensor] = None):
    """`q8_0_roundtrip` without a workspace: the kernel's scratch is a fixed array inside the library.

    For callers that must not allocate device memory.  At most ``abi.STATIC_MAX_VALUES`` values per
    call; calls on one device share the scratch, so only stream-ordered calls are safe.  (The
    outputs are still the caller's; pass them in to avoid torch allocating them here.)
    """
    _device_tensor(x, "x")
    if x.dtype != torch.bfloat16 or x.numel() % 32:
        raise ValueError("q8_0_roundtrip_static takes bf16 input with a multiple of 32 values")
    if blocks is None:
        blocks = _new(q8_0_bytes(x.numel()), torch.uint8, x.device)
    if decoded is None:
        decoded = _new_like(x)
    if sum_out is None:
        sum_out = _new(1, torch.float64, x.device)
    abi.check("hyle_b200_q8_0_roundtrip_bf16_static", abi.load().hyle_b200_q8_0_roundtrip_bf16_static(
        _stream(), x.data_ptr(), x.numel(), blocks.data_ptr(), decoded.data_ptr(), sum_out.data_ptr(),
        _ptr(status)))
    return blocks, decoded, sum_out


def random_bits(identities: torch.Tensor, word_count: int) -> torch.Tensor:
    """sampling_ops::RandomBits: u32 identities [rows, 4] (carried as int32) -> counter-generator words [rows, word_count]."""
    _device_tensor(identities, "identities")
    if identities.dtype != torch.int32 or identities.dim() != 2 or identities.shape[1] != 4:
        raise ValueError("identities must be int32 [rows, 4] holding the u32 words")
    out = _new((identities.shape[0], word_count), torch.int32, identities.device)
    abi.check("hyle_b200_random_bits", abi.load().hyle_b200_random_bits(
        _stream(), identities.data_ptr(), identities.shape[0], word_count, out.data_ptr()))
    return out


def categorical(log_weights: torch.Tensor, identities: torch.Tensor, want_log_probability: bool = True,
                status: Optional[torch.Tensor] = None):
    """sampling_ops::Categorical: one index per row (i32; -1 for a rejected row) and optionally its log-probability."""
    _device_tensor(log_weights, "log_weights"), _device_tensor(identities, "identities")
    if log_weights.dtype not in _DTYPE or log_weights.dim() != 2:
        raise ValueError("log_weights must be f32 / bf16 / f16 [rows, cols]")
    rows, cols = log_weights.shape
    if identities.dtype != torch.int32 or tuple(identities.shape) != (rows, 4):
        raise ValueError("identities must be int32 [rows, 4] holding the u32 words")
    index = _new(rows, torch.int32, log_weights.device)
    logp = _new(rows, torch.float32, log_weights.device) if want_log_probability else None
    abi.check("hyle_b200_categorical", abi.load().hyle_b200_categorical(
        _stream(), _DTYPE[log_weights.dtype], log_weights.data_ptr(), identities.data_ptr(), rows, cols,
        index.data_ptr(), _ptr(logp), _ptr(status)))
    return index, logp


def select(condition: torch.Tensor, when_true: torch.Tensor, when_false: torch.Tensor) -> torch.Tensor:
    """Select: condition (uint8 / bool bytes, shape of the result) picks when_true or when_false; each branch has
    the result's shape or its trailing axes (a one-element tensor is a scalar)."""
    _device_tensor(condition, "condition"), _device_tensor(when_true, "when_true"), _device_tensor(when_false, "when_false")
    if when_true.dtype != when_false.dtype or condition.element_size() != 1:
        raise ValueError("branches must share a type and the condition must be one byte per element")
    code = {torch.float32: abi.F32, torch.int32: abi.I32, torch.bfloat16: abi.BF16, torch.float16: abi.F16}[when_true.dtype]
    out = _new(condition.shape, when_true.dtype, condition.device)
    abi.check("hyle_b200_select", abi.load().hyle_b200_select(
        _stream(), code, condition.data_ptr(), when_true.data_ptr(), when_false.data_ptr(), out.data_ptr(),
        condition.numel(), max(when_true.numel(), 1), max(when_false.numel(), 1)))
    return out


def masked_softmax_f16(x: torch.Tensor, mask: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Softmax{scale, mask} over the last axis of an f16 tensor; the mask has x's shape or its trailing axes
    including the last one.  A one-byte mask is Boolean (0 masks); an f16 mask is additive (added after the
    scaling, -inf masks)."""
    _device_tensor(x, "x"), _device_tensor(mask, "mask")
    additive = mask.dtype == torch.float16
    if x.dtype != torch.float16 or not (additive or mask.element_size() == 1):
        raise ValueError("masked_softmax_f16 takes f16 values and a one-byte (Boolean) or f16 (additive) mask")
    if not x.is_contiguous() or not mask.is_contiguous():
        raise ValueError("masked_softmax_f16 takes dense tensors")
    cols = x.shape[-1]
    out = _new_like(x)
    name = "hyle_b200_additive_masked_softmax_f16" if additive else "hyle_b200_masked_softmax_f16"
    abi.check(name, getattr(abi.load(), name)(
        _stream(), x.data_ptr(), mask.data_ptr(), mask.numel(), scale, out.data_ptr(), x.numel() // cols if cols else 0, cols))
    return out

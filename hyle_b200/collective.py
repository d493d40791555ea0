"""The one exchange of the sharded sweep: an NCCL all-reduce of the per-GPU sums of squares.

`torch.distributed` provides rendezvous; the all-reduce itself is issued straight on the stream the
kernels run on (ncclAllReduce through ctypes on the NCCL library torch ships), so a step is
kernel -> all-reduce -> next kernel on ONE stream.  torch's own `dist.all_reduce` runs on an
internal stream fenced by two cross-stream events, which costs several microseconds per step --
visible when a step is 230 us.
"""
from __future__ import annotations

import ctypes
import glob
import os

NCCL_FLOAT64 = 8
NCCL_SUM = 0


class _UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def _library() -> ctypes.CDLL:
    import torch

    candidates = glob.glob(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "nccl", "lib", "libnccl.so*"))
    return ctypes.CDLL(candidates[0] if candidates else "libnccl.so.2")


class StreamAllReduce:
    """Sum-all-reduce of f64 device buffers on a caller-chosen CUDA stream, one communicator per process."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.lib = _library()
        self.lib.ncclGetErrorString.restype = ctypes.c_char_p
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        unique = _UniqueId()
        if self.rank == 0:
            self._check(self.lib.ncclGetUniqueId(ctypes.byref(unique)), "ncclGetUniqueId")
        payload = torch.frombuffer(bytearray(bytes(unique)), dtype=torch.uint8).cuda()
        dist.broadcast(payload, src=0)
        ctypes.memmove(ctypes.byref(unique), bytes(payload.cpu().numpy().tobytes()), 128)
        self.comm = ctypes.c_void_p()
        self.lib.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _UniqueId, ctypes.c_int]
        self._check(self.lib.ncclCommInitRank(ctypes.byref(self.comm), self.world, unique, self.rank), "ncclCommInitRank")
        self.lib.ncclAllReduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_void_p, ctypes.c_void_p]

    def _check(self, code: int, what: str) -> None:
        if code != 0:
            raise RuntimeError(f"{what} failed: {self.lib.ncclGetErrorString(code).decode()}")

    def sum_f64(self, tensor, stream: int) -> None:
        """In-place sum over all ranks of an f64 CUDA tensor, recorded on `stream` (a cudaStream_t value)."""
        self._check(self.lib.ncclAllReduce(tensor.data_ptr(), tensor.data_ptr(), tensor.numel(), NCCL_FLOAT64, NCCL_SUM,
                                           self.comm, stream), "ncclAllReduce")

    def close(self) -> None:
        if self.comm:
            self.lib.ncclCommDestroy.argtypes = [ctypes.c_void_p]
            self.lib.ncclCommDestroy(self.comm)
            self.comm = ctypes.c_void_p()

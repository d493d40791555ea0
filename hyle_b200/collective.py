"""The one exchange of the sharded sweep: the sum over GPUs of the per-GPU sums of squares.

Two forms.  `PeerExchange` sets up what `hyle_b200_q8_0_roundtrip_bf16_exchange` needs: the kernel's
finishing CTA itself writes the 8 bytes into every peer's mailbox over NVLink and adds what it
receives, so a step is ONE kernel.  `StreamAllReduce` is the library form, kernel + ncclAllReduce:

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


class PeerMappingUnavailable(RuntimeError):
    """The GPUs' memory could not be mapped between the processes (CUDA IPC refused on this machine)."""


class PeerExchange:
    """Mailboxes for `hyle_b200_q8_0_roundtrip_bf16_exchange`, one process per GPU.

    Every rank creates a mailbox on its own GPU, the CUDA IPC handles travel through
    `torch.distributed` (any backend), and every rank maps the others' mailboxes.  `pointers` is the
    array the entry point takes; `next_epoch()` numbers the collective calls 1, 2, 3, ...
    """

    def __init__(self, library=None):
        """`library`: an object with the four hyle_b200_exchange_* functions (tests pass a stand-in
        to exercise the set-up protocol without GPUs); by default the kernel library."""
        import torch.distributed as dist

        from . import abi

        self.abi = abi
        self.lib = abi.load() if library is None else library
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        if self.world > abi.EXCHANGE_MAX_RANKS:
            raise ValueError(f"at most {abi.EXCHANGE_MAX_RANKS} ranks")
        self.mailbox = ctypes.c_void_p()
        self.pointers = (ctypes.c_void_p * self.world)()
        self.opened = []
        self.epoch = 0
        # Set-up is collective: every step (create, exchange handles, map) is attempted by every rank
        # and the outcome agreed on, so that either all ranks hold a complete table or all raise
        # PeerMappingUnavailable -- never a mixture that would leave some ranks waiting in a kernel.
        handle = ctypes.create_string_buffer(abi.EXCHANGE_HANDLE_BYTES)
        failure = None
        code = self.lib.hyle_b200_exchange_create(ctypes.byref(self.mailbox), handle)
        if code != abi.OK:
            failure = f"hyle_b200_exchange_create returned {code}"
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw if failure is None else None)
        if failure is None and any(raw is None for raw in handles):
            failure = "a peer could not create its mailbox"
        if failure is None:
            for peer, raw in enumerate(handles):
                if peer == self.rank:
                    self.pointers[peer] = self.mailbox.value
                    continue
                mapped = ctypes.c_void_p()
                code = self.lib.hyle_b200_exchange_open(raw, ctypes.byref(mapped))
                if code != abi.OK:
                    failure = f"hyle_b200_exchange_open returned {code} for rank {peer}"
                    break
                self.pointers[peer] = mapped.value
                self.opened.append(mapped)
        outcomes = [None] * self.world
        dist.all_gather_object(outcomes, failure)  # also the barrier: every mailbox is mapped everywhere
        problems = [f"rank {r}: {text}" for r, text in enumerate(outcomes) if text is not None]
        if problems:
            self._release()
            raise PeerMappingUnavailable("; ".join(problems))

    def next_epoch(self) -> int:
        self.epoch = self.epoch % 0xFFFFFFFE + 1  # 1 ... 2^32-2, so consecutive values always differ in parity
        return self.epoch

    def _release(self) -> None:
        for mapped in self.opened:
            self.lib.hyle_b200_exchange_close(mapped)
        self.opened = []
        if self.mailbox:
            self.lib.hyle_b200_exchange_destroy(self.mailbox)
            self.mailbox = ctypes.c_void_p()

    def close(self) -> None:
        import torch
        import torch.distributed as dist

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier()  # no peer is still writing into a mailbox that is about to go
        self._release()

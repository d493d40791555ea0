"""File -> pinned -> device streaming of on-disk Q8_0 banks (`hyle_b200_file_stream_*`).

A seeded weight tensor is encoded by the CPU checker into the GGUF Q8_0 layout (rows of k/32 blocks of
34 bytes, src/compute_ops/low_precision.cc:269-297), written to a file behind a header, streamed through
the pipeline and decoded on the GPU; the decoded bf16 must equal the checker's decode bit for bit, for
chunk sizes that do and do not divide the bank and for the smallest ring.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from hyle_b200 import abi, ops
from hyle_b200 import workloads as wl
from oracle import binding as ob


def _bank(tmp_path, rows, header=4096):
    oracle = ob.Oracle()
    weights = wl.q8_sweep_inputs(rows)
    blocks, invalid = oracle.q8_0_encode(ob.BF16, weights)
    assert not invalid
    path = tmp_path / "bank.q8_0"
    with open(path, "wb") as f:
        f.write(b"\xEE" * header)       # whatever precedes the tensor in a model file
        f.write(blocks.tobytes())
        f.write(b"\xDD" * 777)          # and what follows it
    return str(path), weights.size, header, oracle.q8_0_decode(blocks, weights.size), blocks


def test_open_reports_bad_files_without_a_gpu(tmp_path):
    lib = abi.load()
    handle = ctypes.c_void_p()
    assert lib.hyle_b200_file_stream_open(os.fsencode(str(tmp_path / "absent")), 0, 16, None, ctypes.byref(handle)) == abi.IO_ERROR
    short = tmp_path / "short"
    short.write_bytes(b"x" * 100)
    assert lib.hyle_b200_file_stream_open(os.fsencode(str(short)), 50, 51, None, ctypes.byref(handle)) == abi.IO_ERROR
    options = abi.FileStreamOptions(1024, 1, 0, 0)   # a ring of one slot cannot overlap anything
    assert lib.hyle_b200_file_stream_open(os.fsencode(str(short)), 0, 100, ctypes.addressof(options), ctypes.byref(handle)) == abi.INVALID_VALUE
    assert lib.hyle_b200_file_stream_open(None, 0, 0, None, ctypes.byref(handle)) == abi.INVALID_VALUE
    assert b"file stream" in lib.hyle_b200_result_string(abi.IO_ERROR)
    assert lib.hyle_b200_file_stream_close(None) == abi.OK


@pytest.mark.gpu
@pytest.mark.parametrize("chunk_bytes,slots", [(0, 0), (1 << 20, 2), (300_000, 3), (34 * 8, 2)])
def test_q8_0_bank_streams_from_disk_and_decodes_bit_exactly(tmp_path, chunk_bytes, slots):
    rows = 96 if chunk_bytes != 34 * 8 else 2
    path, count, header, want, _ = _bank(tmp_path, rows)
    for _ in range(2):
        out, report = ops.q8_0_decode_file(path, count, file_offset=header, chunk_bytes=chunk_bytes, slots=slots)
        torch.cuda.synchronize()
        assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)
        nbytes = count // 32 * 34
        assert report.bytes_read == nbytes and report.bytes_copied == nbytes
        assert report.chunk_bytes % (34 * 8) == 0 and report.copies == report.chunks == -(-nbytes // report.chunk_bytes)
        assert report.staging_bytes == report.device_bytes == report.chunk_bytes * (slots or 4)


@pytest.mark.gpu
def test_chunks_arrive_in_file_order_and_slots_are_recycled(tmp_path):
    path, count, header, _, blocks = _bank(tmp_path, 64)
    nbytes = blocks.size
    pieces = []
    runtime = ctypes.CDLL("libcudart.so.12")  # the runtime torch and the kernel library already share
    with ops.FileStream(path, nbytes, file_offset=header, chunk_bytes=50_000, slots=2) as stream:
        for pointer, size, offset in stream:
            piece = torch.empty(size, dtype=torch.uint8, device="cuda")
            # copy out on the consumer's stream before asking for the next chunk (which may recycle this slot)
            assert runtime.cudaMemcpyAsync(ctypes.c_void_p(piece.data_ptr()), ctypes.c_void_p(pointer), ctypes.c_size_t(size), 3,
                                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0  # 3 = device to device
            pieces.append((offset, piece))
        report = stream.report()
    torch.cuda.synchronize()
    assert [offset for offset, _ in pieces] == list(range(0, nbytes, 50_000))
    assert np.array_equal(torch.cat([p for _, p in pieces]).cpu().numpy(), blocks)
    assert report.chunks == len(pieces) > 4 and report.io_calls >= report.chunks


@pytest.mark.gpu
def test_a_file_that_ends_inside_the_range_is_an_error_not_a_hang(tmp_path):
    path, count, header, _, blocks = _bank(tmp_path, 64)   # 557 056 bytes: nine chunks of 64 KiB
    lib = abi.load()
    handle = ctypes.c_void_p()
    options = abi.FileStreamOptions(65536, 2, 0, 0)
    assert lib.hyle_b200_file_stream_open(os.fsencode(path), header, blocks.size, ctypes.addressof(options), ctypes.byref(handle)) == abi.OK
    os.truncate(path, header + 100_000)          # the file shrinks under the open stream
    codes = []
    for _ in range(8):
        pointer, size = ctypes.c_void_p(), ctypes.c_uint64()
        codes.append(lib.hyle_b200_file_stream_next(handle, torch.cuda.current_stream().cuda_stream, ctypes.byref(pointer),
                                                    ctypes.byref(size), None))
        if codes[-1] != abi.OK:
            break
    assert codes[-1] == abi.IO_ERROR and codes.count(abi.OK) >= 1
    assert lib.hyle_b200_file_stream_close(handle) == abi.OK


@pytest.mark.gpu
def test_a_group_of_ranges_lands_in_the_callers_tensors(tmp_path):
    """read_group: ranges of one file -> device tensors of the caller's own (how the tensors of a weight file reach
    their buffers): ragged sizes, unaligned offsets and destinations, a range longer than all slots together, an
    empty range; two groups in a row reuse the slots; a range beyond the end is refused before anything is copied."""
    rng = np.random.default_rng(5)
    payload = rng.integers(0, 256, 3_000_001, dtype=np.uint8)
    path = tmp_path / "weights.bin"
    payload.tofile(path)
    with ops.FileStream(str(path), 0, chunk_bytes=64 << 10, slots=3) as stream:
        assert stream.report().device_bytes == 0 and stream.report().staging_bytes == 3 * (64 << 10)
        big = torch.zeros(1_000_003, dtype=torch.uint8, device="cuda")
        odd = torch.zeros(4099, dtype=torch.uint8, device="cuda")[3:]            # an unaligned destination
        words = torch.zeros(1000, dtype=torch.float32, device="cuda")
        empty = torch.zeros(0, dtype=torch.uint8, device="cuda")
        stream.read_group([(17, big), (2_000_000, odd), (1_500_000, words), (5, empty)])
        tail = torch.zeros(257, dtype=torch.uint8, device="cuda")
        stream.read_group([(payload.size - 257, tail)])
        torch.cuda.synchronize()
        assert np.array_equal(big.cpu().numpy(), payload[17:17 + big.numel()])
        assert np.array_equal(odd.cpu().numpy(), payload[2_000_000:2_000_000 + odd.numel()])
        assert np.array_equal(words.cpu().numpy().view(np.uint8), payload[1_500_000:1_500_000 + 4000])
        assert np.array_equal(tail.cpu().numpy(), payload[-257:])
        report = stream.report()
        assert report.bytes_copied == big.numel() + odd.numel() + 4000 + 257 and report.copies >= 16 + 1 + 1 + 1
        before = big.clone()
        with pytest.raises(abi.KernelError):
            stream.read_group([(0, big), (payload.size - 100, tail)])             # the second range ends beyond the file
        torch.cuda.synchronize()
        assert torch.equal(big, before)                                           # refused as a whole
    with ops.FileStream(str(path), 1024) as sequential:                           # a sequential stream has no groups
        with pytest.raises(abi.KernelError):
            sequential.read_group([(0, tail)])

"""The cross-GPU sum fused into the Q8_0 round trip (hyle_b200_q8_0_roundtrip_bf16_exchange).

On one GPU: a world of one exchanges with itself, and a world of two whose second mailbox nobody
writes makes the bounded wait run out, which must end the kernel normally with the timeout status.
On two or more GPUs (skipped otherwise): two processes, one per GPU, mailboxes mapped through CUDA
IPC; both must report the same bits, equal to the sum of the two shards' own sums.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mailbox(abi, lib):
    pointer = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(abi.EXCHANGE_HANDLE_BYTES)
    abi.check("create", lib.hyle_b200_exchange_create(ctypes.byref(pointer), handle))
    return pointer


def _call(abi, lib, ops, x, pointers, world, rank, epoch, poll_limit):
    count = x.numel()
    workspace = ops.make_workspace("cuda", count)
    blocks = ops.new_output(ops.q8_0_bytes(count), torch.uint8)
    decoded = ops.new_output(x.shape, x.dtype)
    total = ops.new_output(1, torch.float64).zero_()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    abi.check("exchange", lib.hyle_b200_q8_0_roundtrip_bf16_exchange(
        torch.cuda.current_stream().cuda_stream, x.data_ptr(), count, blocks.data_ptr(), decoded.data_ptr(),
        total.data_ptr(), status.data_ptr(), workspace.data_ptr(), workspace.numel(), pointers, world, rank,
        epoch, poll_limit))
    torch.cuda.synchronize()
    return blocks, decoded, float(total.item()), int(status.item())


def test_world_of_one_matches_plain_round_trip():
    from hyle_b200 import abi, ops

    lib = abi.load()
    x = (torch.randn(96, 8192, device="cuda") * 0.02).to(torch.bfloat16)
    plain_blocks, plain_decoded, plain_sum = ops.q8_0_roundtrip(x, ops.make_workspace("cuda", x.numel()))
    box = _mailbox(abi, lib)
    try:
        pointers = (ctypes.c_void_p * 1)(box.value)
        for epoch in (1, 2, 3):
            blocks, decoded, total, status = _call(abi, lib, ops, x, pointers, 1, 0, epoch, 0)
            assert status == 0
            assert total == float(plain_sum.item())
            assert torch.equal(blocks, plain_blocks) and torch.equal(decoded, plain_decoded)
    finally:
        lib.hyle_b200_exchange_destroy(box)


def test_wait_runs_out_and_context_survives():
    from hyle_b200 import abi, ops

    lib = abi.load()
    x = (torch.randn(64, 8192, device="cuda") * 0.02).to(torch.bfloat16)
    own, silent = _mailbox(abi, lib), _mailbox(abi, lib)  # nobody ever writes for rank 1
    try:
        pointers = (ctypes.c_void_p * 2)(own.value, silent.value)
        blocks, decoded, total, status = _call(abi, lib, ops, x, pointers, 2, 0, 1, 2000)
        assert status & abi.STATUS_EXCHANGE_TIMEOUT
        assert np.isnan(total)
        # the kernel ended normally: outputs are complete and the next call works
        plain_blocks, plain_decoded, plain_sum = ops.q8_0_roundtrip(x, ops.make_workspace("cuda", x.numel()))
        assert torch.equal(blocks, plain_blocks) and torch.equal(decoded, plain_decoded)
        assert np.isfinite(float(plain_sum.item()))
    finally:
        lib.hyle_b200_exchange_destroy(own)
        lib.hyle_b200_exchange_destroy(silent)


def test_argument_checks():
    from hyle_b200 import abi, ops

    lib = abi.load()
    x = torch.zeros(32, dtype=torch.bfloat16, device="cuda")
    box = _mailbox(abi, lib)
    try:
        pointers = (ctypes.c_void_p * 1)(box.value)
        for world, rank, epoch in ((0, 0, 1), (9, 0, 1), (1, 1, 1), (1, 0, 0)):
            with pytest.raises(abi.KernelError):
                _call(abi, lib, ops, x, pointers, world, rank, epoch, 0)
    finally:
        lib.hyle_b200_exchange_destroy(box)


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["HYLE_B200_ROOT"])
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
from hyle_b200 import abi, ops, workloads as wl
from hyle_b200.collective import PeerExchange
lib = abi.load()
peers = PeerExchange()
shard = wl.shard_rows(2048, world, rank)
x = wl.q8_sweep_device_shard(shard)
count = x.numel()
workspace = ops.make_workspace("cuda", count)
blocks = torch.empty(ops.q8_0_bytes(count), dtype=torch.uint8, device="cuda")
decoded = torch.empty_like(x)
total = torch.zeros(1, dtype=torch.float64, device="cuda")
status = torch.zeros(1, dtype=torch.int32, device="cuda")
own = ops.q8_0_roundtrip(x, ops.make_workspace("cuda", count))[2].item()
values = []
for _ in range(5):
    abi.check("exchange", lib.hyle_b200_q8_0_roundtrip_bf16_exchange(
        torch.cuda.current_stream().cuda_stream, x.data_ptr(), count, blocks.data_ptr(), decoded.data_ptr(),
        total.data_ptr(), status.data_ptr(), workspace.data_ptr(), workspace.numel(), peers.pointers, world, rank,
        peers.next_epoch(), 1 << 22))
    torch.cuda.synchronize()
    values.append(total.item())
assert int(status.item()) == 0, status
gathered = [None] * world
dist.all_gather_object(gathered, (own, values))
expected = 0.0
for part, _ in gathered:
    expected += part            # rank order, as the kernel adds
for _, seen in gathered:
    assert all(v == expected for v in seen), (seen, expected)
peers.close()
dist.destroy_process_group()
print("exchange ok", rank, expected)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_agree_bit_for_bit(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    environment = dict(os.environ, HYLE_B200_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", WORLD_SIZE="2")
    workers = [subprocess.Popen([sys.executable, str(script)], env=dict(environment, RANK=str(r)),
                                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outputs = []
    for worker in workers:
        try:
            out, _ = worker.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            worker.kill()
            out, _ = worker.communicate()
        outputs.append(out)
    for worker, out in zip(workers, outputs):
        assert worker.returncode == 0 and "exchange ok" in out, out[-2000:]

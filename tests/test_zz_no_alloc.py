"""The workspace-free Q8_0 round trip (`hyle_b200_q8_0_roundtrip_bf16_static`).

It exists for callers that cannot allocate device memory (a host framework that owns the whole
device pool, an enqueue path that must not allocate, a fixed start-up memory budget): its scratch
is an array inside the library image instead of a caller-supplied workspace.  The test calls it
through the C ABI twice in a row -- the second call meets whatever the first left in the shared
scratch -- and compares every output with the ordinary entry point's.  Collected last on purpose
(file name), so a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from hyle_b200 import abi, ops
from hyle_b200 import workloads as wl

pytestmark = pytest.mark.gpu

F32_REL = 1e-5  # the tolerance the other tests use for the f32 sum of squares


def _bf16_dev(words):
    return torch.from_numpy(words.view(np.int16)).to("cuda").view(torch.bfloat16)


@pytest.mark.parametrize("rows", [3, 1024])
def test_static_scratch_round_trip_matches_workspace_round_trip_twice(rows):
    lib = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    x = _bf16_dev(wl.q8_sweep_inputs(rows))
    count = x.numel()
    # reference results from the existing entry point (caller-supplied workspace)
    workspace = ops.make_workspace("cuda", count)
    want_blocks, want_decoded, want_sum = ops.q8_0_roundtrip(x, workspace)
    torch.cuda.synchronize()

    blocks = ops.new_output(ops.q8_0_bytes(count), torch.uint8)
    decoded = ops.new_output(x.shape, x.dtype)
    total = ops.new_output(1, torch.float64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sums = []
    for call in range(2):
        blocks.fill_(0xAB)
        decoded.zero_()
        total.fill_(-1.0)
        code = lib.hyle_b200_q8_0_roundtrip_bf16_static(stream, x.data_ptr(), count, blocks.data_ptr(),
                                                        decoded.data_ptr(), total.data_ptr(), status.data_ptr())
        assert code == abi.OK, f"call {call}: {lib.hyle_b200_result_string(code)}"
        torch.cuda.synchronize()
        assert torch.equal(blocks, want_blocks), f"call {call}: Q8_0 bytes differ"
        assert torch.equal(decoded.view(torch.int16), want_decoded.view(torch.int16)), f"call {call}: decoded differs"
        assert abs(total.item() - want_sum.item()) <= F32_REL * abs(want_sum.item()), f"call {call}: sum differs"
        assert status.item() == 0
        sums.append(total.cpu().numpy().view(np.uint64)[0])
    # deterministic for one device and grid: two calls in a row return the same bits (they need not be
    # the workspace entry's bits, whose summation order differs)
    assert sums[0] == sums[1]


def test_static_scratch_rejects_counts_beyond_its_capacity():
    lib = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(128, dtype=torch.uint8, device="cuda")
    total = torch.full((1,), 7.0, dtype=torch.float64, device="cuda")
    too_many = abi.STATIC_MAX_VALUES + 32
    code = lib.hyle_b200_q8_0_roundtrip_bf16_static(stream, x.data_ptr(), too_many, out.data_ptr(), out.data_ptr(),
                                                    total.data_ptr(), None)
    assert code == abi.STATIC_SCRATCH_EXCEEDED
    assert b"STATIC_MAX_VALUES" in lib.hyle_b200_result_string(code)
    torch.cuda.synchronize()
    assert total.item() == 7.0  # nothing was launched
    # the ordinary argument checks still apply
    assert lib.hyle_b200_q8_0_roundtrip_bf16_static(stream, x.data_ptr(), 33, out.data_ptr(), out.data_ptr(),
                                                    total.data_ptr(), None) == abi.INVALID_VALUE

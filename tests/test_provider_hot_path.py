"""The adapter's HOT path on a GPU, through the reference's own submit().

`tests/provider/hot_path_test.cc` creates a reference `Context` on the thin CUDA-12 backend
(hyle_b200/provider/b200_backend.cc), and for each of the adapter's 22 entries runs
prepare -> create_invocation (poisoned caller workspace) -> submit -> wait twice through the reference's
`OperationInvocation::submit` (src/compute/operation.cc:1878-1957), comparing every output byte with the
direct C-ABI call; then the error protocol (device status word -> the Completion's terminal Status), and
three host threads with a Queue each that prepare and submit concurrently on the one Context.
The program is built where the reference tree is mounted (tests/provider/Makefile) and travels as a
prebuilt binary under oracle/_ref/provider.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "oracle", "_ref", "provider", "b200_hot_path_test")


# the plain build, and the build with the adapter's trace zones compiled in (-DHYLE_B200_NVTX, b200_trace.h)
@pytest.mark.gpu
@pytest.mark.parametrize("binary", [BINARY, BINARY + "_trace"], ids=["plain", "trace-zones"])
def test_every_entry_runs_under_the_reference_submit_and_matches_the_direct_call(binary):
    if not os.path.exists(binary):
        pytest.skip("no prebuilt %s (built where the reference tree is mounted)" % os.path.relpath(binary, ROOT))
    run = subprocess.run([binary], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-6000:] + run.stderr[-3000:]
    assert "0 failure(s)" in run.stdout and "FAIL" not in run.stdout
    assert run.stdout.count("ok  ") >= 30
    for line in ("every Entry of the adapter (22) ran through submit()",
                 "CacheEncode{q8_0} with a NaN completes with Status::InvalidArgument",
                 "Scan i32 whose prefix leaves int32 completes with Status::OutOfRange",
                 "concurrent Queues: b200-q8_0-roundtrip", "concurrent Queues: b200-logits-reduce",
                 "concurrent Queues: CacheEncode{q8_0}"):
        assert line in run.stdout


REGION_BINARY = os.path.join(ROOT, "oracle", "_ref", "provider", "b200_region_test")


@pytest.mark.gpu
def test_graph_regions_replay_on_the_gpu_and_match_the_fused_kernels():
    """`tests/provider/region_test.cc`, GPU half: the model graph (residual add + norm, silu * up, softmax ->
    bf16 beside a greedy TopK) compiled by the reference's graph::compile with the region provider, replayed
    through graph::Invocation::submit on a Queue of the CUDA-12 backend; every published value equals the
    direct C-ABI call of the fused kernel byte for byte."""
    if not os.path.exists(REGION_BINARY):
        pytest.skip("no prebuilt oracle/_ref/provider/b200_region_test (built where the reference tree is mounted)")
    run = subprocess.run([REGION_BINARY], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-6000:] + run.stderr[-3000:]
    assert "0 failure(s)" in run.stdout and "FAIL" not in run.stdout
    assert run.stdout.count("ok    GPU:") >= 5 and "the GPU half was skipped" not in run.stdout

"""Host logic of the row-sharded Q8_0 sweep, on CPU: shard arithmetic, and the world_size-2 path
(per-rank partial sums of squares combined by one all-reduce) over gloo with the CPU checker
standing in for the kernel."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from hyle_b200 import workloads as wl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("total,world", [(1024, 1), (1024, 2), (262144, 8), (1000, 3), (5, 8), (0, 4)])
def test_shards_partition_the_rows(total, world):
    shards = [wl.shard_rows(total, world, r) for r in range(world)]
    assert shards[0].first_row == 0
    assert sum(s.rows for s in shards) == total
    for a, b in zip(shards, shards[1:]):
        assert a.first_row + a.rows == b.first_row
    assert max(s.rows for s in shards) - min(s.rows for s in shards) <= 1


def test_shard_rows_rejects_bad_ranks():
    with pytest.raises(ValueError):
        wl.shard_rows(10, 2, 2)
    with pytest.raises(ValueError):
        wl.shard_rows(10, 0, 0)


def test_workload_generators_are_deterministic_and_shaped():
    a1, b1 = wl.broadcast_add_inputs(8, 64)
    a2, b2 = wl.broadcast_add_inputs(8, 64)
    assert np.array_equal(a1, a2) and np.array_equal(b1, b2) and np.abs(b1).max() <= 1.0
    logits, tied = wl.logits_inputs(16, cols=512)
    assert logits.shape == (16, 512) and len(tied) >= 1
    for row in tied:
        assert (logits[row] == logits[row].max()).sum() >= 2
    w = wl.q8_sweep_inputs(4)
    assert w.shape == (4, wl.SWEEP_COLS) and w.dtype == np.uint16
    assert 0.015 < wl.bf16_to_f32(w).std() < 0.025


RANK_SCRIPT = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, os.environ["HYLE_ROOT"])
    import numpy as np, torch, torch.distributed as dist
    from hyle_b200 import workloads as wl
    from oracle.binding import Oracle
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rows = 64
    full = wl.q8_sweep_inputs(rows)
    shard = wl.shard_rows(rows, world, rank)
    mine = full[shard.first_row: shard.first_row + shard.rows]
    oracle = Oracle(); oracle.set_threads(1)
    blocks, decoded, partial, invalid = oracle.q8_0_roundtrip(mine)
    total = torch.tensor([partial], dtype=torch.float64)
    dist.all_reduce(total)                                  # the one exchange of the path
    want_blocks, want_decoded, want_total, _ = oracle.q8_0_roundtrip(full)
    lo = shard.first_row * wl.SWEEP_COLS
    assert np.array_equal(blocks, want_blocks[lo // 32 * 34: (lo + mine.size) // 32 * 34])
    assert np.array_equal(decoded, want_decoded[lo: lo + mine.size])
    assert abs(total.item() - want_total) <= 1e-12 * want_total
    dist.barrier(); dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_rank_sweep_over_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, HYLE_ROOT=ROOT, OMP_NUM_THREADS="1")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
        env=env, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-2000:]
    assert result.stdout.count("ok") == 2


EXCHANGE_SCRIPT = textwrap.dedent("""
    import ctypes, os, sys
    sys.path.insert(0, os.environ["HYLE_ROOT"])
    import torch.distributed as dist
    from hyle_b200.collective import PeerExchange, PeerMappingUnavailable

    class FakeLibrary:
        # The four set-up calls of the kernel library, on host memory; `refuse` makes this rank's
        # mapping of rank 0's mailbox fail the way a refused CUDA IPC open does.
        def __init__(self, rank, refuse):
            self.rank, self.refuse, self.live = rank, refuse, 0
        def hyle_b200_exchange_create(self, mailbox, handle):
            mailbox._obj.value = 0x1000 * (self.rank + 1)
            handle.raw = bytes([self.rank + 1]) * 64
            self.live += 1
            return 0
        def hyle_b200_exchange_open(self, raw, mapped):
            if self.refuse and raw[0] == 1:
                return 201
            mapped._obj.value = 0x100000 * raw[0]
            self.live += 1
            return 0
        def hyle_b200_exchange_close(self, mapped):
            self.live -= 1
            return 0
        def hyle_b200_exchange_destroy(self, mailbox):
            self.live -= 1
            return 0

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # 1: everything maps -> a complete pointer table on every rank, epochs 1, 2, 3
    library = FakeLibrary(rank, refuse=False)
    peers = PeerExchange(library)
    table = [peers.pointers[r] for r in range(world)]
    assert table[rank] == 0x1000 * (rank + 1)
    assert all(table[r] == 0x100000 * (r + 1) for r in range(world) if r != rank)
    assert [peers.next_epoch() for _ in range(3)] == [1, 2, 3]
    peers.epoch = 0xFFFFFFFE
    assert peers.next_epoch() == 1                      # wraps without repeating a parity
    peers.close()
    assert library.live == 0
    # 2: one rank cannot map a peer -> EVERY rank raises, nothing stays mapped
    library = FakeLibrary(rank, refuse=(rank == 1))
    try:
        PeerExchange(library)
        raise SystemExit("no exception on rank %d" % rank)
    except PeerMappingUnavailable as problem:
        assert "rank 1" in str(problem)
    assert library.live == 0
    dist.barrier(); dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_peer_exchange_setup_is_collective_over_gloo(tmp_path):
    """The mailbox set-up of the fused exchange with a stand-in for the kernel library: either all
    ranks end with a full table or all raise together."""
    script = tmp_path / "exchange.py"
    script.write_text(EXCHANGE_SCRIPT)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
        env=dict(os.environ, HYLE_ROOT=ROOT), capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-2000:]
    assert result.stdout.count("ok") == 2

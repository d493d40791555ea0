"""Seeded synthetic inputs for the five benchmark workloads, and the row sharding of the sweep.

Host generators return numpy arrays (bf16 as uint16 storage words) so the CPU checker and the GPU
kernels read the very same bits; device generators build the large tensors in HBM for timing.
Shapes follow a Qwen3.5-2B-like model: hidden 2048, FFN 6144, vocabulary 151936.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

import numpy as np

HIDDEN = 2048
FFN = 6144
VOCAB = 151936
SWEEP_COLS = 8192
SWEEP_ROWS = [1024 << i for i in range(9)]  # 1024 ... 262144 (16 MiB ... 4 GiB of bf16)

SEEDS = {1: 0xB2000001, 2: 0xB2000002, 3: 0xB2000003, 4: 0xB2000004, 5: 0xB2000005}


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 storage words (finite inputs; NaN keeps a quiet NaN)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    a = u & np.uint32(0x7FFFFFFF)
    incr = np.where(a < 0x7F800000, np.uint32(0x7FFF) + ((u >> 16) & 1), np.uint32(0)).astype(np.uint32)
    quiet = np.where(a > 0x7F800000, np.uint32(1 << 6), np.uint32(0)).astype(np.uint32)
    return (quiet | ((u + incr) >> 16)).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _rng(config: int, salt: int = 0) -> np.random.Generator:
    return np.random.default_rng([SEEDS[config], salt])


def broadcast_add_inputs(rows: int = 4096, cols: int = 4096) -> Tuple[np.ndarray, np.ndarray]:
    """Workload 1: A ~ N(0,1) f32 [rows, cols], bias ~ U(-1,1) f32 [cols]."""
    rng = _rng(1)
    a = rng.standard_normal((rows, cols), dtype=np.float32)
    bias = rng.uniform(-1.0, 1.0, cols).astype(np.float32)
    return a, bias


def rms_norm_inputs(tokens: int, hidden: int = HIDDEN):
    """Workload 2: x, residual ~ N(0,1) bf16 [tokens, hidden]; weight ~ U(0.5,1.5) as bf16 and f32."""
    rng = _rng(2, tokens)
    x = f32_to_bf16(rng.standard_normal((tokens, hidden), dtype=np.float32))
    residual = f32_to_bf16(rng.standard_normal((tokens, hidden), dtype=np.float32))
    weight_f32 = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    return x, residual, f32_to_bf16(weight_f32), weight_f32


def swiglu_inputs(tokens: int, cols: int = FFN):
    """Workload 3: gate, up ~ N(0, 1.5^2) bf16 [tokens, cols]."""
    rng = _rng(3, tokens)
    gate = f32_to_bf16(1.5 * rng.standard_normal((tokens, cols), dtype=np.float32))
    up = f32_to_bf16(1.5 * rng.standard_normal((tokens, cols), dtype=np.float32))
    return gate, up


def logits_inputs(batch: int, cols: int = VOCAB, tie_rows: bool = True) -> Tuple[np.ndarray, List[int]]:
    """Workload 4: logits ~ N(0, 4^2) f32 [batch, cols].

    In 1 % of the rows (at least one when batch >= 16, and row 0 when tie_rows is set for smaller
    batches) the row maximum is copied to one lower and one higher index, so the lowest-index rule
    decides the argmax.  Returns the logits and the list of tied rows.
    """
    rng = _rng(4, batch)
    logits = (4.0 * rng.standard_normal((batch, cols), dtype=np.float32)).astype(np.float32)
    count = max(1, batch // 100) if (batch >= 16 or tie_rows) else 0
    tied = sorted(rng.choice(batch, size=min(count, batch), replace=False).tolist()) if count else []
    for row in tied:
        peak = int(np.argmax(logits[row]))
        value = logits[row, peak]
        lower = int(rng.integers(0, peak)) if peak > 0 else peak
        higher = int(rng.integers(peak + 1, cols)) if peak + 1 < cols else peak
        logits[row, lower] = value
        logits[row, higher] = value
    return logits, tied


def q8_sweep_inputs(rows: int, cols: int = SWEEP_COLS) -> np.ndarray:
    """Workload 5: W ~ N(0, 0.02^2) bf16 [rows, cols] (host copy; small row counts only)."""
    rng = _rng(5)
    return f32_to_bf16(0.02 * rng.standard_normal((rows, cols), dtype=np.float32))


# ---- row sharding of the sweep -------------------------------------------------------------------
@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    first_row: int
    rows: int


def shard_rows(total_rows: int, world: int, rank: int) -> RowShard:
    """Contiguous row blocks; the first ``total_rows % world`` ranks take one extra row.

    A Q8_0 block is 32 consecutive values of one row, so no block crosses a shard and the shards
    need no exchange except the sum of the per-shard sums of squares.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(total_rows, world)
    rows = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return RowShard(rank, world, first, rows)


GENERATOR_CHUNK_ROWS = 1024


def q8_sweep_device_shard(shard: RowShard, cols: int = SWEEP_COLS, device="cuda"):
    """The shard's rows of W ~ N(0, 0.02^2) as a bf16 CUDA tensor.

    Rows are generated in chunks of 1024 rows, each chunk from its own seed, so a row holds the same
    values whatever the number of shards (shard boundaries of the sweep are multiples of 1024 rows).
    """
    import torch

    out = torch.empty((shard.rows, cols), dtype=torch.bfloat16, device=device)
    generator = torch.Generator(device=device)
    row = shard.first_row
    end = shard.first_row + shard.rows
    while row < end:
        chunk = row // GENERATOR_CHUNK_ROWS
        chunk_first = chunk * GENERATOR_CHUNK_ROWS
        chunk_rows = min(GENERATOR_CHUNK_ROWS, end - chunk_first)
        generator.manual_seed(SEEDS[5] * 1_000_003 + chunk)
        values = torch.randn((GENERATOR_CHUNK_ROWS, cols), generator=generator, device=device,
                             dtype=torch.float32).mul_(0.02).to(torch.bfloat16)
        take_from = row - chunk_first
        take = min(chunk_rows - take_from, end - row)
        out[row - shard.first_row: row - shard.first_row + take] = values[take_from: take_from + take]
        row += take
    return out

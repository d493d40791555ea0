"""Paged append (KV cache row mover): oracle against a plain numpy model on CPU; on the GPU the
product kernel against the oracle and, where it was built, against the reference's own CUDA kernel.
Bytes are moved, so every comparison is bit-exact."""
import numpy as np
import pytest
import torch

from hyle_b200 import abi, ops
from oracle import binding as ob


def make_episode(seed, page_rows, pages, input_rows, capacity, malformed=True):
    """Random instructions with disjoint destinations: destinations in the lower half of the pages
    (one range per page), arena sources in the upper half.  Returns (uint32 words, good count)."""
    rng = np.random.default_rng(seed)
    lower = pages // 2
    instructions = []
    for page in rng.permutation(lower)[: max(1, capacity * 2 // 3)]:
        rows = int(rng.integers(1, page_rows + 1))
        row = int(rng.integers(0, page_rows - rows + 1))
        if rng.random() < 0.6 and input_rows >= rows:
            instructions.append((0, int(rng.integers(0, 1 << 32)), int(rng.integers(0, input_rows - rows + 1)), int(page), row, rows))
        else:
            instructions.append((1, int(rng.integers(lower, pages)), int(rng.integers(0, page_rows - rows + 1)), int(page), row, rows))
    good = len(instructions)
    bad = []
    if malformed:
        bad = [
            (0, 0, 0, 0, 0, 0),                              # no rows
            (2, 0, 0, 0, 0, 1),                              # unknown source kind
            (0, 0, 0, pages, 0, 1),                          # destination page outside the arena
            (0, 0, 0, 0, page_rows, 1),                      # destination row overflow
            (0, 0, 0, 0, page_rows + 1, 0xFFFFFFFF),         # unsigned wrap in rows
            (0, 0, input_rows, 0, 0, 1),                     # input overflow
            (0, 0, 0xFFFFFFFF, 0, 0, 2),                     # source row wrap
            (1, pages, 0, 0, 0, 1),                          # source page outside the arena
            (1, lower, page_rows, 0, 0, 1),                  # source row overflow
        ]
    everything = instructions + bad
    order = rng.permutation(len(everything))
    everything = [everything[i] for i in order][:capacity]
    words = np.zeros(4 + 8 * capacity, np.uint32)
    words[0] = len(everything)
    for slot, fields in enumerate(everything):
        words[4 + 8 * slot: 10 + 8 * slot] = fields
    return words, good


def numpy_model(arena, new_rows, words, page_rows):
    """Row-at-a-time model written straight from the wire format."""
    arena = arena.copy()
    pages = arena.shape[0] // page_rows
    capacity = (words.size - 4) // 8
    if words[0] > capacity or words[1:4].any():
        return arena
    before = arena.copy()  # ranges are disjoint: sources can be read from the state before the episode
    for i in range(int(words[0])):
        kind, spage, srow, page, row, rows, r0, r1 = (int(w) for w in words[4 + 8 * i: 12 + 8 * i])
        if r0 or r1 or rows == 0 or kind > 1 or page >= pages or row + rows > page_rows:
            continue
        if kind == 0:
            if srow + rows > new_rows.shape[0]:
                continue
            source = new_rows[srow: srow + rows]
        else:
            if spage >= pages or srow + rows > page_rows:
                continue
            source = before[spage * page_rows + srow: spage * page_rows + srow + rows]
        arena[page * page_rows + row: page * page_rows + row + rows] = source
    return arena


@pytest.fixture(scope="module")
def oracle():
    return ob.Oracle()


@pytest.mark.parametrize("page_rows,pages,input_rows,capacity,row_bytes", [
    (16, 12, 40, 8, 64), (1, 9, 3, 4, 34), (7, 20, 5, 32, 2), (32, 6, 64, 3, 1088)])
def test_oracle_matches_numpy_model(oracle, page_rows, pages, input_rows, capacity, row_bytes):
    rng = np.random.default_rng(page_rows * 1000 + pages)
    arena = rng.integers(0, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(0, 256, (input_rows, row_bytes), dtype=np.uint8)
    for seed in range(6):
        words, good = make_episode(seed, page_rows, pages, input_rows, capacity)
        want = numpy_model(arena, new_rows, words, page_rows)
        got = oracle.paged_append(arena, new_rows, words, page_rows)
        assert np.array_equal(got, want)
        if good and seed == 0:
            clean, _ = make_episode(seed, page_rows, pages, input_rows, capacity, malformed=False)
            assert not np.array_equal(oracle.paged_append(arena, new_rows, clean, page_rows), arena)


def test_oracle_malformed_episode_does_nothing(oracle):
    rng = np.random.default_rng(5)
    arena = rng.integers(0, 256, (64, 32), dtype=np.uint8)
    new_rows = rng.integers(0, 256, (8, 32), dtype=np.uint8)
    words, _ = make_episode(1, 8, 8, 8, 4, malformed=False)
    for edit in [(0, 5), (1, 1), (2, 7), (3, 0x80000000)]:  # active_count > capacity, reserved words
        broken = words.copy()
        broken[edit[0]] = edit[1]
        assert np.array_equal(oracle.paged_append(arena, new_rows, broken, 8), arena)
    reserved = words.copy()
    reserved[4 + 6] = 1  # first instruction's reserved word: only that instruction is skipped
    assert np.array_equal(oracle.paged_append(arena, new_rows, reserved, 8), numpy_model(arena, new_rows, reserved, 8))


def test_metadata_packing_matches_wire_format():
    packed = ops.paged_append_metadata([(0, 0, 1, 2, 3, 4), (1, 0xFFFFFFFF, 0, 0, 0, 1)], 3)
    assert packed.dtype == torch.int32 and packed.numel() == 4 + 8 * 3
    words = packed.numpy().view(np.uint32)
    assert words[:4].tolist() == [2, 0, 0, 0]
    assert words[4:12].tolist() == [0, 0, 1, 2, 3, 4, 0, 0]
    assert words[12:20].tolist() == [1, 0xFFFFFFFF, 0, 0, 0, 1, 0, 0]
    assert not words[20:].any()
    with pytest.raises(ValueError):
        ops.paged_append_metadata([(0, 0, 0, 0, 0, 1)] * 2, 1)


# ---- GPU ---------------------------------------------------------------------------------------
def device_bytes(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_product(arena, new_rows, words, page_rows):
    d_arena = device_bytes(arena)
    d_rows = device_bytes(new_rows) if new_rows is not None and new_rows.shape[0] else None
    d_words = torch.from_numpy(words.view(np.int32).copy()).cuda()
    ops.paged_append(d_arena, d_rows, d_words, page_rows)
    torch.cuda.synchronize()
    return d_arena.cpu().numpy()


def run_reference_kernel(ref, arena, new_rows, words, page_rows):
    d_arena = device_bytes(arena)
    d_rows = device_bytes(new_rows)
    d_words = torch.from_numpy(words.view(np.int32).copy()).cuda()
    code = ref.paged_append(torch.cuda.current_stream().cuda_stream, d_arena.data_ptr(), d_rows.data_ptr(), d_words.data_ptr(),
                            page_rows, arena.shape[0] // page_rows, new_rows.shape[0], (words.size - 4) // 8, arena.shape[1])
    assert code == 0
    torch.cuda.synchronize()
    return d_arena.cpu().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("page_rows,pages,input_rows,capacity,row_bytes", [
    (16, 64, 128, 48, 8704),     # a Q8_0 carrier row of 8192 values
    (16, 64, 128, 48, 8192),     # an FP8 row of 8192 values
    (256, 24, 512, 12, 256),     # long pages of short rows: several slices per instruction
    (1, 300, 200, 300, 34),      # one-row pages, a row size without 16-byte alignment
    (7, 40, 9, 20, 2),           # the smallest row
    (33, 10, 70, 5, 20000)])     # slices that end inside a row
def test_paged_append_matches_oracle_and_reference_kernel(oracle, page_rows, pages, input_rows, capacity, row_bytes):
    abi.load()
    rng = np.random.default_rng(row_bytes)
    arena = rng.integers(0, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(0, 256, (input_rows, row_bytes), dtype=np.uint8)
    ref = ob.RefPaged() if ob.RefPaged.available() else None
    for seed in range(4):
        words, _ = make_episode(seed, page_rows, pages, input_rows, capacity)
        want = oracle.paged_append(arena, new_rows, words, page_rows)
        got = run_product(arena, new_rows, words, page_rows)
        assert np.array_equal(got, want)
        if ref is not None:
            assert np.array_equal(run_reference_kernel(ref, arena, new_rows, words, page_rows), want)


@pytest.mark.gpu
def test_paged_append_malformed_episode_unaligned_bases_and_arguments(oracle):
    library = abi.load()
    rng = np.random.default_rng(11)
    page_rows, pages, row_bytes = 8, 16, 48
    arena = rng.integers(0, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(0, 256, (20, row_bytes), dtype=np.uint8)
    words, _ = make_episode(3, page_rows, pages, 20, 8, malformed=False)
    for index, value in [(0, 9), (1, 1), (3, 2)]:
        broken = words.copy()
        broken[index] = value
        assert np.array_equal(run_product(arena, new_rows, broken, page_rows), arena)
    # Bases that are only 2-byte aligned take the 16-bit element path.
    backing = torch.zeros(arena.size + 16, dtype=torch.uint8, device="cuda")
    shifted = backing[2: 2 + arena.size].view(arena.shape)
    shifted.copy_(torch.from_numpy(arena))
    d_words = torch.from_numpy(words.view(np.int32).copy()).cuda()
    ops.paged_append(shifted, device_bytes(new_rows), d_words, page_rows)
    assert np.array_equal(shifted.cpu().numpy(), oracle.paged_append(arena, new_rows, words, page_rows))
    # Arena-only episode without new rows.
    only_arena = words.copy()
    for slot in range(int(only_arena[0])):
        if only_arena[4 + 8 * slot] == 0:
            only_arena[4 + 8 * slot + 5] = 0
    assert np.array_equal(run_product(arena, None, only_arena, page_rows), oracle.paged_append(arena, None, only_arena, page_rows))
    stream = torch.cuda.current_stream().cuda_stream
    d_arena = device_bytes(arena)
    args = (d_arena.data_ptr(), None, d_words.data_ptr())
    assert library.hyle_b200_paged_append(stream, *args, page_rows, pages, 0, 0, row_bytes) == abi.OK
    assert library.hyle_b200_paged_append(stream, *args, page_rows, pages, 0, 8, 47) == abi.INVALID_VALUE
    assert library.hyle_b200_paged_append(stream, *args, 0, pages, 0, 8, row_bytes) == abi.INVALID_VALUE
    assert library.hyle_b200_paged_append(stream, None, None, d_words.data_ptr(), page_rows, pages, 0, 8, row_bytes) == abi.INVALID_VALUE
    assert library.hyle_b200_paged_append(stream, *args, page_rows, pages, 5, 8, row_bytes) == abi.INVALID_VALUE
    torch.cuda.synchronize()
    assert np.array_equal(d_arena.cpu().numpy(), arena)


@pytest.mark.gpu
def test_paged_append_replays_in_a_cuda_graph_with_new_metadata(oracle):
    page_rows, pages, input_rows, capacity, row_bytes = 16, 32, 64, 16, 4352
    rng = np.random.default_rng(2)
    arena = rng.integers(0, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(0, 256, (input_rows, row_bytes), dtype=np.uint8)
    d_arena, d_rows = device_bytes(arena), device_bytes(new_rows)
    d_words = torch.zeros(4 + 8 * capacity, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        ops.paged_append(d_arena, d_rows, d_words, page_rows)  # an empty episode: warm-up
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            ops.paged_append(d_arena, d_rows, d_words, page_rows)
    want = arena
    for seed in range(3):
        words, _ = make_episode(seed, page_rows, pages, input_rows, capacity)
        d_words.copy_(torch.from_numpy(words.view(np.int32).copy()))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        want = oracle.paged_append(want, new_rows, words, page_rows)
        assert np.array_equal(d_arena.cpu().numpy(), want)

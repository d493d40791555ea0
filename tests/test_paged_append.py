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
    """A device copy placed by the operators' output allocator: inside guard bands during a GPU test,
    because the arenas made here are written in place by the kernels under test."""
    a = np.ascontiguousarray(a)
    out = ops.new_output(a.shape, torch.from_numpy(a).dtype)
    out.copy_(torch.from_numpy(a))
    return out


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
    assert int(backing[:2].sum()) == 0 and int(backing[2 + arena.size:].sum()) == 0  # margins untouched
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


# ---- device-lengths variant ----------------------------------------------------------------------
def make_lengths_episode(seed, page_rows, pages, input_rows, capacity, requests):
    """Requests with random history and query lengths and the dirty pages their new rows touch.
    Destinations are distinct pages of the lower half; copy-on-write sources come from the upper half
    (or are the destination itself).  Returns (uint32 words, q, kv)."""
    rng = np.random.default_rng(seed)
    lower = pages // 2
    free = list(rng.permutation(lower))
    budget = input_rows
    bounds, records, q_all, kv_all = [], [], [], []
    room = capacity - 1 - requests
    for r in range(requests):
        previous = int(rng.integers(0, 3 * page_rows))
        q = int(rng.integers(0, min(budget, 2 * page_rows) + 1))
        first, last = previous // page_rows, (previous + q - 1) // page_rows
        if q and (len(free) < last - first + 1 or room < last - first + 1):
            q = 0
        budget -= q
        kv = previous + q
        bounds.append((q + int(rng.integers(0, 3)), max(0, previous - 1), previous + 2, kv + int(rng.integers(0, 5))))
        q_all.append(q), kv_all.append(kv)
        if not q:
            continue
        for logical in range(first, last + 1):
            destination = int(free.pop())
            live = min(page_rows, kv - logical * page_rows)
            initialized = int(rng.integers(live, page_rows + 1))
            inherited = max(0, min(initialized, previous - logical * page_rows))
            if inherited and rng.random() < 0.5:
                source, source_rows = int(rng.integers(lower, pages)), int(rng.integers(inherited, page_rows + 1))
            elif inherited:
                source, source_rows = destination, inherited
            else:
                source, source_rows = 0xFFFFFFFF, 0
            records.append((r, logical, destination, initialized, source, source_rows))
            room -= 1
    words = np.zeros(4 + 8 * capacity, np.uint32)
    words[0] = 1 + requests + len(records)
    words[4:6] = (requests, len(records))
    for r, b in enumerate(bounds):
        words[12 + 8 * r: 16 + 8 * r] = b
    for i, p in enumerate(records):
        words[12 + 8 * (requests + i): 18 + 8 * (requests + i)] = p
    return words, np.array(q_all, np.int32), np.array(kv_all, np.int32)


def lengths_model(arena, new_rows, words, q, kv, page_rows):
    """Row-at-a-time model of a well-formed device-lengths episode."""
    before, arena = arena, arena.copy()
    requests, pages = int(words[4]), int(words[5])
    offsets = np.concatenate([[0], np.cumsum(q)])
    for i in range(pages):
        r, logical, destination, initialized, source = (int(w) for w in words[12 + 8 * (requests + i): 17 + 8 * (requests + i)])
        prior = int(kv[r]) - int(q[r])
        for row in range(initialized):
            g = logical * page_rows + row
            if g < prior:
                value = before[source * page_rows + row]
            elif g < kv[r]:
                value = new_rows[offsets[r] + g - prior]
            else:
                value = 0
            arena[destination * page_rows + row] = value
    return arena


LENGTHS_CASES = [(16, 40, 96, 40, 4, 256), (4, 64, 40, 48, 32, 34), (8, 30, 30, 20, 1, 1088), (3, 50, 20, 30, 7, 2)]


@pytest.mark.parametrize("page_rows,pages,input_rows,capacity,requests,row_bytes", LENGTHS_CASES)
def test_oracle_device_lengths_matches_numpy_model(oracle, page_rows, pages, input_rows, capacity, requests, row_bytes):
    rng = np.random.default_rng(page_rows + pages)
    arena = rng.integers(1, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(1, 256, (input_rows, row_bytes), dtype=np.uint8)
    changed = 0
    for seed in range(8):
        words, q, kv = make_lengths_episode(seed, page_rows, pages, input_rows, capacity, requests)
        got, status = oracle.paged_append_device_lengths(arena, new_rows, words, q, kv, page_rows)
        assert status == 0
        assert np.array_equal(got, lengths_model(arena, new_rows, words, q, kv, page_rows))
        changed += not np.array_equal(got, arena)
    assert changed >= 4


def broken_lengths_episodes(words, q, kv, requests, input_rows, pages):
    """(name, words, q, kv, expected status) for inconsistent episodes built from a well-formed one."""
    cases = []

    def edit(name, status, word=None, value=None, dq=None, dkv=None):
        w, a, b = words.copy(), q.copy(), kv.copy()
        if word is not None:
            w[word] = value
        if dq is not None:
            a[dq[0]] = dq[1]
        if dkv is not None:
            b[dkv[0]] = dkv[1]
        cases.append((name, w, a, b, status))

    edit("no records", 4, 0, 0)
    edit("more records than capacity", 4, 0, (words.size - 4) // 8 + 1)
    edit("header reserved", 4, 2, 1)
    edit("directory names other request count", 4, 4, requests + 1)
    edit("directory pages exceed records", 4, 5, int(words[0]))
    edit("directory reserved", 4, 9, 1)
    edit("bounds reserved", 4, 12 + 5, 1)
    edit("negative query length", 4, dq=(0, -1))
    edit("query longer than its bound", 4, dq=(0, int(words[12]) + 1), dkv=(0, int(kv[0]) + int(words[12]) + 1 - int(q[0])))
    edit("kv beyond its bound", 4, dkv=(0, int(words[15]) + 1))
    edit("history outside its bounds", 4, dkv=(0, int(kv[0]) + 5), word=15, value=int(kv[0]) + 9)
    if int(words[5]):
        page = 12 + 8 * requests
        edit("page of an unknown request", 1, page, requests)
        edit("page outside the arena", 1, page + 2, pages)
        edit("page without rows", 1, page + 3, 0)
        edit("page record reserved", 1, page + 7, 1)
    return cases


def test_oracle_device_lengths_statuses(oracle):
    page_rows, pages, input_rows, capacity, requests, row_bytes = 8, 32, 40, 24, 3, 32
    rng = np.random.default_rng(9)
    arena = rng.integers(1, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(1, 256, (input_rows, row_bytes), dtype=np.uint8)
    words, q, kv = make_lengths_episode(2, page_rows, pages, input_rows, capacity, requests)
    assert int(words[5]) > 0 and q[0] > 0
    got, status = oracle.paged_append_device_lengths(arena, new_rows, words, q, kv, page_rows, status=3)
    assert status == 3 and np.array_equal(got, arena)  # an earlier failure in the sequence: nothing is done
    for name, w, a, b, expected in broken_lengths_episodes(words, q, kv, requests, input_rows, pages):
        got, status = oracle.paged_append_device_lengths(arena, new_rows, w, a, b, page_rows)
        assert status == expected, name
        if expected == 4:
            assert np.array_equal(got, arena), name


def run_lengths(call, arena, new_rows, words, q, kv, page_rows, status=0):
    d_arena, d_rows = device_bytes(arena), device_bytes(new_rows)
    d_words = torch.from_numpy(words.view(np.int32).copy()).cuda()
    d_q, d_kv = torch.from_numpy(q.copy()).cuda(), torch.from_numpy(kv.copy()).cuda()
    d_status = torch.full((1,), status, dtype=torch.int32, device="cuda")
    call(d_arena, d_rows, d_words, d_q, d_kv, d_status)
    torch.cuda.synchronize()
    return d_arena.cpu().numpy(), int(d_status.item())


def product_lengths(page_rows):
    return lambda arena, rows, words, q, kv, status: ops.paged_append_device_lengths(arena, rows, words, q, kv, page_rows, status)


def reference_lengths(ref, page_rows):
    def call(arena, rows, words, q, kv, status):
        code = ref.paged_append_device_lengths(
            torch.cuda.current_stream().cuda_stream, arena.data_ptr(), rows.data_ptr(), words.data_ptr(), q.data_ptr(),
            kv.data_ptr(), page_rows, arena.shape[0] // page_rows, rows.shape[0], (words.numel() - 4) // 8,
            arena.shape[1], q.numel(), status.data_ptr())
        assert code == 0
    return call


@pytest.mark.gpu
@pytest.mark.parametrize("page_rows,pages,input_rows,capacity,requests,row_bytes",
                         LENGTHS_CASES + [(16, 128, 512, 100, 32, 8704), (64, 24, 200, 16, 2, 4352), (5, 40, 33, 30, 6, 40000)])
def test_device_lengths_matches_oracle_and_reference_kernel(oracle, page_rows, pages, input_rows, capacity, requests, row_bytes):
    abi.load()
    rng = np.random.default_rng(row_bytes + requests)
    arena = rng.integers(1, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(1, 256, (input_rows, row_bytes), dtype=np.uint8)
    ref = ob.RefPaged() if ob.RefPaged.available() else None
    for seed in range(5):
        words, q, kv = make_lengths_episode(seed, page_rows, pages, input_rows, capacity, requests)
        want, want_status = oracle.paged_append_device_lengths(arena, new_rows, words, q, kv, page_rows)
        got, status = run_lengths(product_lengths(page_rows), arena, new_rows, words, q, kv, page_rows)
        assert status == want_status == 0
        assert np.array_equal(got, want)
        if ref is not None:
            theirs, their_status = run_lengths(reference_lengths(ref, page_rows), arena, new_rows, words, q, kv, page_rows)
            assert their_status == 0 and np.array_equal(theirs, want)


@pytest.mark.gpu
def test_device_lengths_statuses_match_the_reference_kernel(oracle):
    library = abi.load()
    page_rows, pages, input_rows, capacity, requests, row_bytes = 8, 32, 40, 24, 3, 32
    rng = np.random.default_rng(9)
    arena = rng.integers(1, 256, (pages * page_rows, row_bytes), dtype=np.uint8)
    new_rows = rng.integers(1, 256, (input_rows, row_bytes), dtype=np.uint8)
    words, q, kv = make_lengths_episode(2, page_rows, pages, input_rows, capacity, requests)
    ref = ob.RefPaged() if ob.RefPaged.available() else None
    got, status = run_lengths(product_lengths(page_rows), arena, new_rows, words, q, kv, page_rows, status=3)
    assert status == 3 and np.array_equal(got, arena)
    for name, w, a, b, expected in broken_lengths_episodes(words, q, kv, requests, input_rows, pages):
        got, status = run_lengths(product_lengths(page_rows), arena, new_rows, w, a, b, page_rows)
        assert status == expected, name
        if expected == 4:
            assert np.array_equal(got, arena), name
        if ref is not None:
            _, their_status = run_lengths(reference_lengths(ref, page_rows), arena, new_rows, w, a, b, page_rows)
            assert their_status == expected, name
    # The domain the reference's prepare step qualifies.
    stream = torch.cuda.current_stream().cuda_stream
    d = torch.zeros(64, dtype=torch.int32, device="cuda")
    pointers = (d.data_ptr(),) * 5
    assert library.hyle_b200_paged_append_device_lengths(stream, *pointers, 8, 8, 8, 40, 32, 33, d.data_ptr()) == abi.NOT_SUPPORTED
    assert library.hyle_b200_paged_append_device_lengths(stream, *pointers, 8, 8, 8, 4, 32, 3, d.data_ptr()) == abi.NOT_SUPPORTED
    assert library.hyle_b200_paged_append_device_lengths(stream, *pointers, 8, 8, 8, 40, 33, 3, d.data_ptr()) == abi.INVALID_VALUE
    assert library.hyle_b200_paged_append_device_lengths(stream, *pointers, 8, 8, 8, 40, 32, 3, None) == abi.INVALID_VALUE

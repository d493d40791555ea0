"""The streaming logits kernel's ordered task list, decoded on the host (no GPU needed).

The kernel works through one list of (pass, row, chunk) tasks:
  P1(0) ... P1(w-1), P2(0), P1(w), P2(1), ..., P2(rows-w) ... P2(rows-1)      (each entry = all its chunks)
What the kernel relies on: the list is a permutation of every (pass, row, chunk); a row's second pass
comes after ALL chunks of its first pass, exactly `window * chunks` positions after the row's first
chunk while passes interleave; and the first `window * chunks` positions are first-pass tasks (that is
where the tasks a CTA takes by position must lie).
"""
import ctypes

import pytest

from hyle_b200 import abi


def decode(lib, rows, chunks, window, task):
    kind, row, chunk = ctypes.c_uint32(), ctypes.c_uint64(), ctypes.c_uint32()
    code = lib.hyle_b200_logits_stream_task(rows, chunks, window, task, ctypes.byref(kind), ctypes.byref(row), ctypes.byref(chunk))
    assert code == abi.OK
    return kind.value, row.value, chunk.value


@pytest.mark.parametrize("window", [8, 13, 32, 40, 64])
@pytest.mark.parametrize("chunks", [1, 2, 15, 30, 32])
def test_task_list_is_an_ordered_permutation(window, chunks):
    lib = abi.load()
    for rows in (window, window + 1, 2 * window + 3, 100):
        if rows < window:
            continue
        total = 2 * rows * chunks
        position = {}
        for task in range(total):
            kind, row, chunk = decode(lib, rows, chunks, window, task)
            assert kind in (0, 1) and row < rows and chunk < chunks
            assert (kind, row, chunk) not in position
            position[(kind, row, chunk)] = task
        assert len(position) == total
        assert decode(lib, rows, chunks, window, total)[0] == 2 and decode(lib, rows, chunks, window, total + 12345)[0] == 2
        for task in range(window * chunks):                   # the head is first-pass only
            assert decode(lib, rows, chunks, window, task)[0] == 0
        for row in range(rows):
            last_first = max(position[(0, row, c)] for c in range(chunks))
            first_second = min(position[(1, row, c)] for c in range(chunks))
            assert first_second > last_first                    # a second pass never precedes its first pass
            assert first_second - position[(0, row, 0)] >= window * chunks  # and lags it by the window at least
        for kind in (0, 1):                                   # rows ascend within a pass, chunks within a row
            order = sorted((task, row, chunk) for (k, row, chunk), task in position.items() if k == kind)
            assert [(row, chunk) for _, row, chunk in order] == [(r, c) for r in range(rows) for c in range(chunks)]


def test_task_decode_rejects_inconsistent_arguments():
    lib = abi.load()
    kind, row, chunk = ctypes.c_uint32(), ctypes.c_uint64(), ctypes.c_uint32()
    refs = (ctypes.byref(kind), ctypes.byref(row), ctypes.byref(chunk))
    assert lib.hyle_b200_logits_stream_task(8, 4, 9, 0, *refs) == abi.INVALID_VALUE   # window > rows
    assert lib.hyle_b200_logits_stream_task(8, 0, 4, 0, *refs) == abi.INVALID_VALUE
    assert lib.hyle_b200_logits_stream_task(8, 4, 4, 0, None, None, None) == abi.INVALID_VALUE

"""Cast / copy from strided views: the dense result must equal the oracle's cast of the same view
made dense on the host.  Bit-exact (NaN payloads as for the dense cast)."""
import ctypes

import numpy as np
import pytest
import torch

from hyle_b200 import abi, ops
from oracle import binding as ob


@pytest.fixture(scope="module")
def oracle():
    return ob.Oracle()


def views(base):
    """Named views of a 4-D base tensor [6, 10, 12, 16]."""
    return {
        "dense": base,
        "slice_inner": base[..., 3:11],
        "slice_outer_step": base[1::2, :, ::3],
        "transpose_last_two": base.transpose(-1, -2),
        "permute_all": base.permute(3, 1, 0, 2),
        "broadcast": base[:, :1, :, :].expand(6, 7, 12, 16),
        "scalar_broadcast": base[2, 3, 4, 5].expand(5, 9),
        "rank8": base.reshape(2, 3, 2, 5, 3, 4, 4, 4).permute(7, 0, 5, 2, 3, 1, 6, 4),
        "single": base[1, 2, 3, 4],
    }


@pytest.mark.gpu
@pytest.mark.parametrize("pair", [(abi.F32, abi.F32), (abi.F32, abi.BF16), (abi.BF16, abi.F32), (abi.F16, abi.BF16),
                                  (abi.F32, abi.E4M3), (abi.E4M3, abi.F16), (abi.E5M2, abi.E4M3), (abi.I32, abi.F32),
                                  (abi.F16, abi.BOOL), (abi.BOOL, abi.F32), (abi.BF16, abi.BF16), (abi.E4M3, abi.E4M3)])
def test_strided_cast_matches_dense_cast_of_the_same_view(oracle, pair):
    abi.load()
    source, destination = pair
    rng = np.random.default_rng(source * 10 + destination)
    shape = (6, 10, 12, 16)
    if source == abi.F32:
        host = (rng.standard_normal(shape) * 50).astype(np.float32)
    elif source == abi.I32:
        host = rng.integers(-2 ** 31, 2 ** 31 - 1, shape, dtype=np.int64).astype(np.int32)
    elif source in (abi.BF16, abi.F16):
        host = rng.integers(0, 1 << 16, shape, dtype=np.uint16)
    elif source == abi.BOOL:
        host = rng.integers(0, 3, shape).astype(np.uint8)
    else:
        host = rng.integers(0, 256, shape, dtype=np.uint8)
    carrier = {abi.F32: torch.float32, abi.I32: torch.int32, abi.BF16: torch.bfloat16, abi.F16: torch.float16}.get(source, torch.uint8)
    device = torch.from_numpy(host).cuda()
    device = device.view(carrier) if device.dtype != carrier else device
    for (name, d_view), h_view in zip(views(device).items(), views(torch.from_numpy(host)).values()):
        dense_host = np.ascontiguousarray(h_view.numpy())
        if source == destination:
            want = dense_host
        else:
            want = oracle.cast(source, destination, dense_host.view(ob.CAST_WORD[source]))
        got = ops.strided_cast_raw(d_view, source, destination)
        assert tuple(got.shape) == tuple(d_view.shape), name
        got_bits = got.cpu().contiguous().reshape(-1).view(torch.uint8).numpy()
        want_bits = np.ascontiguousarray(want).view(np.uint8).reshape(-1)
        if destination in (abi.F32, abi.BF16, abi.F16) and source != destination:
            # NaN payloads are not part of the contract: compare NaN-ness, and bits elsewhere
            kind, top, frac = {abi.F32: (np.uint32, 0x7f800000, 0x007fffff), abi.BF16: (np.uint16, 0x7f80, 0x007f),
                               abi.F16: (np.uint16, 0x7c00, 0x03ff)}[destination]
            g, w = got_bits.view(kind), want_bits.view(kind)
            nan_g = ((g & top) == top) & ((g & frac) != 0)
            nan_w = ((w & top) == top) & ((w & frac) != 0)
            assert np.array_equal(nan_g, nan_w), name
            assert np.array_equal(g[~nan_w], w[~nan_w]), name
        else:
            assert np.array_equal(got_bits, want_bits), name


@pytest.mark.gpu
@pytest.mark.parametrize("pair", [(abi.F32, abi.F32), (abi.F32, abi.BF16), (abi.F16, abi.F32), (abi.E4M3, abi.E4M3)])
def test_strided_cast_long_inner_runs(oracle, pair):
    """Views whose merged innermost axis has 256 elements or more take the run-based kernel."""
    source, destination = pair
    rng = np.random.default_rng(7 + source)
    shape = (4, 300, 9, 700)
    host = {abi.F32: lambda: rng.standard_normal(shape).astype(np.float32),
            abi.F16: lambda: rng.integers(0, 1 << 16, shape, dtype=np.uint16),
            abi.E4M3: lambda: rng.integers(0, 256, shape, dtype=np.uint8)}[source]()
    carrier = {abi.F32: torch.float32, abi.F16: torch.float16}.get(source, torch.uint8)
    device = torch.from_numpy(host).cuda()
    device = device.view(carrier) if device.dtype != carrier else device

    def long_views(t):
        return {
            "inner_slice": t[..., 10:590],
            "inner_slice_on_four_element_boundaries": t[..., 8:592],  # four elements per access
            "inner_slice_of_every_other_row": t[:, ::2, :, 16:528],
            "inner_step": t[1, :, 2, ::2],
            "inner_is_a_permuted_axis": t[:, :, :, 5].permute(0, 2, 1),
            "inner_broadcast": t[:, :1, :, :1].expand(4, 3, 9, 1000),
            "one_axis": t[2, 7, 3, 40:],
            "ragged_segments": t[0, :2, :, : 2048 // 3 + 1],
            # transposing views: the innermost axis is strided and another one is contiguous (tiled path)
            "transpose_with_batches": t.transpose(-1, -3),
            "transpose_2d": t[0, :, 3, :].t(),
            "transpose_ragged_tiles": t[1, :37, :, :45].permute(2, 1, 0),
            "transpose_of_a_slice": t[2, 5:200, 1, 3:500:2].t(),
        }

    for (name, d_view), h_view in zip(long_views(device).items(), long_views(torch.from_numpy(host)).values()):
        dense_host = np.ascontiguousarray(h_view.numpy())
        want = dense_host if source == destination else oracle.cast(source, destination, dense_host.view(ob.CAST_WORD[source]))
        got = ops.strided_cast_raw(d_view, source, destination)
        got_bits = got.cpu().contiguous().reshape(-1).view(torch.uint8).numpy()
        want_bits = np.ascontiguousarray(want).view(np.uint8).reshape(-1)
        if source == abi.F16 and destination == abi.F32:  # NaN payloads are not part of the contract
            g, w = got_bits.view(np.uint32), want_bits.view(np.uint32)
            nan = (w & 0x7fffffff) > 0x7f800000
            assert np.array_equal((g & 0x7fffffff) > 0x7f800000, nan), name
            assert np.array_equal(g[~nan], w[~nan]), name
        else:
            assert np.array_equal(got_bits, want_bits), name


@pytest.mark.gpu
def test_strided_cast_negative_strides_and_arguments():
    library = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.arange(24, dtype=torch.float32, device="cuda").reshape(4, 6)
    out = ops.new_output((4, 6), torch.float32)
    dims = (ctypes.c_int64 * 2)(4, 6)
    strides = (ctypes.c_int64 * 2)(-24, -4)  # both axes reversed, starting from the last element
    last = x.data_ptr() + 23 * 4
    assert library.hyle_b200_strided_cast(stream, abi.F32, abi.F32, last, out.data_ptr(), 2, dims, strides) == abi.OK
    torch.cuda.synchronize()
    assert torch.equal(out, x.flip(0, 1))
    odd = (ctypes.c_int64 * 2)(24, 2)
    assert library.hyle_b200_strided_cast(stream, abi.F32, abi.F32, x.data_ptr(), out.data_ptr(), 2, dims, odd) == abi.INVALID_VALUE
    assert library.hyle_b200_strided_cast(stream, abi.F32, abi.F32, x.data_ptr(), out.data_ptr(), 9, dims, strides) == abi.INVALID_VALUE
    assert library.hyle_b200_strided_cast(stream, abi.F32, abi.I32, x.data_ptr(), out.data_ptr(), 2, dims, strides) == abi.NOT_SUPPORTED
    empty = (ctypes.c_int64 * 2)(0, 6)
    assert library.hyle_b200_strided_cast(stream, abi.F32, abi.F32, None, None, 2, empty, strides) == abi.OK
    assert library.hyle_b200_strided_cast(stream, abi.F32, abi.BF16, x.data_ptr(), out.data_ptr(), 0, None, None) == abi.OK  # a scalar


# ---- the mirror: a dense result placed into a strided destination ---------------------------------------------


def scatter_destinations(base):
    """Views of a base tensor [6, 40, 12, 320] that do not overlap themselves."""
    return {
        "dense": base,
        "slice_inner": base[..., 16:272],            # contiguous runs of 256 elements: 16-byte groups when aligned
        "slice_inner_odd": base[..., 3:300],          # ragged, unaligned runs
        "slice_outer_step": base[1::2, :, ::3],
        "short_inner": base[..., 5:12],               # the element-wise kernel
        "transpose_last_two": base.transpose(-1, -2),     # dense in a permuted order: the tiled transposition
        "permute_all": base.permute(3, 1, 0, 2),
        "transposed_slice": base[..., 3:300].transpose(-1, -2),  # a transposition with gaps: element by element
        "inner_step": base[2, :, 3, ::2],
        "one_row": base[1, 2, 3, 8:],
        "single": base[1, 2, 3, 4],
        "rank8": base.reshape(2, 3, 5, 8, 3, 4, 16, 20).permute(7, 0, 5, 2, 3, 1, 6, 4),
    }


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8])
def test_strided_scatter_places_a_dense_tensor_into_a_view_and_touches_nothing_else(dtype):
    abi.load()
    rng = np.random.default_rng(91)
    shape = (6, 40, 12, 320)
    word = {torch.float32: np.uint32, torch.bfloat16: np.uint16, torch.uint8: np.uint8}[dtype]
    before = rng.integers(0, np.iinfo(word).max, shape, dtype=word, endpoint=True)
    for name in scatter_destinations(torch.from_numpy(before)):
        host = before.copy()
        h_view = scatter_destinations(torch.from_numpy(host))[name]
        payload = rng.integers(0, np.iinfo(word).max, tuple(h_view.shape), dtype=word, endpoint=True)
        h_view.copy_(torch.from_numpy(payload))  # what the destination's storage must look like afterwards
        storage = torch.from_numpy(before.copy()).cuda()
        storage = storage.view(dtype) if dtype != torch.uint8 else storage
        d_view = scatter_destinations(storage)[name]
        dense = torch.from_numpy(payload).cuda()
        dense = dense.view(dtype) if dtype != torch.uint8 else dense
        returned = ops.strided_scatter(dense.reshape(d_view.shape), d_view)
        assert returned.data_ptr() == d_view.data_ptr()
        got = storage.cpu().view(torch.uint8).numpy().reshape(-1)
        assert np.array_equal(got, host.view(np.uint8).reshape(-1)), name


@pytest.mark.gpu
def test_strided_scatter_then_strided_cast_is_the_identity_and_arguments_are_checked():
    library = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.arange(24, dtype=torch.float32, device="cuda").reshape(4, 6)
    storage = torch.full((8, 12), -1.0, dtype=torch.float32, device="cuda")
    view = storage[1:8:2, 1:12:2]
    ops.strided_scatter(x, view)
    assert torch.equal(ops.strided_cast(view), x)
    assert torch.equal(storage[::2], torch.full((4, 12), -1.0, device="cuda"))
    dims = (ctypes.c_int64 * 2)(4, 6)
    # both axes reversed, starting from the last element of a dense [4, 6] destination
    out = torch.zeros(4, 6, dtype=torch.float32, device="cuda")
    reverse = (ctypes.c_int64 * 2)(-24, -4)
    assert library.hyle_b200_strided_scatter(stream, abi.F32, x.data_ptr(), out.data_ptr() + 23 * 4, 2, dims, reverse) == abi.OK
    torch.cuda.synchronize()
    assert torch.equal(out, x.flip(0, 1))
    broadcast = (ctypes.c_int64 * 2)(0, 4)  # four rows at one address: not a destination
    assert library.hyle_b200_strided_scatter(stream, abi.F32, x.data_ptr(), out.data_ptr(), 2, dims, broadcast) == abi.INVALID_VALUE
    odd = (ctypes.c_int64 * 2)(24, 2)
    assert library.hyle_b200_strided_scatter(stream, abi.F32, x.data_ptr(), out.data_ptr(), 2, dims, odd) == abi.INVALID_VALUE
    assert library.hyle_b200_strided_scatter(stream, abi.F32, x.data_ptr(), out.data_ptr(), 9, dims, reverse) == abi.INVALID_VALUE
    assert library.hyle_b200_strided_scatter(stream, 99, x.data_ptr(), out.data_ptr(), 2, dims, reverse) == abi.NOT_SUPPORTED
    empty = (ctypes.c_int64 * 2)(0, 6)
    assert library.hyle_b200_strided_scatter(stream, abi.F32, None, None, 2, empty, reverse) == abi.OK
    assert library.hyle_b200_strided_scatter(stream, abi.F32, x.data_ptr(), out.data_ptr(), 0, None, None) == abi.OK  # a scalar

"""Scan{axis=-1}: the oracle against numpy on CPU, the CUDA kernel against the oracle on the GPU.
i32 is exact.  f32: the operator permits reassociation, so sums of values that are exact in any order
(small integers) must match bit for bit and random rows within 1e-5 of the prefix sum of |x|."""
import numpy as np
import pytest
import torch

from hyle_b200 import abi, ops
from oracle import binding as ob


@pytest.fixture(scope="module")
def oracle():
    return ob.Oracle()


def shifted(inclusive):
    out = np.zeros_like(inclusive)
    out[..., 1:] = inclusive[..., :-1]
    return out


def test_oracle_scan_against_numpy(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((7, 1000)).astype(np.float32)
    want = np.cumsum(x, axis=-1, dtype=np.float32)  # numpy accumulates left to right in float32 as well
    got, _ = oracle.scan(x)
    assert np.array_equal(got, want)
    got, _ = oracle.scan(x, exclusive=True)
    assert np.array_equal(got, shifted(want))
    n = rng.integers(-1000, 1000, (5, 333)).astype(np.int32)
    got, status = oracle.scan(n)
    assert status == 0 and np.array_equal(got, np.cumsum(n, axis=-1))
    got, status = oracle.scan(n, exclusive=True)
    assert status == 0 and np.array_equal(got, shifted(np.cumsum(n, axis=-1)).astype(np.int32))


def test_oracle_scan_i32_overflow_writes_nothing(oracle):
    n = np.ones((3, 8), np.int32)
    n[1, 2] = 2 ** 31 - 3  # the prefix passes INT32_MAX at column 3 and never comes back
    got, status = oracle.scan(n)
    assert status == 16 and not got.any()
    n[1, 4] = -(2 ** 31 - 3)  # the row total fits again, an intermediate prefix does not
    got, status = oracle.scan(n, exclusive=True)
    assert status == 16 and not got.any()
    n[1, 3] = 0  # the prefix now stops at 2**31 - 1 exactly: still int32
    got, status = oracle.scan(n)
    assert status == 0 and got[1, 3] == 2 ** 31 - 1


SHAPES = [(1, 1), (3, 7), (5, 1000), (16, 151936), (1, 1 << 20), (2000, 130), (1500, 4096), (300, 4100), (9, 40000)]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("exclusive", [False, True])
def test_scan_f32(oracle, rows, cols, exclusive):
    abi.load()
    rng = np.random.default_rng(rows + cols)
    whole = rng.integers(-8, 9, (rows, cols)).astype(np.float32)  # every partial sum is exact (< 2^24)
    want, _ = oracle.scan(whole, exclusive)
    got = ops.scan(torch.from_numpy(whole).cuda(), exclusive).cpu().numpy()
    assert np.array_equal(got, want)
    x = (rng.standard_normal((rows, cols)) * np.exp(rng.uniform(-3, 3, (rows, 1)))).astype(np.float32)
    exact = np.cumsum(x.astype(np.float64), axis=-1)
    bound = 1e-5 * np.cumsum(np.abs(x).astype(np.float64), axis=-1) + 1e-30
    if exclusive:
        exact, bound = shifted(exact), shifted(bound) + 1e-30
    got = ops.scan(torch.from_numpy(x).cuda(), exclusive).cpu().numpy().astype(np.float64)
    assert np.all(np.abs(got - exact) <= bound)


@pytest.mark.gpu
def test_scan_f32_specials_propagate_from_their_column():
    x = np.ones((4, 5000), np.float32)
    x[0, 1234] = np.inf
    x[1, 77] = np.nan
    x[2, 10], x[2, 4000] = np.inf, -np.inf
    got = ops.scan(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got[0, :1234], np.arange(1, 1235, dtype=np.float32)) and np.all(np.isposinf(got[0, 1234:]))
    assert np.array_equal(got[1, :77], np.arange(1, 78, dtype=np.float32)) and np.all(np.isnan(got[1, 77:]))
    assert np.all(np.isposinf(got[2, 10:4000])) and np.all(np.isnan(got[2, 4000:]))
    assert np.array_equal(got[3], np.arange(1, 5001, dtype=np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("exclusive", [False, True])
def test_scan_i32(oracle, rows, cols, exclusive):
    rng = np.random.default_rng(rows * 3 + cols)
    n = rng.integers(-2000, 2001, (rows, cols)).astype(np.int32)
    n[0, 0] = 2 ** 31 - 1 - int(np.cumsum(n[0].astype(np.int64)).max() - n[0, 0])  # row 0 touches INT32_MAX exactly
    want, want_status = oracle.scan(n, exclusive)
    assert want_status == 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.scan(torch.from_numpy(n).cuda(), exclusive, status).cpu().numpy()
    assert int(status.item()) == 0 and np.array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(37, 4100), (1300, 1024), (1250, 130)])
def test_scan_i32_rows_whose_magnitudes_exceed_int32_but_whose_prefixes_fit(oracle, rows, cols):
    """The deciding pass first sums magnitudes; rows that fail that cheap test are checked exactly.  Swinging
    rows (prefixes between INT32_MIN and INT32_MAX although the magnitudes sum far above) must be scanned, and
    the scan's wrap-around arithmetic must give the true values, including both extremes."""
    rng = np.random.default_rng(9)
    n = rng.integers(-3, 4, (rows, cols)).astype(np.int64)
    n[:, 10::50] = 2 ** 30
    n[:, 35::50] = -(2 ** 30)
    n[5, :] = 0
    n[5, 0], n[5, 1], n[5, 2], n[5, 3] = 2 ** 31 - 1, -(2 ** 31 - 1), -(2 ** 31), 2 ** 31 - 1   # touches both ends of the range
    n = n.astype(np.int32)
    for exclusive in (False, True):
        want, want_status = oracle.scan(n, exclusive)
        assert want_status == 0
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = ops.scan(torch.from_numpy(n).cuda(), exclusive, status).cpu().numpy()
        assert int(status.item()) == 0 and np.array_equal(got, want)
    # one step further and the same row overflows: caught by the exact check, nothing written
    n[5, 1] = 1   # 2^31 - 1, then + 1
    _, want_status = oracle.scan(n)
    assert want_status == 16
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.new_output(n.shape, torch.int32).fill_(-7)
    assert abi.load().hyle_b200_scan(torch.cuda.current_stream().cuda_stream, abi.I32, torch.from_numpy(n).cuda().data_ptr(),
                                     out.data_ptr(), rows, cols, 0, status.data_ptr()) == abi.OK
    torch.cuda.synchronize()
    assert int(status.item()) == abi.STATUS_SCAN_OVERFLOW and bool((out == -7).all())


@pytest.mark.gpu
def test_scan_i32_overflow_reports_and_writes_nothing(oracle):
    library = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    for rows, cols, where in [(300, 4100, (299, 4000)), (2000, 130, (0, 1)), (4, 50000, (2, 49999))]:
        n = np.ones((rows, cols), np.int32)
        n[where] = 2 ** 31 - 1  # with the ones around it the prefix passes INT32_MAX
        if where[1] + 1 < cols:
            n[where[0], where[1] + 1] = -(2 ** 31 - 1)  # and the row total fits again
        _, want_status = oracle.scan(n)
        assert want_status == 16
        d_in = torch.from_numpy(n).cuda()
        d_out = ops.new_output(d_in.shape, d_in.dtype).fill_(-7)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert library.hyle_b200_scan(stream, abi.I32, d_in.data_ptr(), d_out.data_ptr(), rows, cols, 0, status.data_ptr()) == abi.OK
        torch.cuda.synchronize()
        assert int(status.item()) == abi.STATUS_SCAN_OVERFLOW
        assert bool((d_out == -7).all())
    d = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert library.hyle_b200_scan(stream, abi.I32, d.data_ptr(), d[32:].data_ptr(), 1, 32, 0, None) == abi.INVALID_VALUE
    assert library.hyle_b200_scan(stream, abi.F32, d.data_ptr(), d.data_ptr(), 1, 32, 0, None) == abi.INVALID_VALUE
    assert library.hyle_b200_scan(stream, abi.BF16, d.data_ptr(), d[32:].data_ptr(), 1, 32, 0, None) == abi.NOT_SUPPORTED
    assert library.hyle_b200_scan(stream, abi.F32, None, None, 0, 32, 0, None) == abi.OK

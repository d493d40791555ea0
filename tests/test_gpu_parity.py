"""Parity of the sm_100a kernels with the CPU checker, through the C ABI, on the same seeded inputs.

Bars (from the workload definition): Q8_0 bytes and argmax indices bit-exact; f32 elementwise
bit-exact; f32 reductions within 1e-5 (row sums relative to the sum of magnitudes); bf16
elementwise within 1 bf16 ulp; bf16 RMSNorm and softmax within 2e-3 relative of the checker's
unrounded value (and never more than 1 bf16 ulp from its rounded one).
"""
import numpy as np
import pytest
import torch

from hyle_b200 import abi, ops
from hyle_b200 import workloads as wl
from oracle import binding as ob

pytestmark = pytest.mark.gpu

DEV = "cuda"
F32_REL = 1e-5          # fp32 outputs
BF16_REL = 2e-3         # bf16 RMSNorm / softmax against the unrounded checker value
TINY = 1e-37            # absolute slack for subnormal results


# ---- helpers ------------------------------------------------------------------------------------------------
def to_dev_bf16(words: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(words.view(np.int16)).to(DEV).view(torch.bfloat16)


def bf16_words(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def to_dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a).to(DEV)


def u32(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_f32_bits(got, want):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(u32(got)[ok], u32(want)[ok])


def bf16_ulp_distance(a_words, b_words):
    """Distance in bf16 steps on the ordered integer line (handles sign); NaN must match NaN.

    Where both values are below 2^-120 in magnitude (the exponent range in which f32 exponentials
    underflow gradually on the CPU and flush on the GPU's special-function unit) the distance
    counts as 0 when the absolute difference is under 1e-37.
    """
    def ordered(w):
        w = w.astype(np.int32)
        return np.where(w & 0x8000, -(w & 0x7FFF), w & 0x7FFF)
    a_nan, b_nan = (a_words & 0x7FFF) > 0x7F80, (b_words & 0x7FFF) > 0x7F80
    assert np.array_equal(a_nan, b_nan)
    dist = np.abs(ordered(a_words) - ordered(b_words))
    a, b = wl.bf16_to_f32(a_words).astype(np.float64), wl.bf16_to_f32(b_words).astype(np.float64)
    with np.errstate(invalid="ignore"):
        tiny = (np.abs(a) < 2.0 ** -120) & (np.abs(b) < 2.0 ** -120) & (np.abs(a - b) <= TINY)
    dist = np.where(tiny, 0, dist)
    return dist[~a_nan]


def assert_bf16_close(got_words, want_words, want_f32, rel):
    """bf16 outputs of a reduction-based operator against the checker's bf16 outputs.

    A bf16 step is 2^-7 relative, coarser than the 2e-3 bar, so the bar cannot hold per element
    against an unrounded value (a correctly rounded bf16 is up to 3.9e-3 away from it).  Per
    element the result may differ from the checker's ROUNDED output by at most one bf16 step (a
    rounding that tipped the other way because the f32 value differed in its last bits); the 2e-3
    bound is on the relative L2 distance between each row and the checker's row.  `want_f32` (the
    checker's value before rounding) guards the checker itself: its rounding must be the nearest.
    Returns the fraction of elements that are not bit-identical to the checker's.
    """
    dist = bf16_ulp_distance(got_words, want_words)
    assert dist.max(initial=0) <= 1, f"max bf16 ulp distance {dist.max()}"
    cols = want_words.shape[-1]
    got = wl.bf16_to_f32(got_words).reshape(-1, cols).astype(np.float64)
    want = wl.bf16_to_f32(want_words).reshape(-1, cols).astype(np.float64)
    for g_row, w_row in zip(got, want):
        ok = np.isfinite(w_row)
        if ok.any():
            assert np.sqrt(np.sum((g_row[ok] - w_row[ok]) ** 2)) <= rel * np.sqrt(np.sum(w_row[ok] ** 2)) + TINY
    unrounded = np.asarray(want_f32, np.float64).reshape(-1, cols)
    ok = np.isfinite(unrounded)
    assert np.all(np.abs(want[ok] - unrounded[ok]) <= 2.0 ** -8 * np.abs(unrounded[ok]) + TINY)
    return float((dist != 0).mean()) if dist.size else 0.0


@pytest.fixture(scope="module")
def oracle():
    return ob.Oracle()


# ---- workload 1: broadcast add + row reductions (f32) ---------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(4096, 4096), (37, 4096), (5, 1024), (3, 2048), (9, 8192), (7, 1000), (4, 1003), (3, 1)])
def test_add_bias_row_sum_max(oracle, rows, cols):
    a, bias = wl.broadcast_add_inputs(rows, cols)
    c, row_sum, row_max = ops.add_bias_row_sum_max(to_dev(a), to_dev(bias))
    want_c = oracle.binary(ob.ADD, ob.F32, a, bias)
    assert_f32_bits(c.cpu().numpy(), want_c)                                   # one IEEE add: bit-exact
    assert_f32_bits(row_max.cpu().numpy(), oracle.reduce_rows(ob.MAXIMUM, want_c))  # exact
    s64, abs64 = oracle.row_sum_f64(want_c)
    assert np.all(np.abs(row_sum.cpu().numpy().astype(np.float64) - s64) <= F32_REL * abs64)
    # fused == separate launches, bit for bit
    c2 = ops.add(to_dev(a), to_dev(bias))
    assert torch.equal(c2, c)
    assert torch.equal(ops.reduce_rows(abi.REDUCE_SUM, c2), row_sum)
    assert torch.equal(ops.reduce_rows(abi.REDUCE_MAXIMUM, c2), row_max)


def test_binary_variants_and_broadcast_periods(oracle):
    rng = np.random.default_rng(3)
    for count, period in [(4096 * 8, 4096), (1024, 1024), (96, 32), (1000, 8), (77, 7), (35, 1), (12, 12)]:
        lhs = rng.standard_normal(count).astype(np.float32)
        rhs = rng.standard_normal(period).astype(np.float32)
        for kind, okind in [(abi.BINARY_ADD, ob.ADD), (abi.BINARY_MULTIPLY, ob.MULTIPLY)]:
            out = ops.new_output(count, torch.float32, DEV)
            lhs_dev, rhs_dev = to_dev(lhs), to_dev(rhs)
            abi.check("binary", abi.load().hyle_b200_binary(
                torch.cuda.current_stream().cuda_stream, kind, abi.F32, lhs_dev.data_ptr(),
                rhs_dev.data_ptr(), out.data_ptr(), count, period))
            want = oracle.binary(okind, ob.F32, lhs.reshape(-1, period), rhs).ravel()
            assert_f32_bits(out.cpu().numpy(), want)
    # bf16 and f16: f32 operation, one rounding (bit-exact against the checker)
    x16, r16, _, _ = wl.rms_norm_inputs(33)
    got = ops.add(to_dev_bf16(x16), to_dev_bf16(r16))
    assert np.array_equal(bf16_words(got), oracle.binary(ob.ADD, ob.BF16, x16, r16))
    got = ops.multiply(to_dev_bf16(x16), to_dev_bf16(r16[0]))
    assert np.array_equal(bf16_words(got), oracle.binary(ob.MULTIPLY, ob.BF16, x16, r16[0]))
    h = rng.standard_normal((5, 264)).astype(np.float16)
    g = rng.standard_normal((5, 264)).astype(np.float16)
    got = ops.add(to_dev(h), to_dev(g)).cpu().numpy()
    want = oracle.binary(ob.ADD, ob.F16, h.view(np.uint16), g.view(np.uint16))
    assert np.array_equal(got.view(np.uint16), want)
    # subtract, divide, number minimum / maximum: bit-exact in all three storage types, including
    # NaN operands, infinities, subnormals and zeros of either sign in either order
    special = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1.0, -1.0, 3.0e38, 1e-40, -1e-40], np.float32)
    a32 = np.concatenate([np.repeat(special, special.size), rng.standard_normal(4000).astype(np.float32)])
    b32 = np.concatenate([np.tile(special, special.size), rng.standard_normal(4000).astype(np.float32)])
    kinds = [(abi.BINARY_SUBTRACT, ob.SUBTRACT), (abi.BINARY_DIVIDE, ob.DIVIDE),
             (abi.BINARY_MINIMUM, ob.NUMBER_MINIMUM), (abi.BINARY_MAXIMUM, ob.NUMBER_MAXIMUM)]
    for kind, okind in kinds:
        want = oracle.binary(okind, ob.F32, a32, b32)
        got = ops.binary(kind, to_dev(a32), to_dev(b32)).cpu().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
        a16, b16 = wl.f32_to_bf16(a32), wl.f32_to_bf16(b32)
        want16 = oracle.binary(okind, ob.BF16, a16, b16)
        got16 = bf16_words(ops.binary(kind, to_dev_bf16(a16), to_dev_bf16(b16)))
        nan16 = (want16 & 0x7FFF) > 0x7F80
        assert np.array_equal((got16 & 0x7FFF) > 0x7F80, nan16)
        assert np.array_equal(got16[~nan16], want16[~nan16])
        with np.errstate(all="ignore"):
            ah, bh = a32.astype(np.float16), b32.astype(np.float16)
        wanth = oracle.binary(okind, ob.F16, ah.view(np.uint16), bh.view(np.uint16))
        goth = ops.binary(kind, to_dev(ah), to_dev(bh)).cpu().numpy().view(np.uint16)
        nanh = (wanth & 0x7FFF) > 0x7C00
        assert np.array_equal((goth & 0x7FFF) > 0x7C00, nanh)
        assert np.array_equal(goth[~nanh], wanth[~nanh])
        # broadcast of the right operand
        rowvec = b32[:40]
        want = oracle.binary(okind, ob.F32, a32[:4000].reshape(100, 40), rowvec)
        got = ops.binary(kind, to_dev(a32[:4000].reshape(100, 40)), to_dev(rowvec)).cpu().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
    # in place
    t = to_dev(lhs.copy())
    ops.add(t, t.clone(), out=t)
    assert_f32_bits(t.cpu().numpy(), lhs + lhs)


def test_reduce_rules_nan_signed_zero_empty(oracle):
    x = np.zeros((8, 1500), np.float32)
    rng = np.random.default_rng(4)
    x[:] = rng.standard_normal(x.shape)
    x[0, 1499] = np.nan          # NaN in the last lane of the tail
    x[1, 31] = np.nan            # at a warp boundary
    x[2] = -0.0; x[2, 700] = 0.0
    x[3] = -0.0
    x[4, 5] = np.inf; x[5, 9] = -np.inf
    x[6] = -np.inf
    for kind, okind in [(abi.REDUCE_MAXIMUM, ob.MAXIMUM), (abi.REDUCE_MINIMUM, ob.MINIMUM)]:
        got = ops.reduce_rows(kind, to_dev(x)).cpu().numpy()
        assert_f32_bits(got, oracle.reduce_rows(okind, x))
    mean = ops.reduce_rows(abi.REDUCE_MEAN, to_dev(x[7:8])).cpu().numpy()
    s64, abs64 = oracle.row_sum_f64(x[7:8])
    assert abs(float(mean[0]) - s64[0] / 1500) <= F32_REL * abs64[0] / 1500
    empty = torch.zeros((3, 0), dtype=torch.float32, device=DEV)
    assert torch.equal(ops.reduce_rows(abi.REDUCE_SUM, empty).cpu(), torch.zeros(3))
    assert torch.isnan(ops.reduce_rows(abi.REDUCE_MEAN, empty)).all()
    assert (ops.reduce_rows(abi.REDUCE_MINIMUM, empty) == float("inf")).all()
    assert (ops.reduce_rows(abi.REDUCE_MAXIMUM, empty) == float("-inf")).all()


# ---- workload 2: residual add + RMSNorm (bf16) ------------------------------------------------------------------
@pytest.mark.parametrize("tokens", [1, 64, 4096])
@pytest.mark.parametrize("weight_kind", ["bf16", "f32"])
def test_add_rms_norm_config(oracle, tokens, weight_kind):
    x, r, w16, w32 = wl.rms_norm_inputs(tokens)
    w = w16 if weight_kind == "bf16" else w32
    w_dev = to_dev_bf16(w16) if weight_kind == "bf16" else to_dev(w32)
    y, h = ops.add_rms_norm(to_dev_bf16(x), to_dev_bf16(r), w_dev, 1e-6)
    want_y, want_y32, want_h = oracle.add_rms_norm(x, r, w, 1e-6)
    assert np.array_equal(bf16_words(h), want_h)          # f32 add + one RNE: bit-exact
    assert_bf16_close(bf16_words(y), want_y, want_y32, BF16_REL)
    # fused == unfused composition, bit for bit
    y2 = ops.rms_norm(ops.add(to_dev_bf16(x), to_dev_bf16(r)), w_dev, 1e-6)
    assert torch.equal(y2.view(torch.int16), y.view(torch.int16))


@pytest.mark.parametrize("hidden", [1, 8, 127, 128, 129, 256, 257, 512, 1024, 2048, 4096, 5120, 8192])
def test_rms_norm_hidden_sizes(oracle, hidden):
    rng = np.random.default_rng(hidden)
    x = wl.f32_to_bf16(rng.standard_normal((5, hidden)).astype(np.float32))
    r = wl.f32_to_bf16(rng.standard_normal((5, hidden)).astype(np.float32))
    w32 = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    for w, w_dev in [(None, None), (wl.f32_to_bf16(w32), to_dev_bf16(wl.f32_to_bf16(w32))), (w32, to_dev(w32))]:
        y = ops.rms_norm(to_dev_bf16(x), w_dev, 1e-6)
        want_y, want_y32 = oracle.rms_norm(x, w, 1e-6)
        assert_bf16_close(bf16_words(y), want_y, want_y32, BF16_REL)
        y, h = ops.add_rms_norm(to_dev_bf16(x), to_dev_bf16(r), w_dev, 1e-6)
        want_y, want_y32, want_h = oracle.add_rms_norm(x, r, w, 1e-6)
        assert np.array_equal(bf16_words(h), want_h)
        assert_bf16_close(bf16_words(y), want_y, want_y32, BF16_REL)
    # y may alias x
    t = to_dev_bf16(x)
    ops.rms_norm(t, None, 1e-6, out=t)
    assert_bf16_close(bf16_words(t), *oracle.rms_norm(x, None, 1e-6), BF16_REL)
    assert ops.rms_norm(torch.empty((0, hidden), dtype=torch.bfloat16, device=DEV), None, 1e-6).numel() == 0


@pytest.mark.parametrize("hidden", [1, 8, 127, 1000, 1024, 2048, 2056, 4096, 5000, 16384])
def test_rms_norm_f16_and_f32_rows(oracle, hidden):
    """RmsNorm on the other two storages of the CPU route: f16 rows within one f16 step of the checker (the sums
    differ in order), f32 rows within 4e-6 relative; the weight of the row's type or f32; y may be x."""
    rng = np.random.default_rng(7 * hidden + 1)
    rows = 19
    x32 = rng.standard_normal((rows, hidden)).astype(np.float32)
    w32 = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    x16, w16 = x32.astype(np.float16), w32.astype(np.float16)
    for weight, code in ((None, abi.F16), (w16, abi.F16), (w32, abi.F32)):
        want, _ = oracle.rms_norm_stored(abi.F16, x16.view(np.uint16), None if weight is None else
                                         (weight if code == abi.F32 else weight.view(np.uint16)), code, 1e-6)
        got = ops.rms_norm(to_dev(x16), None if weight is None else to_dev(weight), 1e-6)
        distance = np.abs(ordered16(got.cpu().numpy().view(np.uint16)) - ordered16(want))
        assert distance.max() <= 1 and (distance != 0).mean() < 2e-2
    for weight in (None, w32):
        want, _ = oracle.rms_norm_stored(abi.F32, x32, weight, abi.F32, 1e-6)
        got = ops.rms_norm(to_dev(x32), None if weight is None else to_dev(weight), 1e-6).cpu().numpy()
        assert np.allclose(got, want, rtol=4e-6, atol=0)
    t = to_dev(x32)
    ops.rms_norm(t, to_dev(w32), 1e-6, out=t)
    assert np.allclose(t.cpu().numpy(), want, rtol=4e-6, atol=0)
    odd = to_dev(np.concatenate([np.zeros(1, np.float16), x16.reshape(-1)]))[1:].view(rows, hidden)   # 2-byte aligned only
    want, _ = oracle.rms_norm_stored(abi.F16, x16.view(np.uint16), None, abi.F16, 1e-6)
    assert np.abs(ordered16(ops.rms_norm(odd, None, 1e-6).cpu().numpy().view(np.uint16)) - ordered16(want)).max() <= 1
    with pytest.raises(abi.KernelError):
        ops.rms_norm(torch.zeros((2, 16392), device=DEV), None, 1e-6)      # an f32 row beyond 64 KB


@pytest.mark.parametrize("shape", [(1, 1), (7, 13), (300, 1000), (1500, 1024), (5, 16384), (3, 40000), (2000, 136)])
@pytest.mark.parametrize("dtype", [abi.BF16, abi.F16])
def test_narrow_rows_minimum_and_maximum(oracle, shape, dtype):
    """Reduce{kMinimum | kMaximum} of bf16 / f16 rows in their own type: exact, NaN wins, -0 < +0."""
    rng = np.random.default_rng(shape[0] * 31 + shape[1] + dtype)
    values = (50.0 * rng.standard_normal(shape)).astype(np.float32)
    words = oracle.cast(abi.F32, dtype, values)
    if shape[1] > 4:
        words[0, :] = 0x8000; words[0, 3] = 0x0000                        # -0 everywhere, one +0
        if shape[0] > 2:
            words[1, shape[1] // 2] = 0x7E00 if dtype == abi.F16 else 0x7FC0      # a NaN
            words[2, 1] = 0xFC00 if dtype == abi.F16 else 0xFF80                  # -inf
    torch_type = torch.float16 if dtype == abi.F16 else torch.bfloat16
    x = torch.from_numpy(words.view(np.int16)).to(DEV).view(torch_type)
    for kind in (abi.REDUCE_MINIMUM, abi.REDUCE_MAXIMUM):
        want = oracle.reduce_rows_narrow(kind, dtype, words)
        got = ops.reduce_rows(kind, x).view(torch.int16).cpu().numpy().view(np.uint16)
        nan = (want & 0x7FFF) > (0x7C00 if dtype == abi.F16 else 0x7F80)
        assert np.array_equal((got & 0x7FFF) > (0x7C00 if dtype == abi.F16 else 0x7F80), nan)
        assert np.array_equal(got[~nan], want[~nan])
    odd = torch.cat([x.reshape(-1)[:1], x.reshape(-1)])[1:].view(shape)        # 2-byte aligned rows
    assert torch.equal(ops.reduce_rows(abi.REDUCE_MAXIMUM, odd).view(torch.int16), ops.reduce_rows(abi.REDUCE_MAXIMUM, x).view(torch.int16))
    empty = ops.reduce_rows(abi.REDUCE_MINIMUM, torch.empty((3, 0), dtype=torch_type, device=DEV))
    assert torch.isinf(empty.float()).all() and (empty.float() > 0).all()


# ---- workload 3: SwiGLU (bf16) ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("tokens", [1, 8, 32, 4096])
def test_swiglu_config(oracle, tokens):
    gate, up = wl.swiglu_inputs(tokens)
    out = ops.swiglu(to_dev_bf16(gate), to_dev_bf16(up))
    want, want32 = oracle.swiglu(gate, up)
    dist = bf16_ulp_distance(bf16_words(out), want)
    assert dist.max() <= 1                                   # <= 1 bf16 ulp
    assert (dist != 0).mean() < 1e-3                         # and nearly always identical


def test_swiglu_specials_packed_and_odd_shapes(oracle, ):
    specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 80.0, -80.0, 1e-30, -1e-30, 88.7, -88.7, 100.0,
                         -100.0, 1.0, -1.0, 20.0, -20.0, 3e38, -3e38], np.float32)
    rng = np.random.default_rng(9)
    for rows, cols in [(3, 264), (2, 257), (5, 6144), (1, 8)]:
        gate = (1.5 * rng.standard_normal((rows, cols))).astype(np.float32)
        up = (1.5 * rng.standard_normal((rows, cols))).astype(np.float32)
        n = min(specials.size, cols)
        gate[0, :n] = specials[:n]
        up[-1, :n] = specials[:n][::-1]
        g16, u16 = wl.f32_to_bf16(gate), wl.f32_to_bf16(up)
        want, _ = oracle.swiglu(g16, u16)
        out = ops.swiglu(to_dev_bf16(g16), to_dev_bf16(u16))
        assert bf16_ulp_distance(bf16_words(out), want).max() <= 1
        packed = np.concatenate([g16, u16], axis=1)
        out_p = ops.swiglu_packed(to_dev_bf16(packed))
        assert np.array_equal(bf16_words(out_p), bf16_words(out))
    # silu(-inf) * finite = 0, not NaN
    g = wl.f32_to_bf16(np.full((1, 8), -np.inf, np.float32))
    u = wl.f32_to_bf16(np.full((1, 8), 2.0, np.float32))
    assert np.all(wl.bf16_to_f32(bf16_words(ops.swiglu(to_dev_bf16(g), to_dev_bf16(u)))) == 0.0)


# ---- workload 4: logits -> lse, softmax bf16, argmax ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("activation", [abi.GATE_SILU, abi.GATE_GELU, abi.GATE_GELU_TANH])
def test_gated_activation_kinds_and_storage_types(oracle, activation, dtype):
    """GatedActivation{kSilu|kGelu|kGeluTanh} on bf16 and f16: one storage step from the checker; with the
    activated gate rounded first, bit-identical to this library's Unary kernel followed by its Multiply."""
    rng = np.random.default_rng(activation * 2 + (dtype == "f16"))
    torch_dtype = torch.bfloat16 if dtype == "bf16" else torch.float16
    code = ob.BF16 if dtype == "bf16" else ob.F16
    for rows, cols in [(33, 6144), (5, 1000), (3, 7)]:
        g32 = (1.5 * rng.standard_normal((rows, cols))).astype(np.float32)
        u32 = (1.5 * rng.standard_normal((rows, cols))).astype(np.float32)
        g32[0, :4] = [-np.inf, np.inf, np.nan, -0.0]
        gate = torch.from_numpy(g32).to(DEV).to(torch_dtype)
        up = torch.from_numpy(u32).to(DEV).to(torch_dtype)
        gate_words = gate.view(torch.int16).cpu().numpy().view(np.uint16)
        up_words = up.view(torch.int16).cpu().numpy().view(np.uint16)
        to_f64 = (lambda w: wl.bf16_to_f32(w).astype(np.float64)) if dtype == "bf16" else (lambda w: w.view(np.float16).astype(np.float64))
        relative_step = 2.0 ** -8 if dtype == "bf16" else 2.0 ** -11       # half a storage step, relative
        gate64, up64 = to_f64(gate_words), to_f64(up_words)
        for round_gate in (False, True):
            got = ops.gated_activation(gate, up, activation, round_gate).view(torch.int16).cpu().numpy().view(np.uint16)
            want, _ = oracle.gated_activation(activation, code, gate_words, up_words, round_gate)
            a, b = to_f64(got), to_f64(want)
            assert np.array_equal(np.isnan(a), np.isnan(b))
            infinite = np.isinf(b)
            assert np.array_equal(a[infinite], b[infinite])
            ok = ~np.isnan(b) & ~infinite
            # one storage step (two with the extra rounding of the gate), plus what the erf / tanh forms lose to
            # cancellation for negative gates: 2.5e-7 |gate| absolute in the activation, times |up|
            steps = 2 if round_gate else 1
            with np.errstate(invalid="ignore"):
                product = np.nan_to_num(np.abs(gate64[ok] * up64[ok]), nan=0.0, posinf=1e30)
            slack = steps * 2 * relative_step * np.abs(b[ok]) + 2.5e-7 * product * (1 + steps) + 1e-30
            if dtype == "f16":
                slack = slack + steps * 2.0 ** -24                                # subnormal f16 results
            assert np.all(np.abs(a[ok] - b[ok]) <= slack)
        unary_kind = {abi.GATE_SILU: abi.UNARY_SILU, abi.GATE_GELU: abi.UNARY_GELU, abi.GATE_GELU_TANH: abi.UNARY_GELU_TANH}[activation]
        two_steps = ops.multiply(ops.unary(unary_kind, gate), up)
        fused = ops.gated_activation(gate, up, activation, True)
        a, b = two_steps.view(torch.int16), fused.view(torch.int16)
        nan = torch.isnan(two_steps.float())
        assert torch.equal(nan, torch.isnan(fused.float())) and torch.equal(a[~nan], b[~nan])
    with pytest.raises(abi.KernelError):
        abi.check("gate", abi.load().hyle_b200_gated_activation(0, 3, abi.BF16, 0, 1 << 20, 1 << 20, 1 << 20, 1, 8, 8, 8))


def check_logits(oracle, logits, workspace=None):
    lse, probs, index, value = ops.logits_reduce(to_dev(logits), workspace=workspace)
    want_lse, want_p, want_p32, want_i, want_v = oracle.logits_reduce(logits)
    assert np.array_equal(index.cpu().numpy(), want_i)                  # bit-exact, lowest index on ties
    assert_f32_bits(value.cpu().numpy(), want_v)
    got_lse = lse.cpu().numpy()
    assert np.array_equal(np.isnan(got_lse), np.isnan(want_lse))
    ok = ~np.isnan(want_lse)
    assert np.all(np.abs(got_lse[ok] - want_lse[ok]) <= F32_REL * np.abs(want_lse[ok]) + 1e-30)
    mismatch = assert_bf16_close(bf16_words(probs), want_p, want_p32, BF16_REL)
    assert mismatch < 1e-2
    return index


@pytest.mark.parametrize("batch", [1, 16])
def test_logits_config(oracle, batch):
    logits, tied = wl.logits_inputs(batch)
    assert tied
    index = check_logits(oracle, logits)
    for row in tied:  # the duplicated maximum: the lower copy wins
        peak = logits[row].max()
        assert int(index[row]) == int(np.flatnonzero(logits[row] == peak)[0])


def test_logits_config_256_rows_every_row_against_the_checker(oracle):
    """The benchmarked shape itself: all 256 rows of lse, probabilities, argmax index and value are
    compared with the checker, for the cluster kernel and (twice) for the streaming kernel."""
    logits, tied = wl.logits_inputs(256)
    assert len(tied) >= 2
    dev = to_dev(logits)
    want_lse, want_p, want_p32, want_i, want_v = oracle.logits_reduce(logits)

    def compare(lse, probs, index, value):
        assert np.array_equal(index.cpu().numpy(), want_i)
        assert_f32_bits(value.cpu().numpy(), want_v)
        assert np.all(np.abs(lse.cpu().numpy() - want_lse) <= F32_REL * np.abs(want_lse))
        assert assert_bf16_close(bf16_words(probs), want_p, want_p32, BF16_REL) < 1e-2
        assert np.all(np.abs(probs.float().sum(dim=1).cpu().numpy() - 1.0) < 2e-3)

    lse, probs, index, value = ops.logits_reduce(dev)
    compare(lse, probs, index, value)
    for row in tied:  # the duplicated maximum: the lower copy wins
        assert int(index[row]) == int(np.flatnonzero(logits[row] == logits[row].max())[0])
    # standalone argmax agrees with the fused launch
    idx2, val2 = ops.argmax(dev)
    assert torch.equal(idx2, index) and torch.equal(val2, value)
    del lse, probs
    # the streaming kernel (taken when a workspace is given): twice, every launch re-arms the workspace
    scratch = ops.make_logits_workspace("cuda", 256, logits.shape[1])
    for _ in range(2):
        compare(*ops.logits_reduce(dev, workspace=scratch))


@pytest.mark.parametrize("cols", [1024, 4112, 19456, 40000, 151936, 327680])
def test_logits_streaming_kernel_shapes_and_invalid_rows(oracle, cols):
    """Batches of 64 rows or more with a workspace take the two-pass streaming kernel."""
    rng = np.random.default_rng(cols + 1)
    rows = 72 if cols <= 151936 else 65
    x = (4.0 * rng.standard_normal((rows, cols))).astype(np.float32)
    x[1] *= 20.0
    x[2, cols // 2] = np.nan
    x[3, cols - 1] = np.inf
    x[4, :] = -np.inf
    x[5, 0] = -np.inf
    x[6, :] = np.nan; x[6, cols - 2] = -np.inf
    x[7, 5] = x[7, cols - 3] = x[7].max() + 1.0          # a tie across chunks: the lower index wins
    x[8, : cols // 2] = -np.inf                           # whole chunks at -inf
    x[rows - 1, cols - 1] = 1000.0                        # maximum in the last element of the last row
    scratch = ops.make_logits_workspace("cuda", rows, cols)
    for _ in range(2):
        index = check_logits(oracle, x, workspace=scratch)
    assert int(index[7]) == 5
    for log in (False, True):
        got = ops.softmax(to_dev(x), log=log, workspace=scratch).cpu().numpy()
        want = oracle.softmax(x, log=log)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = np.isfinite(want)
        tol = F32_REL * np.abs(want[ok]) + (1e-5 if log else 1e-37)
        assert np.all(np.abs(got[ok] - want[ok]) <= tol)
    # a smaller batch reuses the same workspace
    check_logits(oracle, x[:64], workspace=scratch)


@pytest.mark.parametrize("offset", [0.0, -3.0e4, 1.0e6, 1.0e8, -1.2e8])
def test_logits_of_large_magnitude(oracle, offset):
    """The kernels subtract ONE constant c = RN(max * log2 e) from every exponent of a row, fused into the multiplication.
    c misses max * log2 e by up to half an ulp of c, the same amount for every element: it cancels between a weight
    and the sum, and the lse takes it back out.  That holds while half an ulp of c is a small number, i.e. for logits
    below 2^27 in magnitude -- the domain the header states; both kernels, rows far from zero."""
    rng = np.random.default_rng(17)
    cols = 19456
    spread = max(4.0, abs(offset) * 2.0 ** -20)  # keep neighbours distinguishable in f32 around the offset
    for rows in (8, 72):                          # the cluster kernel, the streaming kernel
        x = (np.float32(offset) + np.float32(spread) * rng.standard_normal((rows, cols)).astype(np.float32)).astype(np.float32)
        x[1, 7] = x[1].max() + np.float32(8.0 * spread)
        scratch = ops.make_logits_workspace("cuda", rows, cols) if rows >= 64 else None
        check_logits(oracle, x, workspace=scratch)


def test_logits_streaming_kernel_reduces_missing_partials_itself(oracle, vectors=10):
    """The rare path, forced: with a window of one row a second-pass task is claimed right behind the
    first-pass tasks it depends on, and with one poll of patience its warps reduce the missing chunks
    themselves from global memory instead of waiting for another CTA.  Results and status must be those
    of the ordinary schedule; the same holds for every schedule a tuning can ask for."""
    rng = np.random.default_rng(vectors)
    rows, cols = 96, 40000
    x = (4.0 * rng.standard_normal((rows, cols))).astype(np.float32)
    x[2, cols // 2] = np.nan
    x[4, :] = -np.inf
    x[7, 5] = x[7, cols - 3] = x[7].max() + 1.0
    want_lse, want_p, want_p32, want_i, want_v = oracle.logits_reduce(x)
    dev = to_dev(x)
    scratch = ops.make_logits_workspace("cuda", rows, cols)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for window, patience, per_sm in [(1, 1, 4), (1, 1, 1), (2, 3, 2), (8, 0, 0), (0, 0, 3), (96, 0, 0)]:
        tuning = abi.StreamTuning(vectors, window, patience, per_sm)
        plan = ops.logits_stream_plan(rows, cols, tuning)
        assert plan is not None and plan.chunk_vectors == vectors
        assert plan.fixed_tasks_per_cta * plan.grid <= plan.window_rows * plan.chunks_per_row  # fixed tasks are first-pass tasks
        lse, probs, index, value = ops.logits_reduce(dev, workspace=scratch, status=status, tuning=tuning)
        assert np.array_equal(index.cpu().numpy(), want_i)
        assert_f32_bits(value.cpu().numpy(), want_v)
        got_lse = lse.cpu().numpy()
        ok = ~np.isnan(want_lse)
        assert np.array_equal(np.isnan(got_lse), ~ok)
        assert np.all(np.abs(got_lse[ok] - want_lse[ok]) <= F32_REL * np.abs(want_lse[ok]))
        assert_bf16_close(bf16_words(probs), want_p, want_p32, BF16_REL)
        assert status.item() == 0
    with pytest.raises(abi.KernelError):  # a tuning names the streaming kernel: shapes that cannot take it are refused
        ops.logits_reduce(dev[:8], workspace=scratch, tuning=abi.StreamTuning(vectors, 0, 0, 0))
    with pytest.raises(abi.KernelError):
        ops.logits_reduce(dev, workspace=scratch, tuning=abi.StreamTuning(7, 0, 0, 0))


def test_logits_stream_plan_of_the_benchmarked_shapes():
    for rows in (64, 256, 1024, 4096):
        plan = ops.logits_stream_plan(rows, wl.VOCAB)
        assert plan is not None
        assert plan.chunk_vectors == 10
        assert plan.chunks_per_row * plan.chunk_values >= wl.VOCAB > (plan.chunks_per_row - 1) * plan.chunk_values
        assert plan.chunk_values % 16 == 0 and plan.chunks_per_row <= 32
        assert 8 <= plan.window_rows <= min(rows, 64)
        assert plan.grid % plan.ctas_per_sm == 0 and 1 <= plan.ctas_per_sm <= 4
        assert plan.fixed_tasks_per_cta * plan.grid <= plan.window_rows * plan.chunks_per_row
    assert ops.logits_stream_plan(16, wl.VOCAB) is None          # small batches take the cluster kernel
    assert ops.logits_stream_plan(256, 151937) is None           # rows must be 64-byte multiples


@pytest.mark.parametrize("cols", [1, 7, 8, 1000, 1024, 19000, 19456, 40000, 151936, 262144])
def test_logits_shapes_and_invalid_rows(oracle, cols):
    rng = np.random.default_rng(cols)
    x = (4.0 * rng.standard_normal((7, cols))).astype(np.float32)
    x[1] *= 20.0
    if cols >= 7:
        x[2, cols // 2] = np.nan
        x[3, cols - 1] = np.inf
        x[4, :] = -np.inf
        x[5, 0] = -np.inf
        x[6, :] = np.nan; x[6, cols - 2] = -np.inf
    check_logits(oracle, x)
    # Softmax / LogSoftmax with f32 output
    for log in (False, True):
        got = ops.softmax(to_dev(x), log=log).cpu().numpy()
        want = oracle.softmax(x, log=log)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = np.isfinite(want)
        tol = F32_REL * np.abs(want[ok]) + (1e-5 if log else 1e-37)
        assert np.all(np.abs(got[ok] - want[ok]) <= tol)
    idx, val = ops.argmax(to_dev(x))
    want_i, want_v = oracle.argmax(x)
    assert np.array_equal(idx.cpu().numpy(), want_i)
    assert_f32_bits(val.cpu().numpy(), want_v)


def test_argmax_golden_cases(oracle, golden):
    x = golden["argmax_x"]
    idx, val = ops.argmax(to_dev(x))
    assert np.array_equal(idx.cpu().numpy(), golden["argmax_index"])
    assert_f32_bits(val.cpu().numpy(), golden["argmax_value"])
    _, _, idx2, _ = ops.logits_reduce(to_dev(x))
    assert np.array_equal(idx2.cpu().numpy(), golden["argmax_index"])


def test_argmax_value_is_the_winning_element_on_signed_zero_ties(oracle):
    """A row whose maximum is zero, first as -0 and later as +0: the index is the first one's and the
    value is THAT element (-0), as the reference's top_k_f32 returns scores[index]."""
    rng = np.random.default_rng(77)
    for rows, cols in [(3, 1000), (70, 40000)]:
        x = -np.abs(rng.standard_normal((rows, cols))).astype(np.float32) - 1.0
        x[0, 3], x[0, cols - 5] = -0.0, 0.0
        x[1, 7], x[1, 2] = -0.0, 0.0            # +0 first: it wins
        x[rows - 1, cols // 2], x[rows - 1, cols - 1] = -0.0, 0.0
        want_i, want_v = oracle.argmax(x)
        assert want_i[0] == 3 and np.signbit(want_v[0]) and want_i[1] == 2 and not np.signbit(want_v[1])
        dev = to_dev(x)
        scratch = ops.make_logits_workspace("cuda", rows, cols)
        for index, value in (ops.argmax(dev), ops.logits_reduce(dev)[2:], ops.logits_reduce(dev, workspace=scratch)[2:]):
            assert np.array_equal(index.cpu().numpy(), want_i)
            assert np.array_equal(value.cpu().numpy().view(np.uint32), want_v.view(np.uint32))


# ---- LayerNorm ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("hidden", [1, 8, 100, 256, 1000, 2048, 4096, 5000, 32768])
def test_layer_norm_hidden_sizes(oracle, hidden):
    """One bf16 step from the checker's rounded output, plus the conditioning of x - mean: the
    mean from another summation order differs by a few 1e-7 of the row's magnitude, which is an
    ABSOLUTE difference of that size (times inverse and scale) in every output, however small."""
    rng = np.random.default_rng(hidden)
    rows = 37 if hidden <= 4096 else 5
    x32 = (3.0 * rng.standard_normal((rows, hidden)) + rng.uniform(-20, 20, (rows, 1))).astype(np.float32)
    x = wl.f32_to_bf16(x32)
    scale = wl.f32_to_bf16(rng.uniform(0.5, 1.5, hidden).astype(np.float32))
    bias = wl.f32_to_bf16(rng.standard_normal(hidden).astype(np.float32))
    xf = wl.bf16_to_f32(x).astype(np.float64)
    inverse = 1.0 / np.sqrt(xf.var(axis=1, keepdims=True) + 1e-5)
    magnitude = np.abs(xf).max(axis=1, keepdims=True)
    for affine in (True, False):
        s, b = (scale, bias) if affine else (None, None)
        want, want32 = oracle.layer_norm(x, s, b, 1e-5)
        got = bf16_words(ops.layer_norm(to_dev_bf16(x), None if s is None else to_dev_bf16(s),
                                        None if b is None else to_dev_bf16(b), 1e-5))
        g, w = wl.bf16_to_f32(got).astype(np.float64), wl.bf16_to_f32(want).astype(np.float64)
        gain = np.abs(wl.bf16_to_f32(scale).astype(np.float64))[None, :] if affine else 1.0
        slack = 2e-6 * magnitude * inverse * gain * (1.0 + np.log2(max(hidden, 2)))
        assert np.all(np.abs(g - w) <= 2.0 ** -7 * np.abs(w) + slack + TINY)
        for g_row, w_row in zip(g, w):
            assert np.sqrt(np.sum((g_row - w_row) ** 2)) <= BF16_REL * np.sqrt(np.sum(w_row ** 2)) + TINY
        if hidden > 1:
            assert (got != want).mean() < 2e-2


# ---- Unary -----------------------------------------------------------------------------------------------------------------
UNARY_BIT_EXACT = {abi.UNARY_ABS, abi.UNARY_NEG, abi.UNARY_SQRT, abi.UNARY_RSQRT, abi.UNARY_RELU}
# gelu = 0.5 x (1 + erf(x / sqrt 2)) and its tanh form cancel for negative x: an error of one ulp in
# erf / tanh (libm and the GPU's functions round differently) is an ABSOLUTE error of about
# 2^-24 |x| in the result, however small the result is.  The bound below allows four such ulps.
UNARY_CANCELLING = {abi.UNARY_GELU, abi.UNARY_GELU_TANH}


@pytest.mark.parametrize("kind", range(13))
def test_unary_all_kinds_and_storage_types(oracle, kind):
    rng = np.random.default_rng(100 + kind)
    special = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1.0, -1.0, 20.0, 20.5, -20.0, 88.0, 89.0, -104.0,
                        1e-40, -1e-40, 3.0e38, 0.5, 7.0, -7.0, 1.0000001, 0.9999999], np.float32)
    x = np.concatenate([special, (4.0 * rng.standard_normal(70001)).astype(np.float32),
                        rng.uniform(-30, 30, 4099).astype(np.float32)])
    with np.errstate(all="ignore"):
        slack = 2.5e-7 * np.abs(x) if kind in UNARY_CANCELLING else np.zeros_like(x)
    want = oracle.unary(kind, ob.F32, x)
    got = ops.unary(kind, to_dev(x)).cpu().numpy()
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    if kind in UNARY_BIT_EXACT:
        assert np.array_equal(got.view(np.uint32)[ok], want.view(np.uint32)[ok])
    else:
        finite = ok & np.isfinite(want)
        assert np.array_equal(got[ok & ~finite], want[ok & ~finite])        # infinities agree
        # 1e-5 relative; results in the subnormal range within one subnormal step (the CPU's libm
        # and the GPU's functions round there differently)
        assert np.all(np.abs(got[finite] - want[finite]) <= F32_REL * np.abs(want[finite]) + 1.5e-45 + slack[finite])
    # unaligned start and a ragged tail take the scalar kernel
    base = to_dev(x)
    got_tail = ops.unary(kind, base[1:1000]).cpu().numpy()
    assert np.array_equal(got_tail.view(np.uint32), got.view(np.uint32)[1:1000])
    # 16-bit storage: f32 math, one rounding -> at most one storage step from the checker
    for name in ("bf16", "f16"):
        with np.errstate(all="ignore"):
            if name == "bf16":
                x16 = wl.f32_to_bf16(x)
                x_back = wl.bf16_to_f32(x16)
                got16 = bf16_words(ops.unary(kind, to_dev_bf16(x16)))
                want16 = oracle.unary(kind, ob.BF16, x16)
                decode, exp_mask, step = wl.bf16_to_f32, 0x7F80, 2.0 ** -7
            else:
                x16 = x.astype(np.float16).view(np.uint16)
                x_back = x16.view(np.float16).astype(np.float32)
                got16 = ops.unary(kind, to_dev(x16.view(np.float16))).cpu().numpy().view(np.uint16)
                want16 = oracle.unary(kind, ob.F16, x16)
                decode, exp_mask, step = (lambda w: w.view(np.float16).astype(np.float32)), 0x7C00, 2.0 ** -10
        nan16 = (want16 & 0x7FFF) > exp_mask
        assert np.array_equal((got16 & 0x7FFF) > exp_mask, nan16)
        if kind in UNARY_BIT_EXACT:
            assert np.array_equal(got16[~nan16], want16[~nan16])
            continue
        distance = np.abs(ordered16(got16[~nan16]) - ordered16(want16[~nan16]))
        if kind in UNARY_CANCELLING:
            with np.errstate(all="ignore"):
                g, w = decode(got16[~nan16]), decode(want16[~nan16])
                bound = step * np.abs(w) + 2.5e-7 * np.abs(x_back[~nan16]) + (6e-8 if name == "f16" else 1e-40)
                same = (g == w) | (np.abs(g - w) <= bound)
            assert np.all(same)
        else:
            assert distance.max() <= 1
            assert (distance != 0).mean() < 1e-2


def ordered16(words):
    """16-bit float words as integers that increase with the value (sign-magnitude -> two's complement)."""
    w = words.astype(np.int32)
    return np.where(w & 0x8000, -(w & 0x7FFF), w)


CAST_PAIRS = [(abi.F32, abi.BF16), (abi.F32, abi.F16), (abi.BF16, abi.F32), (abi.F16, abi.F32), (abi.BF16, abi.F16),
              (abi.F16, abi.BF16), (abi.I32, abi.F32), (abi.F32, abi.BOOL), (abi.BF16, abi.BOOL), (abi.F16, abi.BOOL),
              (abi.BOOL, abi.F32), (abi.BOOL, abi.BF16), (abi.BOOL, abi.F16), (abi.F32, abi.E4M3), (abi.BF16, abi.E4M3),
              (abi.F16, abi.E4M3), (abi.E4M3, abi.F32), (abi.E4M3, abi.BF16), (abi.E4M3, abi.F16), (abi.E5M2, abi.BF16),
              (abi.E5M2, abi.E4M3)]


@pytest.mark.parametrize("pair", CAST_PAIRS, ids=lambda p: f"{p[0]}to{p[1]}")
def test_cast_pairs_bit_exact(oracle, pair):
    source, destination = pair
    rng = np.random.default_rng(source * 16 + destination)
    with np.errstate(all="ignore"):
        half = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)   # every f16 value
        wide = (rng.standard_normal(70003) * np.exp(rng.uniform(-40, 40, 70003))).astype(np.float32)
        edge = np.array([0.0, -0.0, 448.0, 449.0, 464.0, 465.0, 480.0, 57344.0, 65504.0, 65520.0, 2.0 ** -9, 2.0 ** -10,
                         2.0 ** -24, 2.0 ** -25, 1e-45, 3.4e38, -3.4e38, np.inf, -np.inf, np.nan], np.float32)
        values = np.concatenate([half, wide, edge])
        if source == abi.F32:
            words = values
        elif source == abi.BF16:
            words = wl.f32_to_bf16(values)
        elif source == abi.F16:
            words = values.astype(np.float16).view(np.uint16)
        elif source == abi.I32:
            words = np.concatenate([rng.integers(-2 ** 31, 2 ** 31 - 1, 70001, dtype=np.int64).astype(np.int32),
                                    np.array([0, 1, -1, 16777217, 16777219, -16777217, 2 ** 31 - 1, -2 ** 31], np.int32)])
        else:  # the one-byte types: every byte value, many times, at an odd length
            words = np.tile(np.arange(256, dtype=np.uint8), 300)[:70001]
    want = oracle.cast(source, destination, words)
    carrier = {abi.BF16: torch.bfloat16, abi.F16: torch.float16}
    dev = to_dev(words)
    if source in carrier:
        dev = dev.view(carrier[source])
    got = ops.cast(dev, source, destination)
    got_words = got.view(torch.int16 if destination in carrier else got.dtype).cpu().numpy().view(want.dtype)
    if destination in (abi.F32, abi.BF16, abi.F16):  # NaN payloads are not part of the contract, NaN-ness is
        exp_mask, frac = {abi.F32: (0x7F800000, 0x7FFFFF), abi.BF16: (0x7F80, 0x7F), abi.F16: (0x7C00, 0x3FF)}[destination]
        as_int = {abi.F32: np.uint32, abi.BF16: np.uint16, abi.F16: np.uint16}[destination]
        w, g = want.view(as_int), got_words.view(as_int)
        nan = ((w & exp_mask) == exp_mask) & ((w & frac) != 0)
        assert np.array_equal(((g & exp_mask) == exp_mask) & ((g & frac) != 0), nan)
        assert np.array_equal(g[~nan], w[~nan])
    else:
        assert np.array_equal(got_words, want)
    # an unaligned slice takes the scalar kernel and agrees
    tail = ops.cast(dev[3:1003], source, destination)
    raw = {torch.float32: torch.int32, torch.bfloat16: torch.int16, torch.float16: torch.int16}.get(got.dtype, got.dtype)
    assert torch.equal(tail.view(raw), got[3:1003].view(raw))  # compared as bits: NaN is not equal to itself


@pytest.mark.parametrize("dtype", [abi.F32, abi.BF16, abi.F16])
def test_fp8_cache_encode(oracle, dtype):
    rng = np.random.default_rng(40 + dtype)
    x = (rng.standard_normal(100003) * np.exp(rng.uniform(-12, 8, 100003))).astype(np.float32)
    x[:6] = [0.0, -0.0, 448.0 * 0.37, 1e9, -1e9, 2.0 ** -12]
    if dtype == abi.F32:
        words, dev = x, to_dev(x)
    elif dtype == abi.BF16:
        words = wl.f32_to_bf16(x); dev = to_dev_bf16(words)
    else:
        with np.errstate(all="ignore"):
            words = x.astype(np.float16).view(np.uint16)
        dev = to_dev(words.view(np.float16))
    for scale in (1.0, 0.37, 3.0):
        want, want_status = oracle.fp8_e4m3_encode({abi.F32: ob.F32, abi.BF16: ob.BF16, abi.F16: ob.F16}[dtype], words, scale)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        got = ops.fp8_e4m3_encode(dev, scale, status)
        assert np.array_equal(got.cpu().numpy(), want)
        assert int(status.item()) == want_status
        assert torch.equal(ops.fp8_e4m3_encode(dev[1:2001], scale), got[1:2001])      # unaligned: scalar kernel
    if dtype == abi.F32:
        bad = x.copy(); bad[7] = np.nan; bad[70001] = np.inf
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        got = ops.fp8_e4m3_encode(to_dev(bad), 1.0, status).cpu().numpy()
        want, want_status = oracle.fp8_e4m3_encode(ob.F32, bad, 1.0)
        assert np.array_equal(got, want) and got[7] == 0 and got[70001] == 0
        assert int(status.item()) == abi.STATUS_INVALID_FP8_INPUT == want_status


def test_fp8_cache_encode_at_every_rounding_boundary(oracle):
    """The kernel multiplies by the reciprocal of the scale and divides only when the product is within
    2^-21 of a rounding boundary of E4M3.  Inputs placed on and next to every boundary (midpoints of
    neighbouring E4M3 values, times the scale, and their f32 neighbours) must give the bytes of the division;
    so must scales whose reciprocal is not a normal number (every element then takes the division)."""
    codes = np.arange(0, 127, dtype=np.uint8)                       # the non-negative finite codes, ascending
    values = oracle.cast(ob.E4M3, ob.F32, codes).astype(np.float64)
    midpoints = (values[:-1] + values[1:]) / 2
    for scale in (1.0, 0.37, 3.0, 1.0 / 3.0, 1e-3, 417.25, 1e-39, 3e38):
        with np.errstate(over="ignore", under="ignore"):
            centre = (np.concatenate([midpoints, values]) * np.float64(np.float32(scale))).astype(np.float32)
        cases = [centre]
        for direction in (np.float32(np.inf), np.float32(-np.inf)):
            step = centre
            for _ in range(3):
                step = np.nextafter(step, direction)
                cases.append(step)
        x = np.concatenate(cases + [-c for c in cases])
        x = x[np.isfinite(x)]
        x = np.concatenate([x, np.zeros((-x.size) % 8, np.float32)])
        want, want_status = oracle.fp8_e4m3_encode(ob.F32, x, scale)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        got = ops.fp8_e4m3_encode(to_dev(x), scale, status).cpu().numpy()
        assert np.array_equal(got, want), scale
        assert int(status.item()) == want_status == 0


# ---- sampling --------------------------------------------------------------------------------------------------------------
def _identities(rng, rows):
    return rng.integers(0, 2 ** 32, (rows, 4), dtype=np.uint64).astype(np.uint32)


@pytest.mark.parametrize("words", [1, 3, 4, 7, 64, 508, 512, 1001, 2053, 4096])  # rows of 512 words and more take warp spans
def test_random_bits_bit_exact(oracle, golden, words):
    rng = np.random.default_rng(words)
    identities = np.concatenate([golden["random_identities"], _identities(rng, 700)])
    got = ops.random_bits(to_dev(identities.view(np.int32)), words).cpu().numpy().view(np.uint32)
    assert np.array_equal(got, oracle.random_bits(identities, words))
    if words >= 4:
        assert np.array_equal(got[:5, :min(words, 40)], golden["random_words"][:, :min(words, 40)])


@pytest.mark.parametrize("dtype", [abi.F32, abi.BF16, abi.F16])
@pytest.mark.parametrize("cols", [1, 5, 1000, 4099, 151936])
def test_categorical_draws(oracle, dtype, cols):
    """Indices agree with the CPU restatement except where the two summation orders put the threshold
    on different sides of a cumulative boundary; every draw is checked against the cumulative
    distribution itself, and log p against x - lse."""
    rng = np.random.default_rng(cols + dtype)
    rows = 48 if cols > 10000 else 300
    x = (3.0 * rng.standard_normal((rows, cols))).astype(np.float32)
    if cols >= 1000:
        x[3, 10:] = -np.inf
        x[4, :] = -np.inf; x[4, 777] = 0.0
        x[5, : cols // 2] = -np.inf
    identities = _identities(rng, rows)
    if dtype == abi.F32:
        words, dev, odt = x, to_dev(x), ob.F32
    elif dtype == abi.BF16:
        words = wl.f32_to_bf16(x); dev, odt = to_dev_bf16(words), ob.BF16
        x = wl.bf16_to_f32(words)
    else:
        h = x.astype(np.float16); words = h.view(np.uint16); dev, odt = to_dev(h), ob.F16
        x = h.astype(np.float32)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    index, logp = ops.categorical(dev, to_dev(identities.view(np.int32)), True, status)
    index, logp = index.cpu().numpy(), logp.cpu().numpy()
    want_index, want_logp, uniform, invalid = oracle.categorical(odt, words, identities)
    assert invalid == 0 and int(status.item()) == 0
    assert (index == want_index).mean() >= 0.99
    w = np.exp((x - x.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float64)
    c = np.cumsum(w, axis=1)
    for r in range(rows):
        t = c[r, -1] * uniform[r]
        i = int(index[r])
        assert 0 <= i < cols and w[r, i] > 0
        assert c[r, i] > t * (1 - 1e-9) and (i == 0 or c[r, i - 1] <= t * (1 + 1e-9))
        assert abs(logp[r] - (x[r, i] - x[r].max() - np.log(c[r, -1]))) < 2e-5
    if cols >= 1000:
        assert index[4] == 777 and 0 <= index[3] < 10 and index[5] >= cols // 2
    # a row's draw does not depend on where the row sits or on the batch
    perm = rng.permutation(rows)
    index_p, _ = ops.categorical(dev[torch.from_numpy(perm).to(DEV)].contiguous(), to_dev(identities[perm].view(np.int32)), False)
    assert np.array_equal(index_p.cpu().numpy(), index[perm])


def test_categorical_rejects_invalid_rows():
    x = torch.randn(4, 100, device=DEV)
    x[0, 5] = float("nan"); x[1, 6] = float("inf"); x[2, :] = float("-inf")
    identities = torch.arange(16, dtype=torch.int32, device=DEV).reshape(4, 4)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    index, logp = ops.categorical(x, identities, True, status)
    assert index[:3].tolist() == [-1, -1, -1] and int(index[3]) >= 0
    assert bool(torch.isnan(logp[:3]).all()) and int(status.item()) == abi.STATUS_INVALID_CATEGORICAL_ROW


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32])
def test_select_moves_bits(dtype):
    """out = condition ? a : b, bit for bit (NaN payloads, -0), any non-zero byte is true; branches of the full
    shape, of the trailing axes, or scalars; an unaligned slice takes the element-wise kernel."""
    gen = torch.Generator(device="cpu").manual_seed(5)
    shape = (97, 264)
    raw = {torch.float32: torch.int32, torch.int32: torch.int32}.get(dtype, torch.int16)
    bits_a = torch.randint(-2 ** 15, 2 ** 15 - 1, shape, generator=gen).to(raw)
    bits_b = torch.randint(-2 ** 15, 2 ** 15 - 1, shape, generator=gen).to(raw)
    if raw == torch.int32:
        bits_a = bits_a * 65536 + 12345
        bits_b = bits_b * 65536 - 54321
    a, b = bits_a.to(DEV).view(dtype), bits_b.to(DEV).view(dtype)
    condition = torch.randint(0, 3, shape, generator=gen).to(torch.uint8)
    condition[condition == 2] = 200
    cond = condition.to(DEV)
    want = torch.where(cond != 0, a.view(raw), b.view(raw))
    assert torch.equal(ops.select(cond, a, b).view(raw), want)
    row = b[0].contiguous()
    want_row = torch.where(cond != 0, a.view(raw), row.view(raw)[None, :])
    assert torch.equal(ops.select(cond, a, row).view(raw), want_row)
    scalar = a[3, 5:6].contiguous()
    want_scalar = torch.where(cond != 0, scalar.view(raw), b.view(raw))
    assert torch.equal(ops.select(cond, scalar, b).view(raw), want_scalar)
    flat_c, flat_a, flat_b = cond.reshape(-1)[3:2000], a.reshape(-1)[3:2000], b.reshape(-1)[3:2000]
    assert torch.equal(ops.select(flat_c, flat_a, flat_b).view(raw), want.reshape(-1)[3:2000])


@pytest.mark.parametrize("cols", [1, 7, 128, 1000, 1024, 2056, 4096, 5000])
def test_masked_scaled_softmax_f16(oracle, cols):
    rng = np.random.default_rng(cols)
    heads, queries = 3, 17
    x = (4.0 * rng.standard_normal((heads, queries, cols))).astype(np.float16)
    mask = (rng.random((queries, cols)) < 0.7).astype(np.uint8)          # shared by the heads
    mask[:, 0] = 1
    if cols > 1:
        mask[3, :] = 0                                                    # a fully masked row: all NaN
        x[1, 5, cols // 2] = np.nan; mask[5, cols // 2] = 1
        mask[6, :] = 0; mask[6, cols - 1] = 7                             # any non-zero byte is true
    # positive scales take the kernel that folds the scale into the exponent (rows of up to 2048 values); zero, negative
    # and huge ones the plain form
    for scale in (1.0, 0.125, 0.3, -0.5, 0.0, 1e10):
        want16, want32 = oracle.masked_softmax_f16(x.view(np.uint16), mask[None], scale)
        got = ops.masked_softmax_f16(to_dev(x), to_dev(mask), scale).cpu().numpy().view(np.uint16)
        nan = (want16 & 0x7FFF) > 0x7C00
        assert np.array_equal((got & 0x7FFF) > 0x7C00, nan)
        distance = np.abs(ordered16(got[~nan]) - ordered16(want16[~nan]))
        assert distance.max(initial=0) <= 1 and (distance != 0).mean() < 2e-2
    # a mask of the tensor's own shape
    full = (rng.random(x.shape) < 0.5).astype(np.uint8); full[..., 0] = 1
    want16, _ = oracle.masked_softmax_f16(x.view(np.uint16), full, 0.5)
    got = ops.masked_softmax_f16(to_dev(x), to_dev(full), 0.5).cpu().numpy().view(np.uint16)
    nan = (want16 & 0x7FFF) > 0x7C00
    assert np.array_equal((got & 0x7FFF) > 0x7C00, nan)
    assert np.abs(ordered16(got[~nan]) - ordered16(want16[~nan])).max(initial=0) <= 1


@pytest.mark.parametrize("cols", [1, 7, 128, 1000, 1024, 2056, 4096, 5000])
def test_additive_masked_softmax_f16(oracle, cols):
    """Softmax{scale, mask=kAdditive}: f16 addends of the trailing axes or of the tensor's shape; 0 keeps, -inf masks."""
    rng = np.random.default_rng(100 + cols)
    heads, queries = 3, 17
    x = (4.0 * rng.standard_normal((heads, queries, cols))).astype(np.float16)
    addend = (2.0 * rng.standard_normal((queries, cols))).astype(np.float16)
    addend[rng.random((queries, cols)) < 0.3] = -np.inf
    addend[:, 0] = 0
    if cols > 1:
        addend[3, :] = -np.inf                                            # a fully masked row: all NaN
        addend[5, cols // 2] = np.nan                                     # NaN addend: the row is NaN
        addend[6, :] = -np.inf; addend[6, cols - 1] = 3.5
        x[2, 7, cols - 1] = np.inf                                        # +inf score: NaN
        addend[8, 0] = np.inf
    for scale in (1.0, 0.125, -0.7, 100.0):  # beyond |scale| = 32 the kernel keeps the exact subtraction of the maximum
        want16, _ = oracle.masked_softmax_f16(x.view(np.uint16), addend[None], scale)
        got = ops.masked_softmax_f16(to_dev(x), to_dev(addend), scale).cpu().numpy().view(np.uint16)
        nan = (want16 & 0x7FFF) > 0x7C00
        assert np.array_equal((got & 0x7FFF) > 0x7C00, nan)
        distance = np.abs(ordered16(got[~nan]) - ordered16(want16[~nan]))
        assert distance.max(initial=0) <= 1 and (distance != 0).mean() < 2e-2
    full = (rng.standard_normal(x.shape)).astype(np.float16); full[rng.random(x.shape) < 0.5] = -np.inf; full[..., 0] = 0
    want16, _ = oracle.masked_softmax_f16(x.view(np.uint16), full, 0.5)
    got = ops.masked_softmax_f16(to_dev(x), to_dev(full), 0.5).cpu().numpy().view(np.uint16)
    nan = (want16 & 0x7FFF) > 0x7C00
    assert np.array_equal((got & 0x7FFF) > 0x7C00, nan)
    assert np.abs(ordered16(got[~nan]) - ordered16(want16[~nan])).max(initial=0) <= 1
    # all-zero addends are the unmasked scaled softmax: bit-equal to the Boolean kernel with an all-true mask
    zero = np.zeros((queries, cols), np.float16)
    a = ops.masked_softmax_f16(to_dev(x), to_dev(zero), 0.25)
    b = ops.masked_softmax_f16(to_dev(x), to_dev(np.ones((queries, cols), np.uint8)), 0.25)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_cast_rejects_other_pairs():
    x = torch.zeros(16, device=DEV)
    with pytest.raises(abi.KernelError):
        ops.cast(x, abi.F32, abi.E5M2)


def test_cast_f32_to_bf16(oracle):
    rng = np.random.default_rng(2)
    for count in [1, 7, 8, 4096, 100003]:
        x = rng.standard_normal(count).astype(np.float32)
        x[0] = 1.00390625  # a tie: rounds to even
        assert np.array_equal(bf16_words(ops.cast_f32_to_bf16(to_dev(x))), oracle.f32_to_bf16(x))


# ---- workload 5: Q8_0 + sum of squares -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows", [1, 3, 1024])
def test_q8_0_roundtrip_against_checker(oracle, rows):
    w = wl.q8_sweep_inputs(rows)
    dev = to_dev_bf16(w)
    ws = ops.make_workspace(DEV, w.size)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for _ in range(2):  # the workspace is reusable
        blocks, decoded, total = ops.q8_0_roundtrip(dev, ws, status=status)
        want_blocks, want_decoded, want_total, invalid = oracle.q8_0_roundtrip(w)
        assert np.array_equal(blocks.cpu().numpy(), want_blocks)              # bit-exact
        assert np.array_equal(bf16_words(decoded).ravel(), want_decoded)      # bit-exact
        assert abs(total.item() - want_total) <= F32_REL * want_total
        assert status.item() == 0 and not invalid
    # the separate operators give the same bytes
    assert torch.equal(ops.q8_0_encode(dev).ravel(), blocks)
    assert torch.equal(ops.q8_0_decode(blocks, w.size).view(torch.int16), decoded.view(torch.int16).ravel())
    assert abs(ops.sum_squares(dev, ws).item() - want_total) <= F32_REL * want_total


def _encode_case(oracle, values, dtype):
    if dtype == "f32":
        payload, kind, dev = values, ob.F32, to_dev(values)
    elif dtype == "bf16":
        payload, kind = wl.f32_to_bf16(values), ob.BF16
        dev = to_dev_bf16(payload)
    else:
        with np.errstate(over="ignore"):
            half = values.astype(np.float16)
        payload, kind, dev = half.view(np.uint16), ob.F16, to_dev(half)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops.q8_0_encode(dev.reshape(1, -1), status).cpu().numpy().ravel()
    want, invalid = oracle.q8_0_encode(kind, payload)
    assert np.array_equal(got, want)
    assert bool(status.item() & abi.STATUS_INVALID_Q8_INPUT) == invalid
    return got, invalid


def test_q8_0_scale_shortcuts_equal_the_divisions_for_every_magnitude():
    """amax / 127 by multiplication and one fused correction, and 1 / d by the IEEE reciprocal instruction,
    against __fdiv_rn for all 2^31-odd magnitudes the encoder accepts: no disagreement."""
    counter = torch.full((1,), -1, dtype=torch.int64, device=DEV)
    abi.check("selfcheck", abi.load().hyle_b200_selfcheck_q8_0_scale(torch.cuda.current_stream().cuda_stream, counter.data_ptr()))
    assert int(counter.item()) == 0


def test_q8_0_negative_values_that_round_to_zero_decode_to_plus_zero(oracle):
    """The code 0 decodes to +0 whatever the sign of the value it came from ((float)(int8_t)0 is +0 on the CPU)."""
    x = np.zeros((4, 64), np.float32)
    x[:, 0] = 100.0
    x[:, 1:9] = -0.3          # |p| < 0.5: code 0
    x[:, 9:17] = -0.0
    x[2, :32] = -1e-30        # a block whose scale rounds to zero: all codes 0
    words = wl.f32_to_bf16(x)
    want_blocks, want_decoded, _, invalid = oracle.q8_0_roundtrip(words)
    blocks, decoded, _ = ops.q8_0_roundtrip(to_dev_bf16(words), ops.make_workspace(DEV, words.size))
    assert not invalid
    assert np.array_equal(blocks.cpu().numpy().ravel(), want_blocks.ravel())
    assert np.array_equal(bf16_words(decoded).ravel(), want_decoded.ravel())
    assert not (bf16_words(decoded) == 0x8000).any()


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_q8_0_known_answers(oracle, dtype):
    # tests/compute_provider_ggml/native_paged_test.cc:255-276: ties, zero block, three input types
    values = np.array([float(int(i % 23) - 11) * 0.03125 for i in range(256)], np.float32)
    values[:5] = [127.0, 0.5, 1.5, -0.5, -1.5]
    values[32:64] = 0.0
    got, invalid = _encode_case(oracle, values, dtype)
    assert not invalid and got[3] == 1 and got[4] == 2 and got[5].view(np.int8) == -1
    # :288-326: scale boundaries around the smallest non-zero f16 scale
    zero_boundary = np.float32(127.0) * np.float32(2.0 ** -25)
    minimum_scale = np.float32(127.0) * np.float32(2.0 ** -24)
    nxt = lambda v, d: np.nextafter(np.float32(v), np.float32(d))
    amplitudes = [0.0, np.float32(1e-45), np.finfo(np.float32).tiny, 2.0 ** -122, 2.0 ** -120, 2.0 ** -24,
                  nxt(zero_boundary, 0), zero_boundary, nxt(zero_boundary, 1), nxt(minimum_scale, 0),
                  minimum_scale, nxt(minimum_scale, 1), 2.0 ** -14, 65504.0]
    if dtype == "f32":
        amplitudes.append(65504.0 * 127.0)
    values = np.zeros(len(amplitudes) * 64, np.float32)
    for i in range(values.size):
        a = np.float32(amplitudes[i // 64])
        values[i] = [a, -a, a * np.float32(0.125), -a * np.float32(0.125), 0.0, -0.0, 0.0, 0.0][i % 8]
    got, invalid = _encode_case(oracle, values, dtype)
    assert not invalid
    scales = got.reshape(-1, 34)[:, :2].copy().view(np.uint16).ravel()
    assert np.any(scales == 0) and np.any(scales != 0)


def test_q8_0_invalid_payload_sets_status_and_zeroes_the_block(oracle):
    # native_paged_test.cc:339-348
    for bad in (np.nan, np.inf, -np.inf, 9000000.0):
        values = np.ones(64 * 9, np.float32)
        values[19] = bad
        got, invalid = _encode_case(oracle, values, "f32")
        assert invalid and np.all(got[:34] == 0) and np.any(got[34:68] != 0)
    values = np.ones(64, np.float32)
    values[40] = np.inf
    _, invalid = _encode_case(oracle, values, "bf16")
    assert invalid
    _, invalid = _encode_case(oracle, values, "f16")
    assert invalid


def test_q8_0_rounding_ties_and_ragged_tiles(oracle):
    # every k + 0.5 tie and its neighbours with scale exactly 1 (amax 127)
    ks = np.arange(-126, 127, dtype=np.float32)
    ties = np.concatenate([ks + 0.5, np.nextafter(ks + np.float32(0.5), np.float32(1e9)),
                           np.nextafter(ks + np.float32(0.5), np.float32(-1e9))]).astype(np.float32)
    pad = (-ties.size) % 31
    ties = np.concatenate([ties, np.zeros(pad, np.float32)]).reshape(-1, 31)
    values = np.concatenate([np.full((ties.shape[0], 1), 127.0, np.float32), ties], axis=1).ravel()
    _encode_case(oracle, values, "f32")
    # block counts that are not multiples of the 256-block tile
    rng = np.random.default_rng(8)
    for blocks in [1, 3, 255, 257, 513, 1000]:
        w = wl.f32_to_bf16((0.02 * rng.standard_normal(blocks * 32)).astype(np.float32))
        dev = to_dev_bf16(w)
        ws = ops.make_workspace(DEV, w.size)
        got_b, got_d, got_s = ops.q8_0_roundtrip(dev, ws)
        want_b, want_d, want_s, _ = oracle.q8_0_roundtrip(w)
        assert np.array_equal(got_b.cpu().numpy(), want_b)
        assert np.array_equal(bf16_words(got_d), want_d)
        assert abs(got_s.item() - want_s) <= F32_REL * want_s
        # unaligned carrier (2-byte aligned only)
        carrier = torch.zeros(blocks * 34 + 16, dtype=torch.uint8, device=DEV)
        view = carrier[2:2 + blocks * 34]
        ops.q8_0_roundtrip(dev, ws, blocks=view)
        assert np.array_equal(view.cpu().numpy(), want_b)
        assert int(carrier[:2].sum()) == 0 and int(carrier[2 + blocks * 34:].sum()) == 0  # margins untouched
        assert torch.equal(ops.q8_0_decode(view, w.size).view(torch.int16), got_d.view(torch.int16))


def test_q8_0_full_size_properties():
    """At a large size the checker is too slow; use what the format guarantees instead:
    decode(encode(x)) from the fused kernel equals the separate decode of its own blocks,
    encoding the decoded tensor reproduces the codes' scale class (idempotence of the grid),
    the sum of squares is additive over row shards, and the error is within half a step."""
    rows = 32768  # 512 MiB of bf16
    shard = wl.shard_rows(rows, 1, 0)
    w = wl.q8_sweep_device_shard(shard)
    ws = ops.make_workspace(DEV, w.numel())
    blocks, decoded, total = ops.q8_0_roundtrip(w, ws)
    again = ops.q8_0_roundtrip(w, ws)[2]
    assert again.item() == total.item()  # dynamic tile scheduling, yet the same bits every run
    assert torch.equal(ops.q8_0_decode(blocks, w.numel()).view(torch.int16), decoded.view(torch.int16).ravel())
    b = blocks.view(-1, 34)
    scale = b[:, :2].contiguous().view(torch.float16).float()
    err = (decoded.float().view(-1, 32) - w.float().view(-1, 32)).abs()
    bound = 0.5 * scale * (1 + 2 ** -10) + w.float().view(-1, 32).abs() * 2 ** -8 + 1e-12
    assert bool((err <= bound).all())
    assert int(b[:, 2:].view(torch.int8).abs().max()) == 127  # every block uses its full range
    halves = [ops.sum_squares(w[: rows // 2], ws).item(), ops.sum_squares(w[rows // 2:], ws).item()]
    assert abs(sum(halves) - total.item()) <= 1e-9 * total.item()
    reference = (w.double() ** 2).sum().item()
    assert abs(total.item() - reference) <= F32_REL * reference


def test_q8_0_benchmark_size_chunks_against_checker(oracle):
    """R = 262144 x 8192, the size the throughput is quoted on: 2^31 values, byte offsets up to 4 GiB in
    both bf16 tensors, i.e. past the signed 32-bit range from the middle on.  The input is generated on
    the device; three 1024-row chunks (the first rows, the rows straddling the 2 GiB byte offset, the
    last rows) are copied back and their blocks and decoded values must equal, byte for byte, the
    checker's on the very same input words (the formula of tests/compute_provider_ggml/native_paged_test.cc:255-326)."""
    rows, cols, chunk = 262144, wl.SWEEP_COLS, 1024
    free, _ = torch.cuda.mem_get_info()
    if free < 20 * 2 ** 30:
        pytest.skip("needs about 13 GiB of free device memory")
    w = wl.q8_sweep_device_shard(wl.shard_rows(rows, 1, 0))
    ws = ops.make_workspace(DEV, w.numel())
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    blocks, decoded, total = ops.q8_0_roundtrip(w, ws, status=status)
    assert status.item() == 0
    blocks2d = blocks.view(rows, cols // 32 * 34)
    for first in (0, rows // 2 - chunk // 2, rows - chunk):
        words = bf16_words(w[first:first + chunk]).copy()
        want_blocks, want_decoded, _, invalid = oracle.q8_0_roundtrip(words)
        assert not invalid
        assert np.array_equal(blocks2d[first:first + chunk].cpu().numpy().ravel(), want_blocks), first
        assert np.array_equal(bf16_words(decoded[first:first + chunk]).ravel(), want_decoded), first
    # sum of squares against a chunked f64 sum on the device
    reference = 0.0
    for first in range(0, rows, 16384):
        reference += (w[first:first + 16384].double() ** 2).sum().item()
    assert abs(total.item() - reference) <= F32_REL * reference
    # the separate decode of the kernel's own blocks reproduces the fused output across the whole 4 GiB
    again = ops.q8_0_decode(blocks, w.numel())
    assert torch.equal(again.view(torch.int16), decoded.view(torch.int16).ravel())


# ---- stream capture ----------------------------------------------------------------------------------------------------------
def test_a_sequence_of_entry_points_replays_in_a_cuda_graph():
    """The provider declares its kernels capture-compatible (no synchronisation, no allocation, launch shapes that
    depend on sizes only).  One graph holds the residual norm, the gating, the streaming logits reduction with
    its workspace, the Q8_0 round trip with its workspace, the checked scan (two kernels) and the categorical
    draw; three replays on new inputs must give the bits of the same calls made eagerly, which also shows that
    every launch leaves its workspace armed for the next."""
    generator = torch.Generator(device=DEV)
    x = torch.empty((128, 2048), dtype=torch.bfloat16, device=DEV)
    r = torch.empty_like(x)
    w = (torch.rand(2048, device=DEV) + 0.5).bfloat16()
    gate = torch.empty((64, 6144), dtype=torch.bfloat16, device=DEV)
    up = torch.empty_like(gate)
    logits = torch.empty((64, 40000), device=DEV)
    bank = torch.empty((64, 8192), dtype=torch.bfloat16, device=DEV)
    counts = torch.empty((32, 4096), dtype=torch.int32, device=DEV)
    identities = torch.arange(64 * 4, dtype=torch.int32, device=DEV).view(64, 4).contiguous()
    logits_ws = ops.make_logits_workspace(DEV, 64, 40000)
    bank_ws = ops.make_workspace(DEV, bank.numel())
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops.logits_stream_plan(64, 40000) is not None            # this shape does take the streaming kernel

    def refill(seed):
        generator.manual_seed(seed)
        for t, scale in ((x, 1.0), (r, 1.0), (gate, 1.5), (up, 1.5), (logits, 4.0), (bank, 0.02)):
            t.copy_(torch.randn(t.shape, generator=generator, device=DEV) * scale)
        counts.copy_(torch.randint(-1000, 1000, counts.shape, generator=generator, device=DEV, dtype=torch.int32))

    def sequence():
        y, h = ops.add_rms_norm(x, r, w, 1e-6)
        out = ops.swiglu(gate, up)
        lse, probs, index, value = ops.logits_reduce(logits, workspace=logits_ws, status=status)
        blocks, decoded, total = ops.q8_0_roundtrip(bank, bank_ws, status=status)
        prefix = ops.scan(counts, status=status)
        draw, logp = ops.categorical(logits, identities, status=status)
        return [y, h, out, lse, probs, index, value, blocks, decoded, total, prefix, draw, logp]

    refill(0)
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        sequence()                                                   # warm-up outside the capture
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            captured = sequence()
    torch.cuda.synchronize()
    for seed in (1, 2, 3):
        refill(seed)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        eager = sequence()
        torch.cuda.synchronize()
        for got, want in zip(captured, eager):
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
        assert status.item() == 0


# ---- more than 2^31 elements, more than 2^32 bytes ---------------------------------------------------------------------------
def test_elementwise_entries_index_beyond_two_to_the_31_elements():
    """Unary, Binary (trailing-axis broadcast), Select and Cast on 2^31 + 4104 bf16 / f32 elements: the last elements,
    and elements on both sides of the 2^31 element and 2^32 byte marks, carry the values of the small case."""
    count = 2 ** 31 + 4104
    probes = torch.tensor([0, 1, 2 ** 31 - 8, 2 ** 31 - 1, 2 ** 31, 2 ** 31 + 1, 2 ** 31 + 4096, count - 9, count - 1], device=DEV)
    x = torch.empty(count, dtype=torch.bfloat16, device=DEV)
    x.view(torch.int16).copy_(torch.arange(count, device=DEV, dtype=torch.int64).remainder_(24001).sub_(12000).to(torch.int16))
    x.copy_(x.view(torch.int16).to(torch.bfloat16) * 0.25)            # values -3000 ... 3000, exact in bf16 steps
    want = x[probes].float()
    got = ops.unary(abi.UNARY_ABS, x)
    assert torch.equal(got[probes].float(), want.abs())
    del got
    row = torch.arange(8, device=DEV, dtype=torch.float32).bfloat16()       # broadcast of period 8
    got = ops.binary(abi.BINARY_ADD, x.view(-1, 8), row)
    assert torch.equal(got.view(-1)[probes].float(), (want + (probes % 8).float()).bfloat16().float())
    del got
    got = ops.cast(x, abi.BF16, abi.F32)                                    # 8 GiB written
    assert torch.equal(got[probes], want)
    del got
    condition = (torch.arange(count, device=DEV, dtype=torch.int64).remainder_(3) == 0).to(torch.uint8)
    got = ops.select(condition, x, ops.unary(abi.UNARY_NEG, x))
    assert torch.equal(got[probes].float(), torch.where(probes % 3 == 0, want, -want))

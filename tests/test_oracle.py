"""Pins the CPU checker (oracle/hyle_oracle.c) before anything trusts it.

Three anchors: (1) golden outputs produced by running the reference's own scalar floor
(tests/golden/ref_floor.npz, made by tests/golden/make_golden.py); (2) the reference floor itself,
live, where oracle/_ref was built; (3) known-answer vectors and independent formulas re-expressed
from the reference's tests.
"""
import math

import numpy as np
import pytest
import torch

from hyle_b200 import workloads as wl
from oracle import binding as ob


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32 if a.dtype == np.float32 else a.dtype)


def same_f32(a, b):
    """Bit equality, any NaN matching any NaN."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return np.array_equal(np.isnan(a), np.isnan(b)) and np.array_equal(bits(a)[~np.isnan(a)], bits(b)[~np.isnan(b)])


# ---- golden vectors from the reference's scalar floor ------------------------------------------------
def test_swiglu_matches_reference_golden(oracle, golden):
    out, _ = oracle.swiglu(golden["swiglu_gate"], golden["swiglu_up"])
    want = golden["swiglu_out"]
    nan = (want & 0x7FFF) > 0x7F80
    assert np.array_equal(nan, (out & 0x7FFF) > 0x7F80)
    assert np.array_equal(out[~nan], want[~nan])


def test_gated_activation_is_pinned_on_the_reference_floor(oracle, golden):
    """The general gating entry of the checker: its SiLU / bf16 form is the reference's swiglu_bf16 bit for
    bit; the GELU forms are the floor-pinned unary activations times up with one rounding; the rounded-gate
    form is Unary then Multiply."""
    from oracle import binding as ob

    gate, up = golden["swiglu_gate"], golden["swiglu_up"]
    want = golden["swiglu_out"]
    out, _ = oracle.gated_activation(0, ob.BF16, gate, up)
    nan = (want & 0x7FFF) > 0x7F80
    assert np.array_equal(out[~nan], want[~nan]) and np.array_equal(nan, (out & 0x7FFF) > 0x7F80)
    for activation, unary in ((0, ob.SILU), (1, ob.GELU), (2, ob.GELU_TANH)):
        for dtype in (ob.BF16, ob.F16):
            words = gate if dtype == ob.BF16 else (oracle.bf16_to_f32(gate).astype(np.float16).view(np.uint16))
            other = up if dtype == ob.BF16 else (oracle.bf16_to_f32(up).astype(np.float16).view(np.uint16))
            activated = oracle.unary(unary, dtype, words)
            two_steps = oracle.binary(ob.MULTIPLY, dtype, activated, other)
            fused, _ = oracle.gated_activation(activation, dtype, words, other, round_gate=True)
            both_nan = lambda w: (w & 0x7FFF) > (0x7F80 if dtype == ob.BF16 else 0x7C00)
            keep = ~both_nan(two_steps)
            assert np.array_equal(fused[keep], two_steps[keep]) and np.array_equal(both_nan(fused), ~keep)


@pytest.mark.parametrize("hidden", [1, 127, 128, 129, 257, 2048, 4096])
def test_rms_norm_matches_reference_golden(oracle, golden, hidden):
    x, w = golden[f"rms_x_{hidden}"], golden[f"rms_w_{hidden}"]
    assert np.array_equal(oracle.rms_norm(x, w, 1e-6)[0], golden[f"rms_y_{hidden}"])
    assert np.array_equal(oracle.rms_norm(x, None, 1e-6)[0], golden[f"rms_y_noweight_{hidden}"])


@pytest.mark.parametrize("cols", [1, 7, 1000])
def test_softmax_matches_reference_golden(oracle, golden, cols):
    x = golden[f"softmax_x_{cols}"]
    assert same_f32(oracle.softmax(x), golden[f"softmax_y_{cols}"])
    assert same_f32(oracle.softmax(x, log=True), golden[f"log_softmax_y_{cols}"])
    lse, probs, probs32, _, _ = oracle.logits_reduce(x)
    assert same_f32(probs32, golden[f"softmax_y_{cols}"])
    # the log-softmax shift is the log-sum-exp: x - lse == log_softmax
    valid = ~np.isnan(lse)
    assert same_f32((x[valid] - lse[valid, None]).astype(np.float32), golden[f"log_softmax_y_{cols}"][valid])


def test_argmax_matches_reference_golden(oracle, golden):
    index, value = oracle.argmax(golden["argmax_x"])
    assert np.array_equal(index, golden["argmax_index"])
    assert same_f32(value, golden["argmax_value"])
    # spot-check the rules the golden encodes
    assert list(index[:5]) == [int(np.argmax(golden["argmax_x"][0])), 17, 0, 0, 250]


# ---- live against the reference floor, larger seeded inputs --------------------------------------------
def test_oracle_equals_reference_floor_live(oracle, ref_floor):
    gate, up = wl.swiglu_inputs(8)
    assert np.array_equal(oracle.swiglu(gate, up)[0], ref_floor.swiglu(gate, up))
    x, _, w16, _ = wl.rms_norm_inputs(64)
    assert np.array_equal(oracle.rms_norm(x, w16, 1e-6)[0], ref_floor.rms_norm(x, w16, 1e-6))
    logits, tied = wl.logits_inputs(2, cols=151936)
    assert same_f32(oracle.softmax(logits), ref_floor.softmax(logits))
    assert same_f32(oracle.softmax(logits, log=True), ref_floor.softmax(logits, log=True))
    oi, ov = oracle.argmax(logits)
    ri, rv = ref_floor.argmax(logits)
    assert np.array_equal(oi, ri) and same_f32(ov, rv)
    assert tied, "workload 4 must contain a tied row"


def test_conversions_match_reference_floor(oracle, ref_floor):
    rng = np.random.default_rng(5)
    patterns = rng.integers(0, 2**32, 20000, dtype=np.uint64).astype(np.uint32)
    edge = np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001, 0x3F808000,
                     0x3F818000, 0x3F807FFF, 0x33000000, 0x33000001, 0x32FFFFFF, 0x387FC000, 0x477FF000,
                     0x477FEFFF, 0x00000001, 0x007FFFFF], dtype=np.uint32)
    for u in np.concatenate([patterns, edge]):
        f = np.array([u], np.uint32).view(np.float32)[0]
        assert oracle.lib.hyle_oracle_f32_to_bf16(f) == ref_floor.lib.hyle_ref_f32_to_bf16(f)
        assert oracle.lib.hyle_oracle_f32_to_f16(f) == ref_floor.lib.hyle_ref_f32_to_f16(f)
    for h in range(0, 65536, 7):
        a, b = oracle.lib.hyle_oracle_f16_to_f32(h), ref_floor.lib.hyle_ref_f16_to_f32(h)
        assert (math.isnan(a) and math.isnan(b)) or a == b


# ---- independent anchors for the storage conversions ------------------------------------------------------
def test_f16_conversions_against_numpy(oracle):
    halves = np.arange(65536, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32_scalar(int(h)) for h in halves], np.float32)
    assert same_f32(got, want)  # exhaustive, as tests/simd/dtype_test.cc:168-209
    rng = np.random.default_rng(11)
    values = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 100,
                             np.array([65504, 65519.99, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5,
                                       0.0, -0.0, np.inf, -np.inf], np.float32)])
    got = np.array([oracle.f32_to_f16_scalar(float(v)) for v in values], np.uint16)
    with np.errstate(over="ignore"):
        want = values.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_bf16_rounding_against_torch_and_numpy_helper(oracle):
    rng = np.random.default_rng(12)
    values = np.concatenate([rng.standard_normal(50000).astype(np.float32),
                             np.array([1.00390625, 1.01171875, 3.3895314e38, np.inf, -np.inf, 0.0, -0.0], np.float32)])
    want = torch.from_numpy(values).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16(values), want)
    assert np.array_equal(wl.f32_to_bf16(values), want)
    assert oracle.f32_to_bf16_scalar(float("nan")) & 0x7FC0 == 0x7FC0  # NaN stays a quiet NaN


# ---- Binary / Reduce rules ----------------------------------------------------------------------------------
def test_binary_broadcast_is_one_ieee_operation(oracle):
    a, bias = wl.broadcast_add_inputs(64, 256)
    assert np.array_equal(bits(oracle.binary(ob.ADD, ob.F32, a, bias)), bits(a + bias[None, :]))
    assert np.array_equal(bits(oracle.binary(ob.MULTIPLY, ob.F32, a, bias)), bits(a * bias[None, :]))
    x16, r16, _, _ = wl.rms_norm_inputs(4)
    want = wl.f32_to_bf16(wl.bf16_to_f32(x16) + wl.bf16_to_f32(r16))
    assert np.array_equal(oracle.binary(ob.ADD, ob.BF16, x16, r16), want)


def _number_extreme(a, b, minimum):
    """The formula the reference's own test checks simd::fmin / fmax against
    (tests/simd/ops_test.cc:424-444), re-expressed with numpy."""
    both_zero = (a == 0) & (b == 0)
    zero_bits = (a.view(np.uint32) | b.view(np.uint32)) if minimum else (a.view(np.uint32) & b.view(np.uint32))
    with np.errstate(invalid="ignore"):
        picked = np.where(a < b, a, b) if minimum else np.where(a > b, a, b)
    out = np.where(np.isnan(a), b, np.where(np.isnan(b), a, picked)).astype(np.float32)
    return np.where(both_zero, zero_bits.view(np.float32), out)


def test_binary_subtract_divide_and_number_extrema(oracle):
    rng = np.random.default_rng(11)
    special = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1.0, -1.0, 3.0e38, 1e-45], np.float32)
    a = np.concatenate([np.repeat(special, special.size), rng.standard_normal(1000).astype(np.float32)])
    b = np.concatenate([np.tile(special, special.size), rng.standard_normal(1000).astype(np.float32)])
    with np.errstate(all="ignore"):
        assert np.array_equal(bits(oracle.binary(ob.SUBTRACT, ob.F32, a, b)), bits(a - b))
        got, want = oracle.binary(ob.DIVIDE, ob.F32, a, b), a / b
        assert np.array_equal(np.isnan(got), np.isnan(want))  # the sign of a produced NaN is not specified
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)])
    for kind, minimum in ((ob.NUMBER_MINIMUM, True), (ob.NUMBER_MAXIMUM, False)):
        got, want = oracle.binary(kind, ob.F32, a, b), _number_extreme(a, b, minimum)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)])
    # operand order does not decide the sign of a zero
    z = oracle.binary(ob.NUMBER_MINIMUM, ob.F32, np.array([0.0, -0.0], np.float32), np.array([-0.0, 0.0], np.float32))
    assert np.all(np.signbit(z))
    z = oracle.binary(ob.NUMBER_MAXIMUM, ob.F32, np.array([0.0, -0.0], np.float32), np.array([-0.0, 0.0], np.float32))
    assert not np.any(np.signbit(z))
    # half types: f32 operation, one rounding
    x16, r16, _, _ = wl.rms_norm_inputs(4)
    with np.errstate(all="ignore"):
        want = wl.f32_to_bf16(wl.bf16_to_f32(x16) / wl.bf16_to_f32(r16))
    assert np.array_equal(oracle.binary(ob.DIVIDE, ob.BF16, x16, r16), want)


# ---- Cast ----------------------------------------------------------------------------------------------------------------------
def _fp8_probe_values():
    """Every f16 value (covers both 8-bit formats' ranges, ties and subnormals densely) plus wide f32 values."""
    with np.errstate(all="ignore"):
        half = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    rng = np.random.default_rng(23)
    wide = (rng.standard_normal(4096) * np.exp(rng.uniform(-30, 30, 4096))).astype(np.float32)
    edge = np.array([448.0, 449.0, 464.0, 465.0, 480.0, 57344.0, 61440.0, 65536.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10,
                     2.0 ** -16, 2.0 ** -17, 3.0e38, -3.0e38, np.inf, -np.inf, np.nan, -np.nan], np.float32)
    return np.concatenate([half, wide, edge])


def test_fp8_conversions_match_reference(oracle, ref_floor, golden):
    values = _fp8_probe_values()
    for name in ("e4m3", "e5m2"):
        encode_o, encode_r = getattr(oracle.lib, f"hyle_oracle_f32_to_{name}"), getattr(ref_floor.lib, f"hyle_ref_f32_to_{name}")
        decode_o, decode_r = getattr(oracle.lib, f"hyle_oracle_{name}_to_f32"), getattr(ref_floor.lib, f"hyle_ref_{name}_to_f32")
        for v in values[::7]:
            assert encode_o(float(v)) == encode_r(float(v)), (name, v)
        for code in range(256):
            a, b = decode_o(code), decode_r(code)
            assert (np.isnan(a) and np.isnan(b)) or np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32), (name, code)


def test_fp8_conversions_match_golden(oracle, golden):
    values = golden["fp8_values"]
    for name in ("e4m3", "e5m2"):
        encode = getattr(oracle.lib, f"hyle_oracle_f32_to_{name}")
        assert [encode(float(v)) for v in values] == list(golden[f"fp8_{name}_codes"])
        decode = getattr(oracle.lib, f"hyle_oracle_{name}_to_f32")
        got = np.array([decode(c) for c in range(256)], np.float32)
        want = golden[f"fp8_{name}_decoded"]
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)])


def test_cast_rules(oracle):
    # the largest normal saturates, the tie below it rounds to even, infinity saturates in E4M3
    e4 = oracle.cast(ob.F32, ob.E4M3, np.array([448.0, 1e9, np.inf, -np.inf, 464.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, np.nan], np.float32))
    # 2^-9 is the smallest subnormal; 2^-10 is the tie between it and zero and goes to the even one (zero)
    assert list(e4[:8]) == [0x7E, 0x7E, 0x7E, 0xFE, 0x7E, 0x01, 0x00, 0x01] and e4[8] & 0x7F == 0x7F
    # bool is truth of the storage bits; i32 rounds to nearest even
    x = np.array([0.0, -0.0, 1e-45, np.nan, -3.0], np.float32)
    assert list(oracle.cast(ob.F32, ob.BOOL, x)) == [0, 0, 1, 1, 1]
    assert list(oracle.cast(ob.BOOL, ob.F32, np.array([0, 1, 7, 255], np.uint8))) == [0.0, 1.0, 1.0, 1.0]
    ints = np.array([0, 1, -1, 16777217, 16777219, -16777217, 2147483647, -2147483648], np.int32)
    assert np.array_equal(oracle.cast(ob.I32, ob.F32, ints), ints.astype(np.float32))
    # wide pairs go through f32 with one rounding
    h = np.arange(0, 65536, 3, dtype=np.uint16)
    with np.errstate(all="ignore"):
        want = wl.f32_to_bf16(h.view(np.float16).astype(np.float32))
    got = oracle.cast(ob.F16, ob.BF16, h)
    nan = (want & 0x7FFF) > 0x7F80
    assert np.array_equal(got[~nan], want[~nan]) and np.all((got[nan] & 0x7FFF) > 0x7F80)
    with pytest.raises(ValueError):
        oracle.cast(ob.E5M2, ob.F32, np.zeros(4, np.uint8))  # not a pair of the CPU route


def test_fp8_cache_encode_rules(oracle, ref_floor):
    """value / scale, then the reference's own E4M3 conversion; non-finite inputs give byte 0 and the status bit."""
    rng = np.random.default_rng(31)
    x = (rng.standard_normal(4096) * 30).astype(np.float32)
    codes, status = oracle.fp8_e4m3_encode(ob.F32, x, 0.25)
    assert status == 0
    encode = ref_floor.lib.hyle_ref_f32_to_e4m3
    assert list(codes[:512]) == [encode(float(np.float32(v) / np.float32(0.25))) for v in x[:512]]
    x[5], x[9] = np.nan, -np.inf
    codes, status = oracle.fp8_e4m3_encode(ob.F32, x, 0.25)
    assert status == 4 and codes[5] == 0 and codes[9] == 0


def test_masked_scaled_softmax_rules(oracle):
    rng = np.random.default_rng(12)
    x = (3.0 * rng.standard_normal((2, 5, 64))).astype(np.float16)
    mask = np.ones((5, 64), np.uint8); mask[1, 10:] = 0; mask[2, :] = 0; mask[3, 7] = 0
    words, values = oracle.masked_softmax_f16(x.view(np.uint16), mask[None], 0.25)
    assert np.all(values[:, 1, 10:] == 0) and np.allclose(values[:, 1].sum(axis=-1), 1.0, atol=1e-6)
    assert np.all(np.isnan(values[:, 2]))                       # every element masked: the row is invalid
    assert np.all(values[:, 3, 7] == 0)
    ref = np.exp(0.25 * x[0, 0].astype(np.float64)); ref /= ref.sum()
    assert np.allclose(values[0, 0], ref, rtol=1e-5)
    assert np.array_equal(words, values.astype(np.float16).view(np.uint16)) or np.isnan(values).any()
    # additive form: 0 / -inf addends reproduce the Boolean mask exactly, a finite addend biases the score
    addend = np.where(mask != 0, np.float16(0), np.float16(-np.inf)).astype(np.float16)
    words_add, values_add = oracle.masked_softmax_f16(x.view(np.uint16), addend[None], 0.25)
    assert np.array_equal(words_add, words)
    addend[0, 3] = 1.5
    _, biased = oracle.masked_softmax_f16(x.view(np.uint16), addend[None], 0.25)
    z = 0.25 * x[0, 0].astype(np.float64); z[3] += 1.5
    ref = np.exp(z - z.max()); ref /= ref.sum()
    assert np.allclose(biased[0, 0], ref, rtol=1e-5)


# ---- sampling ----------------------------------------------------------------------------------------------------------------
def test_random_bits_match_reference_generator(oracle, golden):
    identities = golden["random_identities"]
    assert np.array_equal(oracle.random_bits(identities, 40), golden["random_words"])
    assert np.array_equal(oracle.random_bits(identities, 37), golden["random_words"][:, :37])   # ragged last block
    from oracle.binding import RefFloor
    if RefFloor.available():
        ref = RefFloor()
        rng = np.random.default_rng(3)
        more = rng.integers(0, 2 ** 32, (16, 4), dtype=np.uint64).astype(np.uint32)
        got = oracle.random_bits(more, 24)
        want = np.array([[ref.lib.hyle_ref_random_word(row.ctypes.data, w) for w in range(24)]
                         for row in np.ascontiguousarray(more)], np.uint32)
        assert np.array_equal(got, want)


def test_categorical_rules(oracle):
    rng = np.random.default_rng(8)
    rows, cols = 64, 1000
    x = (3.0 * rng.standard_normal((rows, cols))).astype(np.float32)
    x[3, 10:] = -np.inf                       # mass on the first ten entries only
    x[4, :] = -np.inf; x[4, 777] = 0.0       # a single entry with mass
    identities = rng.integers(0, 2 ** 32, (rows, 4), dtype=np.uint64).astype(np.uint32)
    index, logp, uniform, invalid = oracle.categorical(ob.F32, x, identities)
    assert invalid == 0 and index[4] == 777 and abs(logp[4]) < 1e-6 and 0 <= index[3] < 10
    assert np.all((uniform > 0) & (uniform < 1))
    # the draw inverts the cumulative distribution at the row's uniform
    w = np.exp((x - x.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float64)
    c = np.cumsum(w, axis=1)
    for r in range(rows):
        t = c[r, -1] * uniform[r]
        assert c[r, index[r]] > t * (1 - 1e-12) and (index[r] == 0 or c[r, index[r] - 1] <= t * (1 + 1e-12))
        assert abs(logp[r] - (x[r, index[r]] - x[r].max() - np.log(c[r, -1]))) < 1e-5
    # the same identity and row give the same draw wherever the row sits
    perm = rng.permutation(rows)
    index_p, _, _, _ = oracle.categorical(ob.F32, x[perm], identities[perm])
    assert np.array_equal(index_p, index[perm])
    # rejected rows
    bad = x[:4].copy(); bad[0, 5] = np.nan; bad[1, 6] = np.inf; bad[2, :] = -np.inf
    index_b, _, _, invalid = oracle.categorical(ob.F32, bad, identities[:4])
    assert invalid == 3 and list(index_b[:3]) == [-1, -1, -1] and index_b[3] >= 0


def _unary_inputs():
    rng = np.random.default_rng(17)
    special = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1.0, -1.0, 20.0, 20.5, -20.0, 88.0, 89.0, -104.0,
                        1e-40, -1e-40, 3.0e38, 0.5, 7.0, -7.0], np.float32)
    return np.concatenate([special, (4.0 * rng.standard_normal(4096)).astype(np.float32),
                           rng.uniform(-30, 30, 2048).astype(np.float32)])


def test_unary_activations_match_reference_floor(oracle, ref_floor):
    """sigmoid, relu, gelu, gelu_tanh, silu: the restatement equals the reference's scalar floor bit for bit."""
    x = _unary_inputs()
    for kind in (ob.SIGMOID, ob.RELU, ob.GELU, ob.GELU_TANH, ob.SILU):
        got, want = oracle.unary(kind, ob.F32, x), ref_floor.activation(kind, x)
        assert np.array_equal(np.isnan(got), np.isnan(want)), kind
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)]), kind


@pytest.mark.parametrize("hidden", [1, 7, 129, 2048, 4100])
def test_layer_norm_matches_reference_floor_and_golden(oracle, golden, hidden, request):
    x, scale, bias = golden[f"layer_x_{hidden}"], golden[f"layer_scale_{hidden}"], golden[f"layer_bias_{hidden}"]
    assert np.array_equal(oracle.layer_norm(x, scale, bias, 1e-5)[0], golden[f"layer_y_{hidden}"])
    assert np.array_equal(oracle.layer_norm(x, None, None, 1e-5)[0], golden[f"layer_y_plain_{hidden}"])
    from oracle.binding import RefFloor
    if RefFloor.available():
        ref = request.getfixturevalue("ref_floor")
        assert np.array_equal(oracle.layer_norm(x, scale, bias, 1e-5)[0], ref.layer_norm(x, scale, bias, 1e-5))


def test_unary_activations_match_golden(oracle, golden):
    """The same pin from the committed vectors, for machines without the reference tree."""
    x = golden["unary_x"]
    for kind in (ob.SIGMOID, ob.RELU, ob.GELU, ob.GELU_TANH, ob.SILU):
        got, want = oracle.unary(kind, ob.F32, x), golden[f"unary_y_{kind}"]
        assert np.array_equal(np.isnan(got), np.isnan(want)), kind
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)]), kind


def test_unary_rules(oracle):
    x = _unary_inputs()
    with np.errstate(all="ignore"):
        assert np.array_equal(bits(oracle.unary(ob.ABS, ob.F32, x)), bits(np.abs(x)))
        assert np.array_equal(bits(oracle.unary(ob.NEG, ob.F32, x)), bits(-x))
        got, want = oracle.unary(ob.SQRT, ob.F32, x), np.sqrt(x)
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)])
        got, want = oracle.unary(ob.RSQRT, ob.F32, x), np.float32(1.0) / np.sqrt(x)
        assert np.array_equal(bits(got)[~np.isnan(want)], bits(want)[~np.isnan(want)])
        for kind, fn in ((ob.EXP, np.exp), (ob.LOG, np.log), (ob.TANH, np.tanh)):
            got, want = oracle.unary(kind, ob.F32, x), fn(x.astype(np.float64))
            ok = np.isfinite(want) & (np.abs(want) < 3.0e38)
            assert np.array_equal(np.isnan(got), np.isnan(want))
            assert np.all(np.abs(got[ok] - want[ok]) <= 2e-7 * np.abs(want[ok]) + 2e-45)  # + half a subnormal step
    # the special values the operator schema spells out (include/hyle/compute/operation.h:70-72)
    sp = oracle.unary(ob.SOFTPLUS, ob.F32, np.array([-np.inf, np.nan, 100.0, 0.0], np.float32))
    assert sp[0] == 0.0 and not np.signbit(sp[0]) and np.isnan(sp[1]) and sp[2] == 100.0
    assert abs(sp[3] - np.log(2.0)) < 1e-7
    for kind in (ob.GELU, ob.GELU_TANH, ob.SILU):
        assert oracle.unary(kind, ob.F32, np.array([-np.inf], np.float32))[0] == 0.0
    assert np.isnan(oracle.unary(ob.RELU, ob.F32, np.array([np.nan], np.float32))[0])
    # 16-bit storage: f32 value, one rounding
    x16 = wl.f32_to_bf16(x)
    with np.errstate(all="ignore"):
        want = wl.f32_to_bf16(np.tanh(wl.bf16_to_f32(x16).astype(np.float64)).astype(np.float32))
    got = oracle.unary(ob.TANH, ob.BF16, x16)
    nan = (want & 0x7FFF) > 0x7F80
    assert np.all(np.abs(got[~nan].astype(np.int32) - want[~nan].astype(np.int32)) <= 1)


def test_reduce_rules_nan_zero_empty(oracle):
    # docs/user/compute.md:384-388 and tests/compute_provider_native/reduction_test.cc:130-222,330-398
    x = np.array([[1.0, np.nan, 3.0], [-0.0, 0.0, -0.0], [-0.0, -0.0, -0.0], [-1.0, -2.0, -np.inf],
                  [np.inf, 1.0, 2.0]], np.float32)
    mx, mn = oracle.reduce_rows(ob.MAXIMUM, x), oracle.reduce_rows(ob.MINIMUM, x)
    assert np.isnan(mx[0]) and np.isnan(mn[0])
    assert mx[1] == 0 and not np.signbit(mx[1]) and mn[1] == 0 and np.signbit(mn[1])
    assert np.signbit(mx[2]) and np.signbit(mn[2])
    assert mx[3] == -1.0 and mn[3] == -np.inf and mx[4] == np.inf
    empty = np.zeros((3, 0), np.float32)
    assert np.array_equal(oracle.reduce_rows(ob.SUM, empty), np.zeros(3, np.float32))
    assert np.all(np.isnan(oracle.reduce_rows(ob.MEAN, empty)))
    assert np.all(oracle.reduce_rows(ob.MINIMUM, empty) == np.inf)
    assert np.all(oracle.reduce_rows(ob.MAXIMUM, empty) == -np.inf)
    a, bias = wl.broadcast_add_inputs(16, 4096)
    c = a + bias
    s64, abs64 = oracle.row_sum_f64(c)
    assert np.all(np.abs(oracle.reduce_rows(ob.SUM, c) - s64) <= 1e-5 * abs64)


# ---- Q8_0 known answers (tests/compute_provider_ggml/native_paged_test.cc:255-348) ------------------------------
def _q8_expected(values_f32):
    """The independent formula of the reference test, in numpy, block by block."""
    values = np.asarray(values_f32, np.float32)
    out = np.zeros(values.size // 32 * 34, np.uint8)
    for b in range(values.size // 32):
        block = values[b * 32:(b + 1) * 32]
        scale = np.float32(np.max(np.abs(block))) / np.float32(127.0)
        stored = np.float32(scale).astype(np.float16).view(np.uint16)
        if stored == 0:
            continue
        out[b * 34] = stored & 0xFF
        out[b * 34 + 1] = stored >> 8
        inverse = np.float32(1.0) / scale
        prod = (block * inverse).astype(np.float32)
        # np.round is half-to-even; the reference uses std::round (half away from zero)
        exact_half = np.abs(prod - np.trunc(prod)) == 0.5
        codes = np.where(exact_half, np.trunc(prod) + np.sign(prod), np.round(prod))
        out[b * 34 + 2:b * 34 + 34] = codes.astype(np.int8).view(np.uint8)
    return out


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_q8_reference_bytes_ties_zero_and_three_input_types(oracle, dtype):
    values = np.array([float(int(i % 23) - 11) * 0.03125 for i in range(256)], np.float32)
    values[:5] = [127.0, 0.5, 1.5, -0.5, -1.5]
    values[32:64] = 0.0
    if dtype == "f32":
        payload, kind, rounded = values, ob.F32, values
    elif dtype == "bf16":
        payload, kind = wl.f32_to_bf16(values), ob.BF16
        rounded = wl.bf16_to_f32(payload)
    else:
        payload, kind = values.astype(np.float16).view(np.uint16), ob.F16
        rounded = values.astype(np.float16).astype(np.float32)
    got, invalid = oracle.q8_0_encode(kind, payload)
    assert not invalid and got.size == 8 * 34
    assert np.array_equal(got, _q8_expected(rounded))
    assert got[3] == 1 and got[4] == 2 and got[5].view(np.int8) == -1  # 0.5 -> 1, 1.5 -> 2, -0.5 -> -1
    assert np.all(got[34:68] == 0)  # the all-zero block is 34 zero bytes


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_q8_scale_boundaries_have_canonical_zero_blocks(oracle, dtype):
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
    if dtype == "f32":
        payload, kind, rounded = values, ob.F32, values
    elif dtype == "bf16":
        payload, kind = wl.f32_to_bf16(values), ob.BF16
        rounded = wl.bf16_to_f32(payload)
    else:
        payload, kind = values.astype(np.float16).view(np.uint16), ob.F16
        rounded = values.astype(np.float16).astype(np.float32)
    got, invalid = oracle.q8_0_encode(kind, payload)
    assert not invalid
    want = _q8_expected(rounded)
    assert np.array_equal(got, want)
    scales = want.reshape(-1, 34)[:, :2].view(np.uint16).ravel()
    assert np.any(scales == 0) and np.any(scales != 0)
    codes = want.reshape(-1, 34)[:, 2:].view(np.int8)
    assert codes.min() >= -127 and codes.max() <= 127


def test_q8_invalid_payload_is_flagged_and_zeroed(oracle):
    for bad in (np.nan, np.inf):
        values = np.ones(64, np.float32)
        values[19] = bad
        got, invalid = oracle.q8_0_encode(ob.F32, values)
        assert invalid and np.all(got[:34] == 0) and np.any(got[34:] != 0)
    got, invalid = oracle.q8_0_encode(ob.F32, np.full(64, 9000000.0, np.float32))
    assert invalid and np.all(got == 0)
    # bf16 threshold: the largest bf16 not above 65504*127 is accepted, the next one is not
    limit16 = np.array([0x4AFD, 0x4AFE], np.uint16)
    for word, expect in zip(limit16, (False, True)):
        payload = np.zeros(32, np.uint16)
        payload[7] = word
        assert oracle.q8_0_encode(ob.BF16, payload)[1] == expect


def test_q8_decode_is_exact_product_then_rne(oracle):
    w = wl.q8_sweep_inputs(4)
    blocks, _ = oracle.q8_0_encode(ob.BF16, w)
    decoded = oracle.q8_0_decode(blocks, w.size)
    b = blocks.reshape(-1, 34)
    scale = b[:, :2].copy().view(np.float16).astype(np.float32)
    want = wl.f32_to_bf16((scale * b[:, 2:].view(np.int8).astype(np.float32)).astype(np.float32))
    assert np.array_equal(decoded, want.ravel())
    # the round trip stays within half a quantisation step (+ one bf16 rounding) of the input
    x = wl.bf16_to_f32(w).reshape(-1, 32)
    err = np.abs(wl.bf16_to_f32(decoded).reshape(-1, 32) - x)
    assert np.all(err <= 0.5 * scale * (1 + 2 ** -10) + np.abs(x) * 2 ** -8 + 1e-12)
    blocks2, decoded2, total, invalid = oracle.q8_0_roundtrip(w)
    assert np.array_equal(blocks2, blocks) and np.array_equal(decoded2, decoded) and not invalid
    assert total == pytest.approx(float(np.sum(wl.bf16_to_f32(w).astype(np.float64) ** 2)), rel=1e-12)

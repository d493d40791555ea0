"""Generate tests/golden/ref_floor.npz by RUNNING the reference's own scalar floor.

Needs oracle/_ref/libhyle_ref_floor.so, i.e. the reference tree mounted (at $HYLE_REF) when
`make -C oracle` ran.  The fixture travels with the repository, so the oracle stays pinned to the
reference's outputs where the reference tree is absent.  Inputs are seeded; special values follow
the edge cases of the reference's tests (tests/simd/math_test.cc:1317-1331 invalid softmax rows,
tests/compute_provider_native/matmul_gated_test.cc:360-372 gate specials,
tests/simd/search_test.cc:157-194,269-279 argmax ties and NaN).

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from hyle_b200.workloads import f32_to_bf16  # noqa: E402
from oracle.binding import RefFloor  # noqa: E402


def main():
    ref = RefFloor()
    ref.set_threads(1)
    rng = np.random.default_rng(20261125)
    out = {}

    # SwiGLU: random values plus specials in the gate and in the up operand.
    specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 80.0, -80.0, 1e-30, -1e-30, 88.7, -88.7,
                         1.0, -1.0, 0.5, -0.5, 20.0, -20.0], dtype=np.float32)
    gate = (1.5 * rng.standard_normal((3, 257))).astype(np.float32)
    up = (1.5 * rng.standard_normal((3, 257))).astype(np.float32)
    gate[0, : specials.size] = specials
    up[1, : specials.size] = specials
    gate[2, : specials.size] = specials
    up[2, : specials.size] = specials[::-1]
    out["swiglu_gate"], out["swiglu_up"] = f32_to_bf16(gate), f32_to_bf16(up)
    out["swiglu_out"] = ref.swiglu(out["swiglu_gate"], out["swiglu_up"])

    # RMSNorm: the hidden sizes the reference's tests use (tests/compute_provider_native/
    # normalization_test.cc:168-323), bf16 weight, eps 1e-6.
    for hidden in (1, 127, 128, 129, 257, 2048, 4096):
        x = f32_to_bf16(rng.standard_normal((2, hidden)).astype(np.float32))
        w = f32_to_bf16(rng.uniform(0.5, 1.5, hidden).astype(np.float32))
        out[f"rms_x_{hidden}"], out[f"rms_w_{hidden}"] = x, w
        out[f"rms_y_{hidden}"] = ref.rms_norm(x, w, 1e-6)
        out[f"rms_y_noweight_{hidden}"] = ref.rms_norm(x, None, 1e-6)

    # Softmax / log-softmax: ordinary rows, wide-range rows, and the invalid rows (NaN, +inf, all -inf).
    for cols in (1, 7, 1000):
        x = (4.0 * rng.standard_normal((6, cols))).astype(np.float32)
        x[1] *= 20.0
        if cols >= 7:
            x[2, 3] = np.nan
            x[3, 5] = np.inf
            x[4, :] = -np.inf
            x[5, 0] = -np.inf
        out[f"softmax_x_{cols}"] = x
        out[f"softmax_y_{cols}"] = ref.softmax(x)
        out[f"log_softmax_y_{cols}"] = ref.softmax(x, log=True)

    # Argmax: ties (first wins), -0/+0, NaN first / last / everywhere, all -inf.
    rows = np.zeros((10, 300), dtype=np.float32)
    rows[0] = rng.standard_normal(300)
    rows[1] = rows[0]; rows[1, 17] = rows[1, 200] = rows[1].max() + 1
    rows[2] = -0.0; rows[2, 5] = 0.0
    rows[3] = np.nan
    rows[4] = np.nan; rows[4, 250] = -np.inf; rows[4, 260] = -np.inf
    rows[5] = rng.standard_normal(300); rows[5, 0] = np.nan
    rows[6] = rng.standard_normal(300); rows[6, 299] = np.nan; rows[6, 100] = np.inf; rows[6, 150] = np.inf
    rows[7] = -np.inf
    rows[8] = 3.0
    rows[9] = rng.standard_normal(300); rows[9, 299] = 100.0
    index, value = ref.argmax(rows)
    out["argmax_x"], out["argmax_index"], out["argmax_value"] = rows, index, value

    # LayerNorm: bf16, eps 1e-5, with and without scale and bias; rows with a large common offset.
    for hidden in (1, 7, 129, 2048, 4100):
        x = f32_to_bf16((3.0 * rng.standard_normal((3, hidden)) + np.array([[0.0], [5.0], [-40.0]])).astype(np.float32))
        scale = f32_to_bf16(rng.uniform(0.5, 1.5, hidden).astype(np.float32))
        bias = f32_to_bf16(rng.standard_normal(hidden).astype(np.float32))
        out[f"layer_x_{hidden}"], out[f"layer_scale_{hidden}"], out[f"layer_bias_{hidden}"] = x, scale, bias
        out[f"layer_y_{hidden}"] = ref.layer_norm(x, scale, bias, 1e-5)
        out[f"layer_y_plain_{hidden}"] = ref.layer_norm(x, None, None, 1e-5)

    # The 8-bit floating formats: every code decoded, and a spread of values encoded.
    with np.errstate(all="ignore"):
        half = np.arange(0, 65536, 5, dtype=np.uint16).view(np.float16).astype(np.float32)
    edge = np.array([448.0, 449.0, 464.0, 465.0, 480.0, 57344.0, 61440.0, 65536.0, 2.0 ** -9, 2.0 ** -10,
                     1.5 * 2.0 ** -10, 2.0 ** -16, 2.0 ** -17, 3.0e38, -3.0e38, np.inf, -np.inf, np.nan], np.float32)
    values = np.concatenate([half, edge])
    out["fp8_values"] = values
    for name in ("e4m3", "e5m2"):
        encode = getattr(ref.lib, f"hyle_ref_f32_to_{name}")
        decode = getattr(ref.lib, f"hyle_ref_{name}_to_f32")
        out[f"fp8_{name}_codes"] = np.array([encode(float(v)) for v in values], np.uint8)
        out[f"fp8_{name}_decoded"] = np.array([decode(c) for c in range(256)], np.float32)

    # The counter generator behind RandomBits: words 0..39 of a few identities.
    identities = np.array([[0, 0, 0, 0], [1, 2, 3, 4], [0xFFFFFFFF] * 4, [0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344],
                           [7, 0, 0xDEADBEEF, 5]], dtype=np.uint32)
    out["random_identities"] = identities
    out["random_words"] = np.array([[ref.lib.hyle_ref_random_word(row.ctypes.data, w) for w in range(40)]
                                    for row in np.ascontiguousarray(identities)], np.uint32)
    high = 4 * ((1 << 32) + 5)  # a counter above 2^32: both counter words in use
    out["random_words_high"] = np.array([ref.lib.hyle_ref_random_word(row.ctypes.data, high + 1)
                                         for row in np.ascontiguousarray(identities)], np.uint32)

    # Unary activations of the scalar floor (UnaryKind numbers): sigmoid 7, relu 8, gelu 9,
    # gelu_tanh 10, silu 11, on specials and a spread of ordinary values.
    special = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1.0, -1.0, 20.0, -20.0, 88.0, -104.0, 1e-40, -1e-40,
                        3.0e38, 0.5, 7.0, -7.0], dtype=np.float32)
    x = np.concatenate([special, (4.0 * rng.standard_normal(1000)).astype(np.float32)])
    out["unary_x"] = x
    for kind in (7, 8, 9, 10, 11):
        out[f"unary_y_{kind}"] = ref.activation(kind, x)

    path = os.path.join(ROOT, "tests", "golden", "ref_floor.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

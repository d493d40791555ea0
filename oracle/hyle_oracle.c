/*
 * CPU restatement of HYLE's elementwise / broadcast / reduction operators -- TEST INFRASTRUCTURE.
 *
 * This file is the checker for the CUDA kernels: only the tests, the smoke check and the CPU
 * baseline leg of the benchmark may load it.  Nothing in the product path calls it.
 *
 * Every function restates, in plain scalar C, what the reference computes on its CPU route; the
 * file:line beside each one is the reference source it follows (paths inside kiroeko/hyle).
 * Third-party arithmetic that is not in the reference tree: Q8_0 row quantisation lives in ggml
 * (module ggml_cpu, pinned at ggml-cpu-snapshot-ffa4e8b80930, called from
 * src/compute_provider_ggml/ggml_cpu_provider.cc:598,613); its published reference algorithm
 * (amax, d = amax/127, id = 1/d, roundf(x*id), f16 scale) is restated here and pinned by the
 * independent formula in tests/compute_provider_ggml/native_paged_test.cc:255-326.
 *
 * Parity status: pinned.  tests/test_oracle.py checks these functions against the reference's
 * own scalar floor compiled from the reference tree (oracle/_ref/libhyle_ref_floor.so, built by
 * oracle/Makefile) and against known-answer vectors re-expressed from the reference's tests.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC  (no -ffast-math: results are compared
 * bit for bit).  Row loops are split over threads in contiguous ranges, the way the reference's
 * parallel_for_ranges does (src/compute_provider_native/native_plan.h:94-111).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };
enum { BIN_ADD = 0, BIN_MUL = 1, BIN_SUB = 2, BIN_DIV = 3, BIN_MIN = 4, BIN_MAX = 5 };
enum { RED_SUM = 0, RED_MEAN = 1, RED_MIN = 2, RED_MAX = 3 };
enum { SM_SOFTMAX = 0, SM_LOG_SOFTMAX = 1 };

ORACLE_API void hyle_oracle_set_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
}

ORACLE_API int hyle_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- storage conversions: include/hyle/simd/dtype.h:55-121 ----------------------------------- */
static inline float bits_to_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* dtype.h:105-107 */
ORACLE_API float hyle_oracle_bf16_to_f32(uint16_t b) { return bits_to_f32((uint32_t)b << 16); }

/* dtype.h:114-121: RNE; inf/NaN are not incremented; NaN gets its quiet bit. */
ORACLE_API uint16_t hyle_oracle_f32_to_bf16(float f) {
  const uint32_t u = f32_to_bits(f);
  const uint32_t a = u & 0x7fffffffu;
  const uint32_t incr = a < 0x7f800000u ? 0x7fffu + ((u >> 16) & 1u) : 0u;
  const uint32_t snan = a > 0x7f800000u ? (1u << 6) : 0u;
  return (uint16_t)(snan | ((u + incr) >> 16));
}

/* dtype.h:55-68 */
ORACLE_API float hyle_oracle_f16_to_f32(uint16_t h) {
  const uint32_t sign = h >> 15, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  if (e == 0) {
    const float sub = (1.0f / 16384) * ((float)m * (1.0f / 1024));
    return sign ? -sub : sub;
  }
  const uint32_t e32 = e == 31 ? 0xff : e + (127 - 15);
  return bits_to_f32((sign << 31) | (e32 << 23) | (m << 13));
}

/* dtype.h:73-101: RNE, overflow to inf, gradual underflow, NaN -> mantissa 0x3ff. */
ORACLE_API uint16_t hyle_oracle_f32_to_f16(float f) {
  const uint32_t b = f32_to_bits(f);
  const uint32_t sign = b >> 31, e32 = (b >> 23) & 0xff, m32 = b & 0x7fffffu;
  int idx = 126 - (int)e32;
  idx = idx < 13 ? 13 : (idx > 24 ? 24 : idx);
  const uint32_t odd = ((m32 | 0x800000u) >> idx) & 1u;
  const uint32_t rounded = m32 + odd + (1u << (idx - 1)) - 1u;
  const int carry = rounded >= (1u << 23);
  const int e = (int)e32 - 127 + carry;
  if (e < -24) return (uint16_t)(sign << 15);
  const int is_nan = e32 == 255 && m32 != 0;
  const int overflow = e >= 16;
  int be = e + 15;
  be = be < 0 ? 0 : (be > 31 ? 31 : be);
  const int sub = (-14 - e) > 0 ? (-14 - e) : 0;
  const uint32_t shifted = (rounded & 0x7fffffu) >> (13 + sub);
  const uint32_t leading = sub == 0 ? 0u : (1024u >> sub);
  const uint32_t m16 = is_nan ? 0x3ffu : (overflow ? 0u : leading + shifted);
  return (uint16_t)((sign << 15) | ((uint32_t)be << 10) | m16);
}

static inline float load_as_f32(const void *p, size_t i, int dtype) {
  if (dtype == DT_F32) return ((const float *)p)[i];
  if (dtype == DT_BF16) return hyle_oracle_bf16_to_f32(((const uint16_t *)p)[i]);
  return hyle_oracle_f16_to_f32(((const uint16_t *)p)[i]);
}
static inline void store_from_f32(void *p, size_t i, int dtype, float v) {
  if (dtype == DT_F32) ((float *)p)[i] = v;
  else if (dtype == DT_BF16) ((uint16_t *)p)[i] = hyle_oracle_f32_to_bf16(v);
  else ((uint16_t *)p)[i] = hyle_oracle_f32_to_f16(v);
}

/* ---- Binary{all six kinds}, trailing-axis broadcast ---------------------------------------------
 * src/compute_provider_native/elementwise.cc:101-133 (dense f32 route, one IEEE op per element),
 * :135-147 (half types: f32 op on 128-element tiles, one rounding), :333-348,540-571 (one dense
 * call per broadcast chunk = rhs repeats with period rhs_period).
 * Minimum / Maximum are "number" extrema (include/hyle/simd/ops.h:77-79): one NaN operand gives the
 * other operand, two zeros give OR (minimum) / AND (maximum) of their bits, so the sign does not
 * depend on operand order (src/simd/ops/kernel_impl.h:256-267). */
static inline float binary_value(int kind, float a, float b) {
  switch (kind) {
    case BIN_ADD: return a + b;
    case BIN_MUL: return a * b;
    case BIN_SUB: return a - b;
    case BIN_DIV: return a / b;
    default: break;
  }
  if (isnan(a)) return b;  /* NaN if b is NaN too */
  if (isnan(b)) return a;
  if (a == 0.0f && b == 0.0f) {
    uint32_t x, y;
    memcpy(&x, &a, 4);
    memcpy(&y, &b, 4);
    x = kind == BIN_MIN ? (x | y) : (x & y);
    memcpy(&a, &x, 4);
    return a;
  }
  if (kind == BIN_MIN) return a < b ? a : b;
  return a > b ? a : b;
}

ORACLE_API void hyle_oracle_binary(int kind, int dtype, const void *lhs, const void *rhs, void *out,
                                   uint64_t count, uint64_t rhs_period) {
  if (count == 0) return;
  const uint64_t chunks = count / rhs_period;
  /* Threads split the rows of a broadcast, or the elements when the operands have one shape: either
   * way contiguous ranges, as the reference's parallel_for_ranges hands them out. */
  if (chunks == 1) {
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < count; ++i)
      store_from_f32(out, i, dtype, binary_value(kind, load_as_f32(lhs, i, dtype), load_as_f32(rhs, i, dtype)));
    return;
  }
#pragma omp parallel for schedule(static)
  for (uint64_t c = 0; c < chunks; ++c) {
    for (uint64_t j = 0; j < rhs_period; ++j) {
      const uint64_t i = c * rhs_period + j;
      const float a = load_as_f32(lhs, i, dtype), b = load_as_f32(rhs, j, dtype);
      store_from_f32(out, i, dtype, binary_value(kind, a, b));
    }
  }
}

/* ---- Reduce over the last axis ----------------------------------------------------------------
 * Extrema: src/compute_provider_native/reduction.cc:22-47 (identities, NaN propagation, fmax/fmin
 * otherwise) with the public zero rule of src/compute_provider_native/aten_cpu_provider.cc:484-496
 * (a zero maximum is -0 only if every zero in the row is -0; a zero minimum is -0 if any is).
 * Sum/Mean: docs/user/compute.md:384-388 (empty Sum = 0, Mean = NaN); summation order is a
 * property of the executing route (src/simd/ops/kernel_impl.h:342-362 uses four accumulators), so
 * the oracle gives the plain left-to-right f32 sum AND, through hyle_oracle_row_sum_f64, the f64
 * sum with the sum of magnitudes that bounds any order's error. */
ORACLE_API void hyle_oracle_reduce_rows_f32(int kind, const float *in, float *out, uint64_t rows,
                                            uint64_t cols) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    const float *x = in + r * cols;
    if (kind == RED_SUM || kind == RED_MEAN) {
      float s = 0.0f;
      for (uint64_t i = 0; i < cols; ++i) s += x[i];
      out[r] = kind == RED_SUM ? s : (cols == 0 ? NAN : s / (float)cols);
    } else {
      const int is_max = kind == RED_MAX;
      float acc = is_max ? -INFINITY : INFINITY;
      int any_nan = 0, zero_pos = 0, zero_neg = 0;
      for (uint64_t i = 0; i < cols; ++i) {
        const float v = x[i];
        if (isnan(v)) { any_nan = 1; continue; }
        if (v == 0.0f) { if (signbit(v)) zero_neg = 1; else zero_pos = 1; }
        acc = is_max ? fmaxf(acc, v) : fminf(acc, v);
      }
      if (any_nan) acc = NAN;
      else if (acc == 0.0f) acc = is_max ? (zero_pos ? 0.0f : -0.0f) : (zero_neg ? -0.0f : 0.0f);
      out[r] = acc;
    }
  }
}

ORACLE_API void hyle_oracle_row_sum_f64(const float *in, double *sum, double *abs_sum, uint64_t rows,
                                        uint64_t cols) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    double s = 0.0, a = 0.0;
    for (uint64_t i = 0; i < cols; ++i) { s += (double)in[r * cols + i]; a += fabs((double)in[r * cols + i]); }
    sum[r] = s;
    if (abs_sum) abs_sum[r] = a;
  }
}

/* ---- RmsNorm (bf16 rows, f32 accumulation) ----------------------------------------------------
 * src/simd/math/activations.cc:124-146: fma accumulation left to right,
 * inverse = 1.0f / sqrtf(sum/n + eps), y = round((x * inverse) * w).
 * weight_dtype DT_BF16 or DT_F32, weight may be NULL.  y_f32 (optional) receives the value before
 * the final rounding, for tolerance checks. */
static void rms_row(const uint16_t *x, const void *w, int wdt, uint16_t *y, float *y_f32, uint64_t n,
                    float eps) {
  if (n == 0) return;
  float ss = 0.0f;
  for (uint64_t i = 0; i < n; ++i) {
    const float v = hyle_oracle_bf16_to_f32(x[i]);
    ss = fmaf(v, v, ss);
  }
  const float inverse = 1.0f / sqrtf(ss / (float)n + eps);
  for (uint64_t i = 0; i < n; ++i) {
    float v = hyle_oracle_bf16_to_f32(x[i]) * inverse;
    if (w != NULL) v = v * load_as_f32(w, i, wdt);
    if (y_f32) y_f32[i] = v;
    y[i] = hyle_oracle_f32_to_bf16(v);
  }
}

ORACLE_API void hyle_oracle_rms_norm_bf16(const uint16_t *x, const void *weight, int weight_dtype,
                                          uint16_t *y, float *y_f32, uint64_t rows, uint64_t hidden,
                                          float eps) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r)
    rms_row(x + r * hidden, weight, weight_dtype, y + r * hidden, y_f32 ? y_f32 + r * hidden : NULL,
            hidden, eps);
}

/* RmsNorm on rows of any floating storage (src/compute_provider_native/normalization.cc:41-80 takes f32,
 * f16 and bf16 rows with a weight of the row's type or of f32): the formula above, the storage's own
 * load, one rounding at the store.  y_f32 receives the value before that rounding. */
ORACLE_API void hyle_oracle_rms_norm(int dtype, const void *x, const void *weight, int weight_dtype, void *y,
                                     float *y_f32, uint64_t rows, uint64_t hidden, float eps) {
  if (hidden == 0) return;
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    float ss = 0.0f;
    for (uint64_t i = 0; i < hidden; ++i) {
      const float v = load_as_f32(x, r * hidden + i, dtype);
      ss = fmaf(v, v, ss);
    }
    const float inverse = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (uint64_t i = 0; i < hidden; ++i) {
      float v = load_as_f32(x, r * hidden + i, dtype) * inverse;
      if (weight != NULL) v = v * load_as_f32(weight, i, weight_dtype);
      if (y_f32) y_f32[r * hidden + i] = v;
      store_from_f32(y, r * hidden + i, dtype, v);
    }
  }
}

/* ---- LayerNorm, bf16 storage, f32 accumulation ------------------------------------------------
 * src/simd/math/activations.cc:148-174: sequential f32 sum -> mean; fma-accumulated centered squares;
 * inverse = 1.0f / sqrt(ss / n + eps); y = round(fma((x - mean) * inverse, scale, bias)) or, without
 * scale and bias, round((x - mean) * inverse). */
ORACLE_API void hyle_oracle_layer_norm_bf16(const uint16_t *x, const uint16_t *scale, const uint16_t *bias,
                                            uint16_t *y, float *y_f32, uint64_t rows, uint64_t hidden,
                                            float eps) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    const uint16_t *row = x + r * hidden;
    float sum = 0.0f;
    for (uint64_t i = 0; i < hidden; ++i) sum += hyle_oracle_bf16_to_f32(row[i]);
    const float mean = sum / (float)hidden;
    float ss = 0.0f;
    for (uint64_t i = 0; i < hidden; ++i) {
      const float c = hyle_oracle_bf16_to_f32(row[i]) - mean;
      ss = fmaf(c, c, ss);
    }
    const float inverse = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (uint64_t i = 0; i < hidden; ++i) {
      const float normalized = (hyle_oracle_bf16_to_f32(row[i]) - mean) * inverse;
      const float v = scale ? fmaf(normalized, hyle_oracle_bf16_to_f32(scale[i]), hyle_oracle_bf16_to_f32(bias[i]))
                            : normalized;
      y[r * hidden + i] = hyle_oracle_f32_to_bf16(v);
      if (y_f32) y_f32[r * hidden + i] = v;
    }
  }
}

/* Binary{kAdd} in bf16 (f32 add, one RNE; docs/user/compute.md:358-359) followed by the RmsNorm
 * above reading the rounded sum: the unfused composition the fused kernel must equal. */
ORACLE_API void hyle_oracle_add_rms_norm_bf16(const uint16_t *x, const uint16_t *residual,
                                              const void *weight, int weight_dtype, uint16_t *y,
                                              float *y_f32, uint16_t *h, uint64_t rows,
                                              uint64_t hidden, float eps) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    uint16_t *hr = h + r * hidden;
    for (uint64_t i = 0; i < hidden; ++i)
      hr[i] = hyle_oracle_f32_to_bf16(hyle_oracle_bf16_to_f32(x[r * hidden + i]) +
                                      hyle_oracle_bf16_to_f32(residual[r * hidden + i]));
    rms_row(hr, weight, weight_dtype, y + r * hidden, y_f32 ? y_f32 + r * hidden : NULL, hidden, eps);
  }
}

/* ---- GatedActivation{kSilu} -------------------------------------------------------------------
 * src/simd/math/activations.cc:21-25 (sigmoid without overflow), :44-47 (silu(-inf) = 0),
 * :114-122 (out = round(silu(gate) * up)). */
static inline float sigmoid_f32(float x) {
  if (isnan(x)) return x;
  const float e = expf(-fabsf(x));
  return x < 0.0f ? e / (1.0f + e) : 1.0f / (1.0f + e);
}
static inline float silu_f32(float x) { return x == -INFINITY ? 0.0f : x * sigmoid_f32(x); }

/* ---- Cast --------------------------------------------------------------------------------------
 * src/compute_provider_native/cast.cc:20-91 (element rules), :128-176 (supported pairs) and the 8-bit
 * formats of include/hyle/simd/dtype.h:125-227: decode is exact; encode rounds to nearest even,
 * saturates finite overflow to the largest normal, keeps infinity only where the format has one
 * (E5M2), emits the canonical NaN with the input's sign, and underflows to a signed zero. */
enum { DT_E4M3 = 3, DT_E5M2 = 4, DT_BOOL = 5, DT_I32 = 6 };

static float f8_decode(uint8_t byte, int exp_bits, int man_bits, int bias, int has_inf) {
  const uint32_t sign = (uint32_t)(byte >> 7), exponent = (byte >> man_bits) & ((1u << exp_bits) - 1u);
  const uint32_t mantissa = byte & ((1u << man_bits) - 1u), max_exp = (1u << exp_bits) - 1u;
  uint32_t bits;
  if (exponent == max_exp && has_inf) bits = (sign << 31) | 0x7f800000u | (mantissa << (23 - man_bits));
  else if (exponent == max_exp && mantissa == (1u << man_bits) - 1u) bits = (sign << 31) | 0x7fc00000u;
  else if (exponent == 0) {
    const float magnitude = ldexpf((float)mantissa, 1 - bias - man_bits);
    return sign ? -magnitude : magnitude;
  } else bits = (sign << 31) | ((exponent - (uint32_t)bias + 127u) << 23) | (mantissa << (23 - man_bits));
  float out;
  memcpy(&out, &bits, 4);
  return out;
}

static uint8_t f8_encode(float value, int exp_bits, int man_bits, int bias, int has_inf, float max_normal,
                         uint8_t max_normal_bits, uint8_t nan_bits) {
  uint32_t u;
  memcpy(&u, &value, 4);
  const uint8_t sign = (uint8_t)((u >> 31) << 7);
  const uint32_t magnitude = u & 0x7fffffffu;
  if (magnitude > 0x7f800000u) return sign | nan_bits;
  if (magnitude == 0x7f800000u)
    return has_inf ? (uint8_t)(sign | (((1u << exp_bits) - 1u) << man_bits)) : (uint8_t)(sign | max_normal_bits);
  if (fabsf(value) > max_normal) return sign | max_normal_bits;
  const int exponent = (int)(magnitude >> 23) - 127 + bias;
  const uint32_t fraction = magnitude & 0x7fffffu;
  if (exponent >= 1) {
    const int drop = 23 - man_bits;
    uint32_t mantissa = fraction >> drop, biased = (uint32_t)exponent;
    const uint32_t rest = fraction & ((1u << drop) - 1u), half = 1u << (drop - 1);
    if (rest > half || (rest == half && (mantissa & 1u))) ++mantissa;
    if (mantissa >> man_bits) {
      mantissa = 0;
      ++biased;
    }
    if ((int)biased >= (1 << exp_bits) - (has_inf ? 1 : 0)) return sign | max_normal_bits;
    return (uint8_t)(sign | (biased << man_bits) | (mantissa & ((1u << man_bits) - 1u)));
  }
  const int shift = 1 - exponent;
  if (shift > man_bits + 1) return sign;
  const uint32_t whole = fraction | 0x800000u;
  const int drop = (23 - man_bits) + shift;
  uint32_t mantissa = whole >> drop;
  const uint32_t rest = whole & ((1u << drop) - 1u), half = 1u << (drop - 1);
  if (rest > half || (rest == half && (mantissa & 1u))) ++mantissa;
  return (uint8_t)(sign | (mantissa & 0xffu));
}

ORACLE_API float hyle_oracle_e4m3_to_f32(uint8_t b) { return f8_decode(b, 4, 3, 7, 0); }
ORACLE_API float hyle_oracle_e5m2_to_f32(uint8_t b) { return f8_decode(b, 5, 2, 15, 1); }
ORACLE_API uint8_t hyle_oracle_f32_to_e4m3(float v) { return f8_encode(v, 4, 3, 7, 0, 448.0f, 0x7e, 0x7f); }
ORACLE_API uint8_t hyle_oracle_f32_to_e5m2(float v) { return f8_encode(v, 5, 2, 15, 1, 57344.0f, 0x7b, 0x7e); }

/* i32 -> f32, round to nearest even on the integer's bits (cast.cc:21-41). */
static float i32_to_f32(int32_t value) {
  const uint32_t raw = (uint32_t)value, sign = raw & 0x80000000u;
  const uint32_t magnitude = value < 0 ? 0u - raw : raw;
  if (magnitude == 0) return 0.0f;
  uint32_t exponent = 31u - (uint32_t)__builtin_clz(magnitude), significand;
  if (exponent <= 23) significand = magnitude << (23 - exponent);
  else {
    const uint32_t shift = exponent - 23, rest = magnitude & ((1u << shift) - 1u), half = 1u << (shift - 1);
    significand = magnitude >> shift;
    if (rest > half || (rest == half && (significand & 1u))) ++significand;
    if (significand == (1u << 24)) {
      significand >>= 1;
      ++exponent;
    }
  }
  const uint32_t bits = sign | ((exponent + 127u) << 23) | (significand & 0x7fffffu);
  float out;
  memcpy(&out, &bits, 4);
  return out;
}

static size_t cast_width(int dtype) { return dtype == DT_F32 || dtype == DT_I32 ? 4 : (dtype == DT_BF16 || dtype == DT_F16 ? 2 : 1); }

/* Returns 0, or 1 for a pair the CPU route does not have. */
ORACLE_API int hyle_oracle_cast(int src, int dst, const void *in, void *out, uint64_t count) {
  const int wide_src = src == DT_F32 || src == DT_BF16 || src == DT_F16, wide_dst = dst == DT_F32 || dst == DT_BF16 || dst == DT_F16;
  const int ok = (wide_src && wide_dst && src != dst) || (src == DT_I32 && dst == DT_F32) || (wide_src && dst == DT_BOOL) ||
                 (src == DT_BOOL && wide_dst) || (wide_src && dst == DT_E4M3) || (src == DT_E4M3 && wide_dst) ||
                 (src == DT_E5M2 && (dst == DT_BF16 || dst == DT_E4M3));
  if (!ok) return 1;
  (void)cast_width;
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < count; ++i) {
    float v;
    if (src == DT_I32) v = i32_to_f32(((const int32_t *)in)[i]);
    else if (src == DT_BOOL) v = ((const uint8_t *)in)[i] != 0 ? 1.0f : 0.0f;
    else if (src == DT_E4M3) v = hyle_oracle_e4m3_to_f32(((const uint8_t *)in)[i]);
    else if (src == DT_E5M2) v = hyle_oracle_e5m2_to_f32(((const uint8_t *)in)[i]);
    else v = load_as_f32(in, i, src);
    if (dst == DT_BOOL) {  /* truth of the STORAGE bits: anything but +-0 */
      uint32_t bits;
      if (src == DT_F32) memcpy(&bits, (const float *)in + i, 4), bits &= 0x7fffffffu;
      else bits = ((const uint16_t *)in)[i] & 0x7fffu;
      ((uint8_t *)out)[i] = bits != 0;
    } else if (dst == DT_E4M3) ((uint8_t *)out)[i] = hyle_oracle_f32_to_e4m3(v);
    else store_from_f32(out, i, dst, v);
  }
  return 0;
}

/* CacheEncode{float8(scale)}: src/compute_provider_ggml/ggml_cpu_provider.cc:589-596.  Returns the
 * status bit (4) if any input was not finite; such a value is stored as byte 0. */
ORACLE_API uint32_t hyle_oracle_fp8_e4m3_encode(int dtype, const void *in, uint64_t count, float scale, uint8_t *out) {
  uint32_t status = 0;
#pragma omp parallel for schedule(static) reduction(| : status)
  for (uint64_t i = 0; i < count; ++i) {
    const float v = load_as_f32(in, i, dtype);
    if (!isfinite(v)) {
      out[i] = 0;
      status |= 4u;
    } else out[i] = hyle_oracle_f32_to_e4m3(v / scale);
  }
  return status;
}

/* ---- Scan{axis = -1, exclusive} ------------------------------------------------------------------
 * src/compute_provider_ggml/standard_index.cc:113-157: f32 rows are summed left to right in float;
 * i32 rows in int64, and if any inclusive prefix leaves the int32 range nothing is written and 16 is
 * returned (the status bit of the GPU library). */
ORACLE_API void hyle_oracle_scan_f32(const float *in, float *out, uint64_t rows, uint64_t cols, int exclusive) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    float sum = 0.0f;
    for (uint64_t c = 0; c < cols; ++c) {
      const float before = sum;
      sum = c == 0 ? in[r * cols] : sum + in[r * cols + c];
      out[r * cols + c] = exclusive ? (c == 0 ? 0.0f : before) : sum;
    }
  }
}

ORACLE_API uint32_t hyle_oracle_scan_i32(const int32_t *in, int32_t *out, uint64_t rows, uint64_t cols, int exclusive) {
  for (uint64_t r = 0; r < rows; ++r) {
    int64_t sum = 0;
    for (uint64_t c = 0; c < cols; ++c) {
      sum += in[r * cols + c];
      if (sum < INT32_MIN || sum > INT32_MAX) return 16u;
    }
  }
  for (uint64_t r = 0; r < rows; ++r) {
    int64_t sum = 0;
    for (uint64_t c = 0; c < cols; ++c) {
      const int64_t before = sum;
      sum += in[r * cols + c];
      out[r * cols + c] = (int32_t)(exclusive ? before : sum);
    }
  }
  return 0;
}

/* ---- paged append (KV cache row mover) ---------------------------------------------------------
 * src/compute_backend_cuda/cuda_paged_append.cu:11-62 on the wire structs of
 * include/hyle/compute/detail/paged_append_wire.h:11-34.  words = {active_count, 0, 0, 0} then
 * capacity x {source_kind, source_page, source_row, destination_page, destination_row, rows, 0, 0}.
 * Instructions run in order here; an episode's ranges are disjoint, so the order cannot matter. */
ORACLE_API void hyle_oracle_paged_append(uint8_t *arena, const uint8_t *input, const uint32_t *words, uint32_t page_rows,
                                         uint32_t physical_pages, uint32_t input_rows, uint32_t capacity,
                                         uint64_t row_bytes) {
  const uint32_t active = words[0];
  if (active > capacity || words[1] != 0 || words[2] != 0 || words[3] != 0) return;
  for (uint32_t i = 0; i < active; ++i) {
    const uint32_t *in = words + 4 + 8 * (uint64_t)i;
    const uint32_t kind = in[0], source_page = in[1], source_row = in[2], page = in[3], row = in[4], rows = in[5];
    if (in[6] != 0 || in[7] != 0 || rows == 0 || kind > 1) continue;
    if (page >= physical_pages || row > page_rows || rows > page_rows - row) continue;
    const uint8_t *source;
    if (kind == 0) {
      if (source_row > input_rows || rows > input_rows - source_row) continue;
      source = input + (uint64_t)source_row * row_bytes;
    } else {
      if (source_page >= physical_pages || source_row > page_rows || rows > page_rows - source_row) continue;
      source = arena + ((uint64_t)source_page * page_rows + source_row) * row_bytes;
    }
    memmove(arena + ((uint64_t)page * page_rows + row) * row_bytes, source, (uint64_t)rows * row_bytes);
  }
}

/* Device-lengths variant: src/compute_backend_cuda/cuda_paged_append.cu:82-146 on the records of
 * include/hyle/compute/detail/device_lengths_paged_append_wire.h:8-24.  words = header, directory,
 * `requests` bounds, `pages` page records, 8 words each after the 4-word header.  Returns the status
 * word after the episode (0 ok, 1 a bad page record, 4 an inconsistent episode); a bad page record is
 * skipped and the remaining pages are still written (the reference leaves that subset unspecified). */
ORACLE_API uint32_t hyle_oracle_paged_append_device_lengths(uint8_t *arena, const uint8_t *input, const uint32_t *words,
                                                            const int32_t *query_lengths, const int32_t *kv_lengths,
                                                            uint32_t page_rows, uint32_t physical_pages, uint32_t input_rows,
                                                            uint32_t capacity, uint64_t row_bytes, uint32_t requests,
                                                            uint32_t status) {
  if (status != 0) return status;
  const uint32_t active = words[0];
  const uint32_t *directory = words + 4;
  const uint32_t listed = directory[0], pages = directory[1];
  int valid = !(active == 0 || active > capacity || words[1] || words[2] || words[3] || listed != requests || listed > 32 ||
                pages > active - 1 || listed > active - 1 - pages);
  for (int i = 2; i < 8; ++i)
    if (directory[i]) valid = 0;
  int32_t offsets[33], previous[32], last[32];
  offsets[0] = 0;
  if (valid) {
    for (uint32_t r = 0; r < requests; ++r) {
      const uint32_t *b = words + 4 + 8 * (uint64_t)(1 + r);
      const int32_t q = query_lengths[r], kv = kv_lengths[r];
      const int64_t old = (int64_t)kv - q, next = (int64_t)offsets[r] + q;
      if (b[4] || b[5] || b[6] || b[7]) valid = 0;
      if (q < 0 || (uint32_t)q > b[0] || kv < 0 || (uint32_t)kv > b[3] || old < (int64_t)b[1] || old > (int64_t)b[2] || next < 0 ||
          next > (int64_t)input_rows) {
        valid = 0;
        offsets[r + 1] = previous[r] = last[r] = 0;
      } else {
        offsets[r + 1] = (int32_t)next;
        previous[r] = (int32_t)old;
        last[r] = kv;
      }
    }
  }
  if (!valid) return 4;
  for (uint32_t index = 0; index < pages; ++index) {
    const uint32_t *p = words + 4 + 8 * (uint64_t)(1 + requests + index);
    const uint32_t request = p[0], logical_page = p[1], destination_page = p[2], initialized = p[3], source_page = p[4],
                   source_rows = p[5];
    if (request >= requests || destination_page >= physical_pages || !initialized || initialized > page_rows ||
        source_rows > page_rows || p[6] || p[7]) {
      status = 1;
      continue;
    }
    const uint64_t begin = (uint64_t)logical_page * page_rows, prior = (uint64_t)previous[request], next = (uint64_t)last[request];
    const uint32_t inherited = begin < prior ? (uint32_t)(initialized < prior - begin ? initialized : prior - begin) : 0u;
    const uint32_t live = begin < next ? (uint32_t)(initialized < next - begin ? initialized : next - begin) : 0u;
    const uint32_t added = live - inherited;
    const uint64_t source_row = added ? (uint64_t)offsets[request] + (begin > prior ? begin : prior) - prior : 0;
    if (inherited > live || (inherited && (source_page >= physical_pages || inherited > source_rows)) ||
        (added && (source_row > input_rows || added > input_rows - source_row))) {
      status = 1;
      continue;
    }
    uint8_t *destination = arena + (uint64_t)destination_page * page_rows * row_bytes;
    if (inherited) memmove(destination, arena + (uint64_t)source_page * page_rows * row_bytes, (uint64_t)inherited * row_bytes);
    if (added) memcpy(destination + (uint64_t)inherited * row_bytes, input + source_row * row_bytes, (uint64_t)added * row_bytes);
    if (initialized > live) memset(destination + (uint64_t)live * row_bytes, 0, (uint64_t)(initialized - live) * row_bytes);
  }
  return status;
}

/* ---- sampling_ops::RandomBits / Categorical ---------------------------------------------------
 * Philox-4x32-10 (Salmon, Moraes, Dror, Shaw 2011) keyed as the CPU route keys it
 * (src/compute_provider_native/sampling.cc:76-88): key = identity[0..1], counter = (index low,
 * index high, identity[2], identity[3]); word w of a row is lane w % 4 of block w / 4. */
static void philox_block(const uint32_t *identity, uint64_t index, uint32_t out[4]) {
  uint32_t x0 = (uint32_t)index, x1 = (uint32_t)(index >> 32), x2 = identity[2], x3 = identity[3];
  uint32_t k0 = identity[0], k1 = identity[1];
  for (int round = 0; round < 10; ++round) {
    const uint64_t a = (uint64_t)0xd2511f53u * x0, b = (uint64_t)0xcd9e8d57u * x2;
    const uint32_t n0 = (uint32_t)(b >> 32) ^ x1 ^ k0, n1 = (uint32_t)b, n2 = (uint32_t)(a >> 32) ^ x3 ^ k1, n3 = (uint32_t)a;
    x0 = n0, x1 = n1, x2 = n2, x3 = n3;
    k0 += 0x9e3779b9u;
    k1 += 0xbb67ae85u;
  }
  out[0] = x0, out[1] = x1, out[2] = x2, out[3] = x3;
}

ORACLE_API void hyle_oracle_random_bits(const uint32_t *identities, uint64_t rows, uint32_t words, uint32_t *out) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r)
    for (uint32_t w = 0; w < words; w += 4) {
      uint32_t block[4];
      philox_block(identities + r * 4, w / 4, block);
      for (uint32_t lane = 0; lane < 4 && w + lane < words; ++lane) out[r * words + w + lane] = block[lane];
    }
}

/* Categorical, src/compute_provider_native/sampling.cc:112-181: reject NaN / +inf / all -inf rows;
 * weights exp(x - max) in f32, total and cumulative sums sequential in f64; the uniform is the
 * 52-bit midpoint of the row's first Philox block; the first index whose cumulative weight exceeds
 * total * uniform, else the last index holding the maximum; log p = x - max - log(total).
 * Returns the number of invalid rows (their index is -1).  uniform_out (may be NULL) receives the
 * uniforms so that tests can judge a draw made with another summation order. */
ORACLE_API uint64_t hyle_oracle_categorical(int dtype, const void *logits, const uint32_t *identities, uint64_t rows,
                                            uint64_t cols, int32_t *index, float *log_probability, double *uniform_out) {
  uint64_t invalid = 0;
#pragma omp parallel for schedule(static) reduction(+ : invalid)
  for (uint64_t r = 0; r < rows; ++r) {
    float maximum = -INFINITY;
    int bad = 0;
    for (uint64_t c = 0; c < cols; ++c) {
      const float v = load_as_f32(logits, r * cols + c, dtype);
      if (isnan(v) || v == INFINITY) bad = 1;
      if (v > maximum) maximum = v;
    }
    uint32_t block[4];
    philox_block(identities + r * 4, 0, block);
    const double uniform = ((double)block[0] * 0x1p20 + (double)(block[1] >> 12) + .5) * 0x1p-52;
    if (uniform_out) uniform_out[r] = uniform;
    if (bad || !isfinite(maximum)) {
      index[r] = -1;
      if (log_probability) log_probability[r] = NAN;
      ++invalid;
      continue;
    }
    double total = 0;
    for (uint64_t c = 0; c < cols; ++c) total += (double)expf(load_as_f32(logits, r * cols + c, dtype) - maximum);
    const double threshold = total * uniform;
    double cumulative = 0;
    uint64_t selected = cols;
    for (uint64_t c = 0; c < cols; ++c) {
      cumulative += (double)expf(load_as_f32(logits, r * cols + c, dtype) - maximum);
      if (cumulative > threshold) {
        selected = c;
        break;
      }
    }
    if (selected == cols)
      for (selected = cols; selected > 0; --selected)
        if (load_as_f32(logits, r * cols + selected - 1, dtype) == maximum) {
          --selected;
          break;
        }
    index[r] = (int32_t)selected;
    if (log_probability)
      log_probability[r] = (float)((double)load_as_f32(logits, r * cols + selected, dtype) - (double)maximum - log(total));
  }
  return invalid;
}

/* ---- Unary{kind} ------------------------------------------------------------------------------
 * src/compute_provider_native/elementwise.cc:30-55 (Neg, Exp, Log, Sqrt, Rsqrt = 1.0f / sqrt, Tanh,
 * Relu keeping NaN, Silu) and :84-100 (16-bit storage: f32 value, one rounding);
 * src/simd/math/activations.cc:21-37 (sigmoid, gelu with erf, gelu_tanh; gelu(-inf) = 0);
 * Softplus: at::softplus(x, 1, 20), src/compute_provider_native/aten_cpu_provider.cc:627-628. */
enum { UN_ABS = 0, UN_NEG, UN_EXP, UN_LOG, UN_SQRT, UN_RSQRT, UN_TANH, UN_SIGMOID, UN_RELU, UN_GELU,
       UN_GELU_TANH, UN_SILU, UN_SOFTPLUS };
static inline float unary_value(int kind, float x) {
  switch (kind) {
    case UN_ABS: return fabsf(x);
    case UN_NEG: return -x;
    case UN_EXP: return expf(x);
    case UN_LOG: return logf(x);
    case UN_SQRT: return sqrtf(x);
    case UN_RSQRT: return 1.0f / sqrtf(x);
    case UN_TANH: return tanhf(x);
    case UN_SIGMOID: return sigmoid_f32(x);
    case UN_RELU: return isnan(x) ? x : (x > 0.0f ? x : 0.0f);
    case UN_GELU: return x == -INFINITY ? 0.0f : 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case UN_GELU_TANH: {
      if (x == -INFINITY) return 0.0f;
      const float inner = 0.79788456080286535588f * x * fmaf(0.044715f, x * x, 1.0f);
      return 0.5f * x * (1.0f + tanhf(inner));
    }
    case UN_SILU: return silu_f32(x);
    default: return x > 20.0f ? x : log1pf(expf(x));
  }
}
ORACLE_API void hyle_oracle_unary(int kind, int dtype, const void *in, void *out, uint64_t count) {
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < count; ++i) store_from_f32(out, i, dtype, unary_value(kind, load_as_f32(in, i, dtype)));
}

ORACLE_API void hyle_oracle_swiglu_bf16(const uint16_t *gate, const uint16_t *up, uint16_t *out,
                                        float *out_f32, uint64_t rows, uint64_t cols,
                                        uint64_t gate_stride, uint64_t up_stride) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    for (uint64_t c = 0; c < cols; ++c) {
      const float g = hyle_oracle_bf16_to_f32(gate[r * gate_stride + c]);
      const float u = hyle_oracle_bf16_to_f32(up[r * up_stride + c]);
      const float v = silu_f32(g) * u;
      if (out_f32) out_f32[r * cols + c] = v;
      out[r * cols + c] = hyle_oracle_f32_to_bf16(v);
    }
  }
}

/* GatedActivation{kSilu | kGelu | kGeluTanh} on bf16 / f16 storage: the activation in f32 (the
 * definitions of src/simd/math/activations.cc:21-47 used by unary_value above), times up in f32, one
 * rounding (src/compute_provider_native/aten_cpu_provider.cc:414-445,654-665).  round_gate: the
 * activated gate is rounded to storage first, i.e. Unary{activation} then Binary{kMultiply}.
 * activation: 0 silu, 1 gelu, 2 gelu_tanh. */
ORACLE_API void hyle_oracle_gated_activation(int activation, int dtype, int round_gate, const uint16_t *gate,
                                             const uint16_t *up, uint16_t *out, float *out_f32, uint64_t rows,
                                             uint64_t cols, uint64_t gate_stride, uint64_t up_stride) {
  const int kind = activation == 0 ? UN_SILU : activation == 1 ? UN_GELU : UN_GELU_TANH;
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    for (uint64_t c = 0; c < cols; ++c) {
      const float g = load_as_f32(gate, r * gate_stride + c, dtype);
      const float u = load_as_f32(up, r * up_stride + c, dtype);
      float a = unary_value(kind, g);
      if (round_gate) {
        uint32_t word = 0;  /* wide enough for any storage type the helpers know */
        store_from_f32(&word, 0, dtype, a);
        a = load_as_f32(&word, 0, dtype);
      }
      const float v = a * u;
      if (out_f32) out_f32[r * cols + c] = v;
      store_from_f32(out, r * cols + c, dtype, v);
    }
  }
}

/* ---- Softmax / LogSoftmax / log-sum-exp -------------------------------------------------------
 * src/simd/math/activations.cc:274-334: finite_row_max rejects NaN and +inf and rows without a
 * finite maximum (all outputs NaN); exp in f32, sum in f64, multiply by float(1/sum);
 * log-softmax shift = max + float(log(sum)). */
static int finite_row_max(const float *x, uint64_t n, float *maximum) {
  float m = -INFINITY;
  for (uint64_t i = 0; i < n; ++i) {
    if (isnan(x[i]) || x[i] == INFINITY) return 0;
    if (x[i] > m) m = x[i];
  }
  *maximum = m;
  return isfinite(m);
}

ORACLE_API void hyle_oracle_softmax_f32(int kind, const float *in, float *out, uint64_t rows,
                                        uint64_t cols) {
  if (cols == 0) return;
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    const float *x = in + r * cols;
    float *y = out + r * cols;
    float m;
    if (!finite_row_max(x, cols, &m)) { for (uint64_t i = 0; i < cols; ++i) y[i] = NAN; continue; }
    double sum = 0.0;
    if (kind == SM_SOFTMAX) {
      for (uint64_t i = 0; i < cols; ++i) { const float e = expf(x[i] - m); y[i] = e; sum += (double)e; }
      const float inverse = (float)(1.0 / sum);
      for (uint64_t i = 0; i < cols; ++i) y[i] *= inverse;
    } else {
      for (uint64_t i = 0; i < cols; ++i) sum += (double)expf(x[i] - m);
      const float shift = m + (float)log(sum);
      for (uint64_t i = 0; i < cols; ++i) y[i] = x[i] - shift;
    }
  }
}

/* TopK{count=1}: src/simd/sort/top_k.cc:13-27 (NaN last, larger value first, lower index on
 * ties) and :51-69 (k == 1 scan starting from element 0). */
static inline int better(float a, uint32_t ai, float b, uint32_t bi) {
  const int an = isnan(a), bn = isnan(b);
  if (an != bn) return !an;
  if (!an) { if (a > b) return 1; if (a < b) return 0; }
  return ai < bi;
}

ORACLE_API void hyle_oracle_argmax_f32(const float *in, int32_t *index, float *value, uint64_t rows,
                                       uint64_t cols) {
  if (cols == 0) return;
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    const float *x = in + r * cols;
    float best = x[0];
    uint32_t bi = 0;
    for (uint64_t i = 1; i < cols; ++i)
      if (better(x[i], (uint32_t)i, best, bi)) { best = x[i]; bi = (uint32_t)i; }
    if (index) index[r] = (int32_t)bi;
    if (value) value[r] = best;
  }
}

/* The fused logits reduction = LogSoftmax shift (lse) + Softmax -> Cast{bf16} + TopK{1}.
 * probs_f32 (optional) receives the softmax before the bf16 rounding. */
ORACLE_API void hyle_oracle_logits_reduce_f32(const float *in, uint64_t rows, uint64_t cols,
                                              float *lse, uint16_t *probs_bf16, float *probs_f32,
                                              int32_t *index, float *value) {
  if (cols == 0) return;
  if (index || value) hyle_oracle_argmax_f32(in, index, value, rows, cols);
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    const float *x = in + r * cols;
    float m;
    if (!finite_row_max(x, cols, &m)) {
      if (lse) lse[r] = NAN;
      for (uint64_t i = 0; i < cols; ++i) {
        if (probs_bf16) probs_bf16[r * cols + i] = hyle_oracle_f32_to_bf16(NAN);
        if (probs_f32) probs_f32[r * cols + i] = NAN;
      }
      continue;
    }
    double sum = 0.0;
    for (uint64_t i = 0; i < cols; ++i) sum += (double)expf(x[i] - m);
    if (lse) lse[r] = m + (float)log(sum);
    const float inverse = (float)(1.0 / sum);
    if (probs_bf16 || probs_f32) {
      for (uint64_t i = 0; i < cols; ++i) {
        const float p = expf(x[i] - m) * inverse;
        if (probs_f32) probs_f32[r * cols + i] = p;
        if (probs_bf16) probs_bf16[r * cols + i] = hyle_oracle_f32_to_bf16(p);
      }
    }
  }
}

/* Cast{f32 -> bf16}: include/hyle/simd/dtype.h:114-121. */
ORACLE_API void hyle_oracle_cast_f32_to_bf16(const float *in, uint16_t *out, uint64_t count) {
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < count; ++i) out[i] = hyle_oracle_f32_to_bf16(in[i]);
}

/* ---- Q8_0 -------------------------------------------------------------------------------------
 * Encode: src/compute_provider_ggml/ggml_cpu_provider.cc:585-615 around ggml's reference row
 * quantiser; block layout src/compute_ops/low_precision.cc:28-29 (f16 scale little endian at
 * bytes 0-1, then 32 int8).  Returns 1 when any block was invalid (the reference then completes
 * with InvalidArgument, :1720-1721). */
ORACLE_API int hyle_oracle_q8_0_encode(int dtype, const void *in, uint64_t count, uint8_t *out) {
  const uint64_t blocks = count / 32;
  int invalid = 0;
#pragma omp parallel for schedule(static) reduction(| : invalid)
  for (uint64_t b = 0; b < blocks; ++b) {
    float v[32];
    int valid = 1;
    float amax = 0.0f;
    for (int j = 0; j < 32; ++j) {
      v[j] = load_as_f32(in, b * 32 + j, dtype);
      valid &= isfinite(v[j]) && fabsf(v[j]) <= 65504.0f * 127.0f;
      amax = fmaxf(amax, fabsf(v[j]));
    }
    uint8_t *dst = out + b * 34;
    if (!valid) { invalid |= 1; memset(dst, 0, 34); continue; }
    const float d = amax / 127.0f;
    const uint16_t scale = hyle_oracle_f32_to_f16(d);
    if (scale == 0) { memset(dst, 0, 34); continue; }
    const float id = 1.0f / d;
    dst[0] = (uint8_t)(scale & 0xff);
    dst[1] = (uint8_t)(scale >> 8);
    for (int j = 0; j < 32; ++j) dst[2 + j] = (uint8_t)(int8_t)roundf(v[j] * id);
  }
  return invalid;
}

/* Decode: value = f32(f16 scale) * code (exact in f32), one RNE to bf16.  The arithmetic the
 * reference's kGgufQ8_0 consumers apply (src/compute_ops/low_precision.cc:269-297). */
ORACLE_API void hyle_oracle_q8_0_decode_bf16(const uint8_t *blocks_in, uint64_t count, uint16_t *out) {
  const uint64_t blocks = count / 32;
#pragma omp parallel for schedule(static)
  for (uint64_t b = 0; b < blocks; ++b) {
    const uint8_t *src = blocks_in + b * 34;
    const float d = hyle_oracle_f16_to_f32((uint16_t)(src[0] | (src[1] << 8)));
    for (int j = 0; j < 32; ++j) out[b * 32 + j] = hyle_oracle_f32_to_bf16(d * (float)(int8_t)src[2 + j]);
  }
}

/* Reduce{kSum, Axes::all()} of Cast(bf16->f32)^2 (include/hyle/compute/operation.h:232-248), with
 * f64 accumulation: the value any f32 route must approach. */
ORACLE_API double hyle_oracle_sum_squares_bf16(const uint16_t *in, uint64_t count) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (uint64_t i = 0; i < count; ++i) {
    const double v = (double)hyle_oracle_bf16_to_f32(in[i]);
    total += v * v;
  }
  return total;
}

/* The fused sweep step of the Q8_0 workload: encode, decode and sum of squares in one row-parallel
 * pass (what a CPU provider would run per row range). */
ORACLE_API int hyle_oracle_q8_0_roundtrip_bf16(const uint16_t *in, uint64_t count, uint8_t *blocks_out,
                                               uint16_t *decoded, double *sum_squares) {
  const int invalid = hyle_oracle_q8_0_encode(DT_BF16, in, count, blocks_out);
  hyle_oracle_q8_0_decode_bf16(blocks_out, count, decoded);
  *sum_squares = hyle_oracle_sum_squares_bf16(in, count);
  return invalid;
}

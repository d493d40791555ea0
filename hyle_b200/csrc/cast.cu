// Cast between the storage types of the tensor library: f32 / bf16 / f16 among themselves, the two
// 8-bit floating formats, bool and i32 -> f32.  Every pair is a pure function of one element and
// bit-exact against the CPU route (src/compute_provider_native/cast.cc:20-176 with the conversions
// of include/hyle/simd/dtype.h):
//   * wide -> narrow floating types round to nearest even once;
//   * E4M3 (bias 7, no infinity, NaN = 0x7F) and E5M2 (bias 15, IEEE-like) encode with
//     round-to-nearest-even and SATURATE finite overflow to the largest normal; an infinite input
//     saturates for E4M3 and stays infinite for E5M2 (dtype.h:163-213);
//   * bool is truth: a floating value converts to 1 unless its magnitude bits are all zero (NaN and
//     subnormals are true, -0 is false); a bool byte converts to 1.0 when non-zero (cast.cc:78-91);
//   * i32 -> f32 rounds to nearest even (cast.cc:21-41).
// HBM-bound: a thread moves eight consecutive elements per step with the widest loads and stores the
// two element sizes allow (8 to 32 bytes), four steps in flight.
#include <cmath>

#include "common.cuh"

#include <type_traits>

namespace hb {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;

// ---- 8-bit floating formats ----------------------------------------------------------------------
template <int kExpBits, int kManBits, int kBias, bool kHasInf>
__device__ __forceinline__ float f8_to_f32(uint32_t byte) {
  const uint32_t sign = (byte & 0x80u) << 24;
  const uint32_t exponent = (byte >> kManBits) & ((1u << kExpBits) - 1u);
  const uint32_t mantissa = byte & ((1u << kManBits) - 1u);
  constexpr uint32_t kMaxExp = (1u << kExpBits) - 1u;
  if (kHasInf && exponent == kMaxExp) return __uint_as_float(sign | 0x7f800000u | (mantissa << (23 - kManBits)));
  if (!kHasInf && exponent == kMaxExp && mantissa == (1u << kManBits) - 1u) return __uint_as_float(sign | 0x7fc00000u);
  if (exponent == 0) {  // zero or subnormal: mantissa * 2^(1 - bias - kManBits), exact in f32
    const float magnitude = static_cast<float>(mantissa) * __uint_as_float((127u + 1 - kBias - kManBits) << 23);
    return __uint_as_float(sign | __float_as_uint(magnitude));
  }
  return __uint_as_float(sign | ((exponent - kBias + 127u) << 23) | (mantissa << (23 - kManBits)));
}

template <int kExpBits, int kManBits, int kBias, bool kHasInf>
__device__ __forceinline__ uint32_t f32_to_f8(float value, uint32_t max_normal_f32_bits, uint32_t max_normal_bits,
                                              uint32_t nan_bits) {
  const uint32_t u = __float_as_uint(value);
  const uint32_t sign = (u >> 31) << 7;
  const uint32_t magnitude = u & 0x7fffffffu;
  if (magnitude > 0x7f800000u) return sign | nan_bits;
  if (magnitude == 0x7f800000u) return kHasInf ? sign | (((1u << kExpBits) - 1u) << kManBits) : sign | max_normal_bits;
  if (magnitude > max_normal_f32_bits) return sign | max_normal_bits;  // finite overflow saturates
  const int exponent = static_cast<int>(magnitude >> 23) - 127 + kBias;  // biased for the 8-bit format
  const uint32_t fraction = magnitude & 0x7fffffu;
  if (exponent >= 1) {
    constexpr int kDrop = 23 - kManBits;
    uint32_t mantissa = fraction >> kDrop;
    const uint32_t rest = fraction & ((1u << kDrop) - 1u), half = 1u << (kDrop - 1);
    uint32_t biased = static_cast<uint32_t>(exponent);
    if (rest > half || (rest == half && (mantissa & 1u))) ++mantissa;
    if (mantissa >> kManBits) {
      mantissa = 0;
      ++biased;
    }
    if (biased >= (1u << kExpBits) - (kHasInf ? 1u : 0u)) return sign | max_normal_bits;
    return sign | (biased << kManBits) | (mantissa & ((1u << kManBits) - 1u));
  }
  const int shift = 1 - exponent;
  if (shift > kManBits + 1) return sign;  // underflow to a signed zero
  const uint32_t whole = fraction | 0x800000u;
  const int drop = (23 - kManBits) + shift;
  uint32_t mantissa = whole >> drop;
  const uint32_t rest = whole & ((1u << drop) - 1u), half = 1u << (drop - 1);
  if (rest > half || (rest == half && (mantissa & 1u))) ++mantissa;  // may carry into the first normal
  return sign | (mantissa & 0xffu);
}

// E4M3 goes through the conversion instructions of the hardware, which implement the same rule
// (round to nearest even, finite overflow and infinity saturate to 448): one instruction instead of
// the forty of the integer algorithm above, which stays as the statement of the rule and serves
// E5M2.  The instruction's NaN is always +NaN; the CPU route keeps a NaN's sign, so that is patched.
__device__ __forceinline__ uint32_t f32_to_e4m3(float v) {
  unsigned short pair;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(v));  // low byte <- v
  const uint32_t code = pair & 0xffu;
  return v != v ? ((__float_as_uint(v) >> 24) & 0x80u) | 0x7fu : code;
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  uint32_t halves;  // every E4M3 value is exact in f16
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(halves) : "h"(static_cast<unsigned short>(b)));
  return f16_to_f32(static_cast<unsigned short>(halves & 0xffffu));  // NaN stays NaN; its sign is not kept
}
__device__ __forceinline__ float e5m2_to_f32(uint32_t b) { return f8_to_f32<5, 2, 15, true>(b); }

// ---- one element: storage word -> f32 -> storage word -------------------------------------------------
template <int kDtype> struct Element;  // bytes per element and the unsigned word that holds it
template <> struct Element<HYLE_B200_F32> { using Word = uint32_t; };
template <> struct Element<HYLE_B200_I32> { using Word = uint32_t; };
template <> struct Element<HYLE_B200_BF16> { using Word = unsigned short; };
template <> struct Element<HYLE_B200_F16> { using Word = unsigned short; };
template <> struct Element<HYLE_B200_E4M3> { using Word = unsigned char; };
template <> struct Element<HYLE_B200_E5M2> { using Word = unsigned char; };
template <> struct Element<HYLE_B200_BOOL> { using Word = unsigned char; };

template <int kSrc>
__device__ __forceinline__ float decode(uint32_t word) {
  if constexpr (kSrc == HYLE_B200_F32) return __uint_as_float(word);
  if constexpr (kSrc == HYLE_B200_I32) return __int2float_rn(static_cast<int>(word));
  if constexpr (kSrc == HYLE_B200_BF16) return bf16_to_f32(static_cast<unsigned short>(word));
  if constexpr (kSrc == HYLE_B200_F16) {
    // cvt.f32.f16 turns every NaN into the positive canonical one; the 8-bit encoders keep a NaN's sign
    if ((word & 0x7fffu) > 0x7c00u) return __uint_as_float(((word & 0x8000u) << 16) | 0x7fc00000u);
    return f16_to_f32(static_cast<unsigned short>(word));
  }
  if constexpr (kSrc == HYLE_B200_E4M3) return e4m3_to_f32(word);
  if constexpr (kSrc == HYLE_B200_E5M2) return e5m2_to_f32(word);
  return word != 0 ? 1.0f : 0.0f;  // bool
}

template <int kDst>
__device__ __forceinline__ uint32_t encode(float value) {
  if constexpr (kDst == HYLE_B200_F32) return __float_as_uint(value);
  if constexpr (kDst == HYLE_B200_BF16) return f32_to_bf16(value);
  if constexpr (kDst == HYLE_B200_F16) return f32_to_f16(value);
  if constexpr (kDst == HYLE_B200_E4M3) return f32_to_e4m3(value);
  // bool: the decoded value is exact for every source type, so "magnitude bits non-zero" is
  // "not equal to zero" (NaN compares unequal; no flush-to-zero is in effect)
  return value == 0.0f ? 0u : 1u;
}

template <int kSrc, int kDst>
__device__ __forceinline__ uint32_t convert(uint32_t word) {
  return encode<kDst>(decode<kSrc>(word));
}

// ---- eight elements per thread-step -----------------------------------------------------------------
template <int kBytes> struct Pack;  // eight elements of kBytes each
template <> struct Pack<1> { uint2 v; };
template <> struct Pack<2> { uint4 v; };
template <> struct Pack<4> { uint4 v[2]; };

template <int kBytes>
__device__ __forceinline__ Pack<kBytes> load_pack(const void *base, uint64_t index) {
  Pack<kBytes> p;
  if constexpr (kBytes == 1) p.v = ld_stream(static_cast<const uint2 *>(base) + index);
  else if constexpr (kBytes == 2) p.v = ld_stream(static_cast<const uint4 *>(base) + index);
  else {
    p.v[0] = ld_stream(static_cast<const uint4 *>(base) + 2 * index);
    p.v[1] = ld_stream(static_cast<const uint4 *>(base) + 2 * index + 1);
  }
  return p;
}
template <int kBytes>
__device__ __forceinline__ void store_pack(void *base, uint64_t index, const Pack<kBytes> &p) {
  if constexpr (kBytes == 1) st_stream(static_cast<uint2 *>(base) + index, p.v);
  else if constexpr (kBytes == 2) st_stream(static_cast<uint4 *>(base) + index, p.v);
  else {
    st_stream(static_cast<uint4 *>(base) + 2 * index, p.v[0]);
    st_stream(static_cast<uint4 *>(base) + 2 * index + 1, p.v[1]);
  }
}
template <int kBytes>
__device__ __forceinline__ void unpack(const Pack<kBytes> &p, uint32_t (&w)[8]) {
  if constexpr (kBytes == 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = (p.v.x >> (8 * i)) & 0xffu;
      w[4 + i] = (p.v.y >> (8 * i)) & 0xffu;
    }
  } else if constexpr (kBytes == 2) {
    const uint32_t q[4] = {p.v.x, p.v.y, p.v.z, p.v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[2 * i] = q[i] & 0xffffu;
      w[2 * i + 1] = q[i] >> 16;
    }
  } else {
    w[0] = p.v[0].x; w[1] = p.v[0].y; w[2] = p.v[0].z; w[3] = p.v[0].w;
    w[4] = p.v[1].x; w[5] = p.v[1].y; w[6] = p.v[1].z; w[7] = p.v[1].w;
  }
}
template <int kBytes>
__device__ __forceinline__ Pack<kBytes> pack(const uint32_t (&w)[8]) {
  Pack<kBytes> p;
  if constexpr (kBytes == 1) {
    p.v.x = w[0] | (w[1] << 8) | (w[2] << 16) | (w[3] << 24);
    p.v.y = w[4] | (w[5] << 8) | (w[6] << 16) | (w[7] << 24);
  } else if constexpr (kBytes == 2) {
    p.v = make_uint4(w[0] | (w[1] << 16), w[2] | (w[3] << 16), w[4] | (w[5] << 16), w[6] | (w[7] << 16));
  } else {
    p.v[0] = make_uint4(w[0], w[1], w[2], w[3]);
    p.v[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
  return p;
}

template <int kSrc, int kDst>
__global__ void __launch_bounds__(kThreads)
cast_kernel(const void *in, void *out, uint64_t packs) {
  grid_dependency_sync();
  constexpr int kIn = sizeof(typename Element<kSrc>::Word), kOut = sizeof(typename Element<kDst>::Word);
  constexpr int kUnroll = kIn == 4 ? 2 : 4;  // bytes in flight per thread: 64 (4-byte source) to 32 (1-byte)
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < packs; i += kUnroll * stride) {
    Pack<kIn> source[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) source[k] = load_pack<kIn>(in, i + k * stride);
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      uint32_t w[8];
      unpack<kIn>(source[k], w);
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = convert<kSrc, kDst>(w[e]);
      store_pack<kOut>(out, i + k * stride, pack<kOut>(w));
    }
  }
  for (; i < packs; i += stride) {
    uint32_t w[8];
    unpack<kIn>(load_pack<kIn>(in, i), w);
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = convert<kSrc, kDst>(w[e]);
    store_pack<kOut>(out, i, pack<kOut>(w));
  }
}

// 4-byte destinations: four values per thread-step, so that a warp's store instruction writes 512
// contiguous bytes.  With eight values per thread the two 16-byte stores of a thread fall into the
// same 32-byte sector as halves, every sector is written by two instructions, and the store path --
// these casts write four times (1-byte source) or twice (2-byte source) what they read -- is the limit.
template <int kSrc, int kDst>
__global__ void __launch_bounds__(kThreads)
cast_quads_kernel(const void *in, void *out, uint64_t quads) {
  grid_dependency_sync();
  constexpr int kIn = sizeof(typename Element<kSrc>::Word);
  static_assert(sizeof(typename Element<kDst>::Word) == 4, "4-byte destinations");
  constexpr int kUnroll = kIn == 4 ? 4 : 8;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  auto load = [&](uint64_t q, uint32_t (&w)[4]) {
    if constexpr (kIn == 1) {
      const uint32_t v = __ldcs(static_cast<const uint32_t *>(in) + q);
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = (v >> (8 * e)) & 0xffu;
    } else if constexpr (kIn == 2) {
      const uint2 v = ld_stream(static_cast<const uint2 *>(in) + q);
      w[0] = v.x & 0xffffu, w[1] = v.x >> 16, w[2] = v.y & 0xffffu, w[3] = v.y >> 16;
    } else {
      const uint4 v = ld_stream(static_cast<const uint4 *>(in) + q);
      w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    }
  };
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < quads; i += kUnroll * stride) {
    uint32_t w[kUnroll][4];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) load(i + k * stride, w[k]);
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
#pragma unroll
      for (int e = 0; e < 4; ++e) w[k][e] = convert<kSrc, kDst>(w[k][e]);
      st_stream(static_cast<uint4 *>(out) + i + k * stride, make_uint4(w[k][0], w[k][1], w[k][2], w[k][3]));
    }
  }
  for (; i < quads; i += stride) {
    uint32_t w[4];
    load(i, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) w[e] = convert<kSrc, kDst>(w[e]);
    st_stream(static_cast<uint4 *>(out) + i, make_uint4(w[0], w[1], w[2], w[3]));
  }
}

// Unaligned tensors and the tail behind the last whole pack.
template <int kSrc, int kDst>
__global__ void __launch_bounds__(kThreads)
cast_scalar_kernel(const typename Element<kSrc>::Word *in, typename Element<kDst>::Word *out, uint64_t count) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride)
    out[i] = static_cast<typename Element<kDst>::Word>(convert<kSrc, kDst>(in[i]));
}

template <int kSrc, int kDst>
int launch_cast(cudaStream_t stream, const void *in, void *out, uint64_t count) {
  using In = typename Element<kSrc>::Word;
  using Out = typename Element<kDst>::Word;
  if (!aligned_to(in, sizeof(In)) || !aligned_to(out, sizeof(Out))) return HYLE_B200_INVALID_VALUE;
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  const bool vector_ok = aligned_to(in, 8 * sizeof(In) > 16 ? 16 : 8 * sizeof(In)) &&
                         aligned_to(out, 8 * sizeof(Out) > 16 ? 16 : 8 * sizeof(Out));
  uint64_t packs = vector_ok ? count / 8 : 0;
  if constexpr (sizeof(Out) == 4) {
    if (packs != 0) {
      const uint64_t quads = packs * 2;
      const unsigned grid = clamp_grid((quads + kThreads * 8 - 1) / (kThreads * 8), resident);
      const int status = launch(cast_quads_kernel<kSrc, kDst>, dim3(grid), dim3(kThreads), 0, stream, in, out, quads);
      if (status != HYLE_B200_OK) return status;
    }
  } else if (packs != 0) {
    const unsigned grid = clamp_grid((packs + kThreads * 4 - 1) / (kThreads * 4), resident);
    const int status = launch(cast_kernel<kSrc, kDst>, dim3(grid), dim3(kThreads), 0, stream, in, out, packs);
    if (status != HYLE_B200_OK) return status;
  }
  const uint64_t done = packs * 8;
  if (done == count) return HYLE_B200_OK;
  const unsigned grid = clamp_grid((count - done + kThreads - 1) / kThreads, resident);
  return launch(cast_scalar_kernel<kSrc, kDst>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const In *>(in) + done,
                static_cast<Out *>(out) + done, count - done);
}

// ---- Select: out = condition ? when_true : when_false, elements moved as bits ------------------------------
// (include/hyle/compute/operation.h:305, src/compute_ops/operation.cc:1309-1328; any non-zero
// condition byte is true, include/hyle/simd/ops.h:80).  Either branch may be the full tensor or repeat
// with a period over the trailing axes (period 1 = one scalar, the masking case).
template <int kBytes>
__global__ void __launch_bounds__(kThreads)
select_kernel(const void *condition, const void *when_true, const void *when_false, void *out, uint64_t packs) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < packs; i += stride) {
    uint32_t c[8], a[8], b[8];
    unpack<1>(load_pack<1>(condition, i), c);
    unpack<kBytes>(load_pack<kBytes>(when_true, i), a);
    unpack<kBytes>(load_pack<kBytes>(when_false, i), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = c[e] != 0 ? a[e] : b[e];
    store_pack<kBytes>(out, i, pack<kBytes>(a));
  }
}

// Broadcast branches, unaligned tensors and tails: one element per thread-step.
template <class Word>
__global__ void __launch_bounds__(kThreads)
select_scalar_kernel(const unsigned char *condition, const Word *when_true, const Word *when_false, Word *out,
                     uint64_t first, uint64_t count, uint64_t true_period, uint64_t false_period) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t i = first + static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride)
    out[i] = condition[i] != 0 ? when_true[i % true_period] : when_false[i % false_period];
}

template <int kBytes>
int launch_select(cudaStream_t stream, const void *condition, const void *when_true, const void *when_false, void *out,
                  uint64_t count, uint64_t true_period, uint64_t false_period) {
  using Word = typename std::conditional<kBytes == 4, uint32_t, unsigned short>::type;
  if (!aligned_to(when_true, kBytes) || !aligned_to(when_false, kBytes) || !aligned_to(out, kBytes))
    return HYLE_B200_INVALID_VALUE;
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  const bool vector_ok = true_period == count && false_period == count && aligned_to(condition, 8) && aligned_to(out, 16) &&
                         aligned_to(when_true, 16) && aligned_to(when_false, 16);
  uint64_t done = 0;
  if (vector_ok && count >= 8) {
    const uint64_t packs = count / 8;
    const unsigned grid = clamp_grid((packs + kThreads * 2 - 1) / (kThreads * 2), resident);
    const int status = launch(select_kernel<kBytes>, dim3(grid), dim3(kThreads), 0, stream, condition, when_true, when_false,
                              out, packs);
    if (status != HYLE_B200_OK) return status;
    done = packs * 8;
  }
  if (done == count) return HYLE_B200_OK;
  const unsigned grid = clamp_grid((count - done + kThreads - 1) / kThreads, resident);
  return launch(select_scalar_kernel<Word>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const unsigned char *>(condition),
                static_cast<const Word *>(when_true), static_cast<const Word *>(when_false), static_cast<Word *>(out), done,
                count, true_period, false_period);
}

// ---- CacheEncode{float8(scale)}: value / scale -> E4M3, a non-finite value -> byte 0 and a status bit -------
// (src/compute_provider_ggml/ggml_cpu_provider.cc:589-596).  The byte is that of the IEEE quotient, but
// the division itself is rarely executed: value * (1 / scale) lies within 2^-22 (relative) of the
// quotient, the conversion is monotone, so when the two values 2^-21 below and above that product
// convert to the same byte (one paired conversion instruction) the quotient converts to it too.
// Otherwise -- the product sits at a rounding boundary of E4M3, about one element in 2^17 -- the division
// decides.  `inverse` = 0 selects the division for every element (scales whose reciprocal is not a
// normal number).
template <int kSrc>
__device__ __forceinline__ uint32_t cache_code(uint32_t word, float scale, bool &invalid) {
  const float value = decode<kSrc>(word);
  if (!isfinite(value)) {
    invalid = true;
    return 0u;
  }
  return f32_to_e4m3(__fdiv_rn(value, scale));
}
// The shortcut for one element: the byte when it is certain, and `unsure` set when the product sits at
// a rounding boundary or the value is not finite (the caller then redoes its pack with cache_code).
template <int kSrc>
__device__ __forceinline__ uint32_t cache_code_fast(uint32_t word, float inverse, bool &unsure) {
  const float value = decode<kSrc>(word);
  const float product = __fmul_rn(value, inverse);
  const float margin = __fmul_rn(product, 4.76837158203125e-7f);  // 2^-21
  unsigned short pair;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(__fadd_rn(product, margin)), "f"(__fsub_rn(product, margin)));
  unsure |= (pair & 0xffu) != (pair >> 8) || !isfinite(value);
  return pair & 0xffu;
}
// Eight elements: branch-free shortcut, and the exact route for the whole pack in the rare unsure case.
template <int kSrc>
__device__ __forceinline__ void cache_codes(uint32_t (&w)[8], float scale, float inverse, bool &invalid) {
  if (inverse != 0.0f) {
    uint32_t fast[8];
    bool unsure = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) fast[e] = cache_code_fast<kSrc>(w[e], inverse, unsure);
    if (!unsure) {
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = fast[e];
      return;
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) w[e] = cache_code<kSrc>(w[e], scale, invalid);
}

template <int kSrc>
__global__ void __launch_bounds__(kThreads)
cache_encode_e4m3_kernel(const void *in, void *out, uint64_t packs, float scale, float inverse, uint32_t *status_word) {
  grid_dependency_sync();
  constexpr int kIn = sizeof(typename Element<kSrc>::Word);
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  bool invalid = false;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + stride < packs; i += 2 * stride) {  // two packs in flight per thread
    uint32_t a[8], b[8];
    const auto first = load_pack<kIn>(in, i), second = load_pack<kIn>(in, i + stride);
    unpack<kIn>(first, a);
    unpack<kIn>(second, b);
    cache_codes<kSrc>(a, scale, inverse, invalid);
    cache_codes<kSrc>(b, scale, inverse, invalid);
    store_pack<1>(out, i, pack<1>(a));
    store_pack<1>(out, i + stride, pack<1>(b));
  }
  for (; i < packs; i += stride) {
    uint32_t w[8];
    unpack<kIn>(load_pack<kIn>(in, i), w);
    cache_codes<kSrc>(w, scale, inverse, invalid);
    store_pack<1>(out, i, pack<1>(w));
  }
  if (status_word != nullptr && __any_sync(kFullMask, invalid) && (threadIdx.x & 31) == 0)
    atomicOr(status_word, HYLE_B200_STATUS_INVALID_FP8_INPUT);
}

template <int kSrc>
__global__ void __launch_bounds__(kThreads)
cache_encode_e4m3_scalar_kernel(const typename Element<kSrc>::Word *in, unsigned char *out, uint64_t count, float scale,
                                uint32_t *status_word) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  bool invalid = false;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride)
    out[i] = static_cast<unsigned char>(cache_code<kSrc>(in[i], scale, invalid));
  if (status_word != nullptr && invalid) atomicOr(status_word, HYLE_B200_STATUS_INVALID_FP8_INPUT);
}

template <int kSrc>
int launch_cache_encode(cudaStream_t stream, const void *in, void *out, uint64_t count, float scale, uint32_t *status_word) {
  using In = typename Element<kSrc>::Word;
  if (!aligned_to(in, sizeof(In))) return HYLE_B200_INVALID_VALUE;
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  const bool vector_ok = aligned_to(in, 16) && aligned_to(out, 8);
  const uint64_t packs = vector_ok ? count / 8 : 0;
  if (packs != 0) {
    const unsigned grid = clamp_grid((packs + kThreads * 4 - 1) / (kThreads * 4), resident);
    // the reciprocal shortcut needs scale and 1 / scale to be normal numbers (relative error bounds hold)
    const float reciprocal = 1.0f / scale;
    const bool normal = std::isnormal(scale) && std::isnormal(reciprocal);
    const int status = launch(cache_encode_e4m3_kernel<kSrc>, dim3(grid), dim3(kThreads), 0, stream, in, out, packs, scale,
                              normal ? reciprocal : 0.0f, status_word);
    if (status != HYLE_B200_OK) return status;
  }
  const uint64_t done = packs * 8;
  if (done == count) return HYLE_B200_OK;
  const unsigned grid = clamp_grid((count - done + kThreads - 1) / kThreads, resident);
  return launch(cache_encode_e4m3_scalar_kernel<kSrc>, dim3(grid), dim3(kThreads), 0, stream,
                static_cast<const In *>(in) + done, static_cast<unsigned char *>(out) + done, count - done, scale, status_word);
}

// ---- strided views --------------------------------------------------------------------------------
// Cast (or plain copy) from a view of rank <= 8 with arbitrary byte strides into a dense tensor: the
// form in which the reference hands non-dense operands to its tensor kernels
// (src/compute_provider_cuda/tensor_kernel.cu:70-108 reads every operand through byte strides).  The
// host merges axes that are contiguous with each other, so typical views (slices, permutations of
// two or three axes, broadcasts) arrive with rank 1-3; a view that collapses to a dense run takes the
// dense kernels above.
struct View {
  uint32_t rank;
  uint64_t dims[8];     // outermost first
  int64_t strides[8];   // bytes
};

template <class Word, int kSrc, int kDst, bool kCopy, class Index>
__global__ void __launch_bounds__(kThreads)
strided_kernel(const unsigned char *__restrict__ in, typename Element<kDst>::Word *__restrict__ out, uint64_t count, const View view) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  auto fetch = [&](uint64_t i) {
    Index rest = static_cast<Index>(i);
    int64_t offset = 0;
#pragma unroll
    for (int d = 7; d >= 1; --d) {
      if (d < static_cast<int>(view.rank)) {
        const Index extent = static_cast<Index>(view.dims[d]);
        const Index outer = rest / extent;
        offset += static_cast<int64_t>(rest - outer * extent) * view.strides[d];
        rest = outer;
      }
    }
    if (view.rank != 0) offset += static_cast<int64_t>(rest) * view.strides[0];  // what is left is the outermost coordinate
    return *reinterpret_cast<const Word *>(in + offset);
  };
  auto put = [&](uint64_t i, Word word) {
    if constexpr (kCopy) out[i] = word;
    else out[i] = static_cast<typename Element<kDst>::Word>(convert<kSrc, kDst>(word));
  };
  constexpr int kGather = 8;  // independent loads in flight per thread: one element each is latency-bound
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kGather - 1) * stride < count; i += kGather * stride) {
    Word words[kGather];
#pragma unroll
    for (int k = 0; k < kGather; ++k) words[k] = fetch(i + k * stride);
#pragma unroll
    for (int k = 0; k < kGather; ++k) put(i + k * stride, words[k]);
  }
  for (; i < count; i += stride) put(i, fetch(i));
}

// Views whose innermost (merged) axis is long: a CTA-step takes a segment of one innermost run, so the
// offset of the run is computed once per step by the whole CTA and no thread divides per element.
template <class Word, int kSrc, int kDst, bool kCopy>
__global__ void __launch_bounds__(kThreads)
strided_runs_kernel(const unsigned char *__restrict__ in, typename Element<kDst>::Word *__restrict__ out, uint64_t runs,
                    const View view) {
  grid_dependency_sync();
  constexpr int kGather = 8;
  constexpr uint64_t kSegment = static_cast<uint64_t>(kThreads) * kGather;
  const uint64_t inner = view.dims[view.rank - 1];
  const int64_t inner_stride = view.strides[view.rank - 1];
  const uint64_t segments = (inner + kSegment - 1) / kSegment;
  for (uint64_t unit = blockIdx.x; unit < runs * segments; unit += gridDim.x) {
    const uint64_t run = unit / segments, segment = unit - run * segments;
    uint64_t rest = run;
    int64_t offset = 0;
#pragma unroll
    for (int d = 6; d >= 1; --d) {
      if (d + 1 < static_cast<int>(view.rank)) {
        const uint64_t outer = rest / view.dims[d];
        offset += static_cast<int64_t>(rest - outer * view.dims[d]) * view.strides[d];
        rest = outer;
      }
    }
    if (view.rank > 1) offset += static_cast<int64_t>(rest) * view.strides[0];
    const uint64_t first = segment * kSegment + threadIdx.x;
    Word words[kGather];
#pragma unroll
    for (int k = 0; k < kGather; ++k) {
      const uint64_t j = first + static_cast<uint64_t>(k) * kThreads;
      if (j < inner) words[k] = *reinterpret_cast<const Word *>(in + offset + static_cast<int64_t>(j) * inner_stride);
    }
#pragma unroll
    for (int k = 0; k < kGather; ++k) {
      const uint64_t j = first + static_cast<uint64_t>(k) * kThreads;
      if (j < inner) {
        if constexpr (kCopy) out[run * inner + j] = words[k];
        else out[run * inner + j] = static_cast<typename Element<kDst>::Word>(convert<kSrc, kDst>(words[k]));
      }
    }
  }
}

// The same with four consecutive elements per access, for views whose innermost axis is contiguous and
// whose runs start on a boundary of four elements on both sides: 16-byte loads of f32 (8 of 16-bit, 4 of
// 8-bit elements) instead of one element per instruction.
template <class T>
struct alignas(4 * sizeof(T)) Four {
  T v[4];
};
template <class Word, int kSrc, int kDst, bool kCopy>
__global__ void __launch_bounds__(kThreads)
strided_runs4_kernel(const unsigned char *__restrict__ in, typename Element<kDst>::Word *__restrict__ out, uint64_t runs,
                     const View view) {
  grid_dependency_sync();
  using Out = typename Element<kDst>::Word;
  constexpr int kGather = 4;  // 4 x 4 elements in flight per thread
  constexpr uint64_t kSegment = static_cast<uint64_t>(kThreads) * kGather;
  const uint64_t inner = view.dims[view.rank - 1], groups = inner / 4;
  const uint64_t segments = (groups + kSegment - 1) / kSegment;
  for (uint64_t unit = blockIdx.x; unit < runs * segments; unit += gridDim.x) {
    const uint64_t run = unit / segments, segment = unit - run * segments;
    uint64_t rest = run;
    int64_t offset = 0;
#pragma unroll
    for (int d = 6; d >= 1; --d) {
      if (d + 1 < static_cast<int>(view.rank)) {
        const uint64_t outer = rest / view.dims[d];
        offset += static_cast<int64_t>(rest - outer * view.dims[d]) * view.strides[d];
        rest = outer;
      }
    }
    if (view.rank > 1) offset += static_cast<int64_t>(rest) * view.strides[0];
    const Four<Word> *source = reinterpret_cast<const Four<Word> *>(in + offset);
    Four<Out> *destination = reinterpret_cast<Four<Out> *>(out + run * inner);
    const uint64_t first = segment * kSegment + threadIdx.x;
    Four<Word> words[kGather];
#pragma unroll
    for (int k = 0; k < kGather; ++k) {
      const uint64_t j = first + static_cast<uint64_t>(k) * kThreads;
      if (j < groups) words[k] = source[j];
    }
#pragma unroll
    for (int k = 0; k < kGather; ++k) {
      const uint64_t j = first + static_cast<uint64_t>(k) * kThreads;
      if (j < groups) {
        Four<Out> result;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if constexpr (kCopy) result.v[e] = words[k].v[e];
          else result.v[e] = static_cast<Out>(convert<kSrc, kDst>(words[k].v[e]));
        }
        destination[j] = result;
      }
    }
  }
}

// Transposing views: the innermost axis of the view is strided in the source while another axis
// (`axis`) is contiguous there.  A 32 x 32 tile goes through shared memory so that the source is read
// along its contiguous axis and the dense destination is written along its innermost one.
struct Transposition {
  uint32_t axis;          // the view axis whose byte stride equals the element size
  uint64_t dense[8];      // row-major element strides of the dense destination, per view axis
};

template <class Word, int kSrc, int kDst, bool kCopy, class Index>
__global__ void __launch_bounds__(256)
strided_tiles_kernel(const unsigned char *__restrict__ in, typename Element<kDst>::Word *__restrict__ out, uint64_t batches,
                     const View view, const Transposition plan) {
  grid_dependency_sync();
  __shared__ Word tile[32][33];
  const uint32_t inner_axis = view.rank - 1;
  const uint64_t inner = view.dims[inner_axis], across = view.dims[plan.axis];
  const uint64_t tiles_inner = (inner + 31) / 32, tiles_across = (across + 31) / 32;
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const uint64_t units = batches * tiles_inner * tiles_across;
  for (uint64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    // index arithmetic in 32 bits whenever the number of tiles allows: a tile is only 1024 elements
    Index rest = static_cast<Index>(unit);
    const Index after_inner = rest / static_cast<Index>(tiles_inner);
    const uint64_t tile_inner = rest - after_inner * static_cast<Index>(tiles_inner);
    rest = after_inner / static_cast<Index>(tiles_across);
    const uint64_t tile_across = after_inner - rest * static_cast<Index>(tiles_across);
    int64_t source = 0;
    uint64_t destination = 0;
#pragma unroll
    for (int d = 6; d >= 0; --d) {  // the batch index runs over every axis but the two of the tile
      if (d < static_cast<int>(inner_axis) && d != static_cast<int>(plan.axis)) {
        const Index outer = rest / static_cast<Index>(view.dims[d]);
        const uint64_t coordinate = rest - outer * static_cast<Index>(view.dims[d]);
        source += static_cast<int64_t>(coordinate) * view.strides[d];
        destination += coordinate * plan.dense[d];
        rest = outer;
      }
    }
#pragma unroll
    for (int step = 0; step < 4; ++step) {
      const uint64_t j = tile_inner * 32 + ty + step * 8, c = tile_across * 32 + tx;
      if (j < inner && c < across)
        tile[ty + step * 8][tx] = *reinterpret_cast<const Word *>(in + source + static_cast<int64_t>(j) * view.strides[inner_axis] +
                                                                  static_cast<int64_t>(c) * view.strides[plan.axis]);
    }
    __syncthreads();
#pragma unroll
    for (int step = 0; step < 4; ++step) {
      const uint64_t c = tile_across * 32 + ty + step * 8, j = tile_inner * 32 + tx;
      if (j < inner && c < across) {
        const Word word = tile[tx][ty + step * 8];
        const uint64_t at = destination + c * plan.dense[plan.axis] + j;
        if constexpr (kCopy) out[at] = word;
        else out[at] = static_cast<typename Element<kDst>::Word>(convert<kSrc, kDst>(word));
      }
    }
    __syncthreads();
  }
}

// The same transposition for 4-byte source words when everything is 16-byte aligned: 64 x 64 tiles moved
// with 16-byte accesses at every step.  A thread loads a 4 x 4 block (four 16-byte vectors from four
// consecutive source rows, all in flight), transposes it in registers (a renaming), and stores the four
// transposed vectors to shared memory, which holds the tile TRANSPOSED, [across][inner], as 16 groups of
// four words per row; it then reads one group per step along the destination's innermost axis and writes
// 16 bytes (or four converted results) to global memory.  The group index is XORed with (row / 4) % 8, so
// the eight lanes of a quarter warp hit eight different bank groups both when storing (eight rows four
// apart, one group) and when loading (one row, eight groups): no padding, no bank conflict, a quarter of
// the shared-memory instructions of a word-by-word transposition.
template <int kSrc, int kDst, bool kCopy, class Index>
__global__ void __launch_bounds__(256)
strided_tiles64_kernel(const unsigned char *__restrict__ in, typename Element<kDst>::Word *__restrict__ out, uint64_t batches,
                       const View view, const Transposition plan) {
  grid_dependency_sync();
  using Out = typename Element<kDst>::Word;
  __shared__ uint4 tile[64][16];
  const uint32_t inner_axis = view.rank - 1;
  const uint64_t inner = view.dims[inner_axis], across = view.dims[plan.axis];
  const uint64_t tiles_inner = (inner + 63) / 64, tiles_across = (across + 63) / 64;
  const uint64_t units = batches * tiles_inner * tiles_across;
  const int64_t inner_stride = view.strides[inner_axis];
  const uint32_t group = threadIdx.x / 16, member = threadIdx.x % 16;  // block rows 4*group.., block columns 4*member..
  for (uint64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    Index rest = static_cast<Index>(unit);
    const Index after_inner = rest / static_cast<Index>(tiles_inner);
    const uint64_t tile_inner = rest - after_inner * static_cast<Index>(tiles_inner);
    rest = after_inner / static_cast<Index>(tiles_across);
    const uint64_t tile_across = after_inner - rest * static_cast<Index>(tiles_across);
    int64_t source = 0;
    uint64_t destination = 0;
#pragma unroll
    for (int d = 6; d >= 0; --d) {
      if (d < static_cast<int>(inner_axis) && d != static_cast<int>(plan.axis)) {
        const Index outer = rest / static_cast<Index>(view.dims[d]);
        const uint64_t coordinate = rest - outer * static_cast<Index>(view.dims[d]);
        source += static_cast<int64_t>(coordinate) * view.strides[d];
        destination += coordinate * plan.dense[d];
        rest = outer;
      }
    }
    uint4 q[4];
    {
      const uint64_t j = tile_inner * 64 + 4 * group, c = tile_across * 64 + 4 * member;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        q[k] = (j + k < inner && c < across)
                   ? ld_stream(reinterpret_cast<const uint4 *>(in + source + static_cast<int64_t>(j + k) * inner_stride + static_cast<int64_t>(c) * 4))
                   : make_uint4(0, 0, 0, 0);
    }
    // transposed block: row 4*member + m of the transposed tile, group `group` (inner 4*group .. +3)
    const uint32_t swizzle = member & 7;  // ((4 * member + m) / 4) % 8
    tile[4 * member + 0][group ^ swizzle] = make_uint4(q[0].x, q[1].x, q[2].x, q[3].x);
    tile[4 * member + 1][group ^ swizzle] = make_uint4(q[0].y, q[1].y, q[2].y, q[3].y);
    tile[4 * member + 2][group ^ swizzle] = make_uint4(q[0].z, q[1].z, q[2].z, q[3].z);
    tile[4 * member + 3][group ^ swizzle] = make_uint4(q[0].w, q[1].w, q[2].w, q[3].w);
    __syncthreads();
#pragma unroll
    for (int step = 0; step < 4; ++step) {
      const uint32_t c_local = group + 16 * step, j_local = 4 * member;
      const uint64_t c = tile_across * 64 + c_local, j = tile_inner * 64 + j_local;
      if (c < across && j < inner) {
        const uint4 words = tile[c_local][member ^ ((c_local / 4) & 7)];
        const uint32_t word[4] = {words.x, words.y, words.z, words.w};
        struct alignas(4 * sizeof(Out)) Results { Out v[4]; } results;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if constexpr (kCopy) results.v[k] = static_cast<Out>(word[k]);
          else results.v[k] = static_cast<Out>(convert<kSrc, kDst>(word[k]));
        }
        *reinterpret_cast<Results *>(out + destination + c * plan.dense[plan.axis] + j) = results;
      }
    }
    __syncthreads();
  }
}

template <int kSrc, int kDst, bool kCopy>
int launch_strided(cudaStream_t stream, const void *in, void *out, uint64_t count, const View &view) {
  using Word = typename Element<kSrc>::Word;
  using Out = typename Element<kDst>::Word;
  if (view.rank >= 2 && view.dims[view.rank - 1] >= 32 && view.strides[view.rank - 1] != static_cast<int64_t>(sizeof(Word))) {
    Transposition plan{};
    uint64_t dense = 1;
    for (int d = static_cast<int>(view.rank) - 1; d >= 0; --d) {
      plan.dense[d] = dense;
      dense *= view.dims[d];
    }
    int axis = -1;
    for (uint32_t d = 0; d + 1 < view.rank; ++d)
      if (view.strides[d] == static_cast<int64_t>(sizeof(Word)) && view.dims[d] >= 32) axis = static_cast<int>(d);
    if (axis >= 0) {
      plan.axis = static_cast<uint32_t>(axis);
      const uint64_t inner = view.dims[view.rank - 1], across = view.dims[axis];
      const uint64_t batches = count / (inner * across);
      if constexpr (sizeof(Word) == 4) {
        // the vector form: whole 16-byte vectors on both sides
        bool aligned = aligned_to(in, 16) && aligned_to(out, 4 * sizeof(Out)) && inner % 4 == 0 && across % 4 == 0 && inner >= 64 &&
                       across >= 64;
        for (uint32_t d = 0; d < view.rank; ++d)
          if (static_cast<int>(d) != axis) aligned = aligned && view.strides[d] % 16 == 0;
        if (aligned) {
          const uint64_t units64 = batches * ((inner + 63) / 64) * ((across + 63) / 64);
          const unsigned grid64 = clamp_grid(units64, static_cast<uint64_t>(sm_count()) * kCtasPerSm);
          auto tiles64 = units64 <= 0xffffffffull ? strided_tiles64_kernel<kSrc, kDst, kCopy, uint32_t>
                                                  : strided_tiles64_kernel<kSrc, kDst, kCopy, uint64_t>;
          return launch(tiles64, dim3(grid64), dim3(256), 0, stream, static_cast<const unsigned char *>(in), static_cast<Out *>(out),
                        batches, view, plan);
        }
      }
      const uint64_t units = batches * ((inner + 31) / 32) * ((across + 31) / 32);
      const unsigned tile_grid = clamp_grid(units, static_cast<uint64_t>(sm_count()) * kCtasPerSm);
      auto tiles = units <= 0xffffffffull ? strided_tiles_kernel<Word, kSrc, kDst, kCopy, uint32_t>
                                          : strided_tiles_kernel<Word, kSrc, kDst, kCopy, uint64_t>;
      return launch(tiles, dim3(tile_grid), dim3(256), 0, stream, static_cast<const unsigned char *>(in),
                    static_cast<Out *>(out), batches, view, plan);
    }
  }
  if (view.rank != 0 && view.dims[view.rank - 1] >= 256) {
    const uint64_t inner = view.dims[view.rank - 1], runs = count / inner;
    bool fours = view.strides[view.rank - 1] == static_cast<int64_t>(sizeof(Word)) && inner % 4 == 0 &&
                 aligned_to(in, 4 * sizeof(Word)) && aligned_to(out, 4 * sizeof(Out));
    for (uint32_t d = 0; d + 1 < view.rank; ++d) fours = fours && view.strides[d] % static_cast<int64_t>(4 * sizeof(Word)) == 0;
    if (fours) {
      const uint64_t units4 = runs * ((inner / 4 + kThreads * 4 - 1) / (kThreads * 4));
      const unsigned grid4 = clamp_grid(units4, static_cast<uint64_t>(sm_count()) * kCtasPerSm);
      return launch(strided_runs4_kernel<Word, kSrc, kDst, kCopy>, dim3(grid4), dim3(kThreads), 0, stream,
                    static_cast<const unsigned char *>(in), static_cast<Out *>(out), runs, view);
    }
    const uint64_t units = runs * ((inner + kThreads * 8 - 1) / (kThreads * 8));
    const unsigned run_grid = clamp_grid(units, static_cast<uint64_t>(sm_count()) * kCtasPerSm);
    return launch(strided_runs_kernel<Word, kSrc, kDst, kCopy>, dim3(run_grid), dim3(kThreads), 0, stream,
                  static_cast<const unsigned char *>(in), static_cast<Out *>(out), runs, view);
  }
  const unsigned grid = clamp_grid((count + kThreads * 8 - 1) / (kThreads * 8), static_cast<uint64_t>(sm_count()) * kCtasPerSm);
  auto kernel = count <= 0xffffffffull ? strided_kernel<Word, kSrc, kDst, kCopy, uint32_t> : strided_kernel<Word, kSrc, kDst, kCopy, uint64_t>;
  return launch(kernel, dim3(grid), dim3(kThreads), 0, stream, static_cast<const unsigned char *>(in), static_cast<Out *>(out), count,
                view);
}

// ---- dense -> strided view ---------------------------------------------------------------------------
// The mirror of the kernels above for OUTPUTS: an operator's dense result is placed into a destination
// that is a view (a slice of a larger tensor, a permuted layout), as the reference's tensor kernels write
// every output through its byte strides (src/compute_provider_cuda/tensor_kernel.cu:70-108).  Bits are
// moved; the element type is the same on both sides.  `Word` may be wider than the element: when the
// innermost axis is contiguous and everything is 16-byte aligned the host widens elements to uint4.
template <class Word, class Index>
__global__ void __launch_bounds__(kThreads)
scatter_kernel(const Word *__restrict__ in, unsigned char *__restrict__ out, uint64_t count, const View view) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  auto place = [&](uint64_t i, Word word) {
    Index rest = static_cast<Index>(i);
    int64_t offset = 0;
#pragma unroll
    for (int d = 7; d >= 1; --d) {
      if (d < static_cast<int>(view.rank)) {
        const Index extent = static_cast<Index>(view.dims[d]);
        const Index outer = rest / extent;
        offset += static_cast<int64_t>(rest - outer * extent) * view.strides[d];
        rest = outer;
      }
    }
    if (view.rank != 0) offset += static_cast<int64_t>(rest) * view.strides[0];
    *reinterpret_cast<Word *>(out + offset) = word;
  };
  constexpr int kBatch = 8;  // dense loads in flight per thread
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kBatch - 1) * stride < count; i += kBatch * stride) {
    Word words[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) words[k] = in[i + k * stride];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) place(i + k * stride, words[k]);
  }
  for (; i < count; i += stride) place(i, in[i]);
}

// A long innermost axis: a CTA-step takes a segment of one innermost run, its offset computed once.
template <class Word>
__global__ void __launch_bounds__(kThreads)
scatter_runs_kernel(const Word *__restrict__ in, unsigned char *__restrict__ out, uint64_t runs, const View view) {
  grid_dependency_sync();
  constexpr int kBatch = 8;
  constexpr uint64_t kSegment = static_cast<uint64_t>(kThreads) * kBatch;
  const uint64_t inner = view.dims[view.rank - 1];
  const int64_t inner_stride = view.strides[view.rank - 1];
  const uint64_t segments = (inner + kSegment - 1) / kSegment;
  for (uint64_t unit = blockIdx.x; unit < runs * segments; unit += gridDim.x) {
    const uint64_t run = unit / segments, segment = unit - run * segments;
    uint64_t rest = run;
    int64_t offset = 0;
#pragma unroll
    for (int d = 6; d >= 1; --d) {
      if (d + 1 < static_cast<int>(view.rank)) {
        const uint64_t outer = rest / view.dims[d];
        offset += static_cast<int64_t>(rest - outer * view.dims[d]) * view.strides[d];
        rest = outer;
      }
    }
    if (view.rank > 1) offset += static_cast<int64_t>(rest) * view.strides[0];
    const uint64_t first = segment * kSegment + threadIdx.x;
    Word words[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const uint64_t j = first + static_cast<uint64_t>(k) * kThreads;
      if (j < inner) words[k] = in[run * inner + j];
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const uint64_t j = first + static_cast<uint64_t>(k) * kThreads;
      if (j < inner) *reinterpret_cast<Word *>(out + offset + static_cast<int64_t>(j) * inner_stride) = words[k];
    }
  }
}

template <class Word>
int launch_scatter(cudaStream_t stream, const void *in, void *out, uint64_t count, const View &view) {
  if (view.rank != 0 && view.dims[view.rank - 1] >= 256) {
    const uint64_t inner = view.dims[view.rank - 1], runs = count / inner;
    const uint64_t units = runs * ((inner + kThreads * 8 - 1) / (kThreads * 8));
    const unsigned grid = clamp_grid(units, static_cast<uint64_t>(sm_count()) * kCtasPerSm);
    return launch(scatter_runs_kernel<Word>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Word *>(in),
                  static_cast<unsigned char *>(out), runs, view);
  }
  const unsigned grid = clamp_grid((count + kThreads * 8 - 1) / (kThreads * 8), static_cast<uint64_t>(sm_count()) * kCtasPerSm);
  auto kernel = count <= 0xffffffffull ? scatter_kernel<Word, uint32_t> : scatter_kernel<Word, uint64_t>;
  return launch(kernel, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Word *>(in), static_cast<unsigned char *>(out),
                count, view);
}

// Drops axes of extent 1 and merges neighbours that are contiguous with each other.
inline View merged_view(uint32_t rank, const int64_t *dims, const int64_t *byte_strides) {
  View view{};
  for (uint32_t d = 0; d < rank; ++d) {
    if (dims[d] == 1) continue;
    if (view.rank != 0 && view.strides[view.rank - 1] == byte_strides[d] * dims[d]) {
      view.dims[view.rank - 1] *= static_cast<uint64_t>(dims[d]);
      view.strides[view.rank - 1] = byte_strides[d];
    } else {
      view.dims[view.rank] = static_cast<uint64_t>(dims[d]);
      view.strides[view.rank] = byte_strides[d];
      ++view.rank;
    }
  }
  return view;
}

// Bits of `width`-byte elements from a (merged) view into a dense tensor.
inline int copy_from_view(cudaStream_t s, int width, const void *in, void *out, uint64_t count, const View &view) {
  if (view.rank == 0 || (view.rank == 1 && view.strides[0] == width))
    return static_cast<int>(cudaMemcpyAsync(out, in, count * width, cudaMemcpyDeviceToDevice, s));
  if (width == 4) return launch_strided<HYLE_B200_F32, HYLE_B200_F32, true>(s, in, out, count, view);
  if (width == 2) return launch_strided<HYLE_B200_BF16, HYLE_B200_BF16, true>(s, in, out, count, view);
  return launch_strided<HYLE_B200_BOOL, HYLE_B200_BOOL, true>(s, in, out, count, view);
}

inline int element_bytes(int dtype) {
  switch (dtype) {
    case HYLE_B200_F32: case HYLE_B200_I32: return 4;
    case HYLE_B200_BF16: case HYLE_B200_F16: return 2;
    case HYLE_B200_E4M3: case HYLE_B200_E5M2: case HYLE_B200_BOOL: return 1;
    default: return 0;
  }
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" int hyle_b200_cast(hyle_b200_stream_t stream, int source_dtype, int destination_dtype, const void *in,
                              void *out, uint64_t count) {
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr) return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
#define HB_CAST(S, D) \
  if (source_dtype == S && destination_dtype == D) return launch_cast<S, D>(s, in, out, count)
  // the pairs of src/compute_provider_native/cast.cc:128-176
  HB_CAST(HYLE_B200_F32, HYLE_B200_BF16);
  HB_CAST(HYLE_B200_F32, HYLE_B200_F16);
  HB_CAST(HYLE_B200_BF16, HYLE_B200_F32);
  HB_CAST(HYLE_B200_F16, HYLE_B200_F32);
  HB_CAST(HYLE_B200_BF16, HYLE_B200_F16);
  HB_CAST(HYLE_B200_F16, HYLE_B200_BF16);
  HB_CAST(HYLE_B200_I32, HYLE_B200_F32);
  HB_CAST(HYLE_B200_F32, HYLE_B200_BOOL);
  HB_CAST(HYLE_B200_BF16, HYLE_B200_BOOL);
  HB_CAST(HYLE_B200_F16, HYLE_B200_BOOL);
  HB_CAST(HYLE_B200_BOOL, HYLE_B200_F32);
  HB_CAST(HYLE_B200_BOOL, HYLE_B200_BF16);
  HB_CAST(HYLE_B200_BOOL, HYLE_B200_F16);
  HB_CAST(HYLE_B200_F32, HYLE_B200_E4M3);
  HB_CAST(HYLE_B200_BF16, HYLE_B200_E4M3);
  HB_CAST(HYLE_B200_F16, HYLE_B200_E4M3);
  HB_CAST(HYLE_B200_E4M3, HYLE_B200_F32);
  HB_CAST(HYLE_B200_E4M3, HYLE_B200_BF16);
  HB_CAST(HYLE_B200_E4M3, HYLE_B200_F16);
  HB_CAST(HYLE_B200_E5M2, HYLE_B200_BF16);
  HB_CAST(HYLE_B200_E5M2, HYLE_B200_E4M3);
#undef HB_CAST
  return HYLE_B200_NOT_SUPPORTED;
}

extern "C" int hyle_b200_fp8_e4m3_encode(hyle_b200_stream_t stream, int dtype, const void *in, uint64_t count,
                                         float scale, void *out, uint32_t *status_word) {
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr || !(scale > 0.0f) || !(scale < INFINITY)) return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == HYLE_B200_F32) return launch_cache_encode<HYLE_B200_F32>(s, in, out, count, scale, status_word);
  if (dtype == HYLE_B200_BF16) return launch_cache_encode<HYLE_B200_BF16>(s, in, out, count, scale, status_word);
  if (dtype == HYLE_B200_F16) return launch_cache_encode<HYLE_B200_F16>(s, in, out, count, scale, status_word);
  return HYLE_B200_INVALID_VALUE;
}

extern "C" int hyle_b200_select(hyle_b200_stream_t stream, int dtype, const void *condition, const void *when_true,
                                const void *when_false, void *out, uint64_t count, uint64_t true_period,
                                uint64_t false_period) {
  if (count == 0) return HYLE_B200_OK;
  if (condition == nullptr || when_true == nullptr || when_false == nullptr || out == nullptr || true_period == 0 ||
      false_period == 0 || count % true_period != 0 || count % false_period != 0)
    return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == HYLE_B200_F32 || dtype == HYLE_B200_I32)
    return launch_select<4>(s, condition, when_true, when_false, out, count, true_period, false_period);
  if (dtype == HYLE_B200_BF16 || dtype == HYLE_B200_F16)
    return launch_select<2>(s, condition, when_true, when_false, out, count, true_period, false_period);
  return HYLE_B200_INVALID_VALUE;
}

extern "C" int hyle_b200_strided_cast(hyle_b200_stream_t stream, int source_dtype, int destination_dtype, const void *in,
                                      void *out, uint32_t rank, const int64_t *dims, const int64_t *byte_strides) {
  const int width = element_bytes(source_dtype), out_width = element_bytes(destination_dtype);
  if (width == 0 || out_width == 0) return HYLE_B200_NOT_SUPPORTED;
  if (rank > 8 || (rank != 0 && (dims == nullptr || byte_strides == nullptr))) return HYLE_B200_INVALID_VALUE;
  uint64_t count = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    if (dims[d] < 0 || byte_strides[d] % width != 0) return HYLE_B200_INVALID_VALUE;
    if (dims[d] != 0 && count > 0xffffffffffffffffull / static_cast<uint64_t>(dims[d])) return HYLE_B200_INVALID_VALUE;
    count *= static_cast<uint64_t>(dims[d]);
  }
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr || !aligned_to(in, width) || !aligned_to(out, out_width)) return HYLE_B200_INVALID_VALUE;
  const View view = merged_view(rank, dims, byte_strides);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const bool dense = view.rank == 0 || (view.rank == 1 && view.strides[0] == width);
  if (source_dtype == destination_dtype) return copy_from_view(s, width, in, out, count, view);
  if (dense) return hyle_b200_cast(stream, source_dtype, destination_dtype, in, out, count);
#define HB_STRIDED(S, D) \
  if (source_dtype == S && destination_dtype == D) return launch_strided<S, D, false>(s, in, out, count, view)
  HB_STRIDED(HYLE_B200_F32, HYLE_B200_BF16);
  HB_STRIDED(HYLE_B200_F32, HYLE_B200_F16);
  HB_STRIDED(HYLE_B200_BF16, HYLE_B200_F32);
  HB_STRIDED(HYLE_B200_F16, HYLE_B200_F32);
  HB_STRIDED(HYLE_B200_BF16, HYLE_B200_F16);
  HB_STRIDED(HYLE_B200_F16, HYLE_B200_BF16);
  HB_STRIDED(HYLE_B200_I32, HYLE_B200_F32);
  HB_STRIDED(HYLE_B200_F32, HYLE_B200_BOOL);
  HB_STRIDED(HYLE_B200_BF16, HYLE_B200_BOOL);
  HB_STRIDED(HYLE_B200_F16, HYLE_B200_BOOL);
  HB_STRIDED(HYLE_B200_BOOL, HYLE_B200_F32);
  HB_STRIDED(HYLE_B200_BOOL, HYLE_B200_BF16);
  HB_STRIDED(HYLE_B200_BOOL, HYLE_B200_F16);
  HB_STRIDED(HYLE_B200_F32, HYLE_B200_E4M3);
  HB_STRIDED(HYLE_B200_BF16, HYLE_B200_E4M3);
  HB_STRIDED(HYLE_B200_F16, HYLE_B200_E4M3);
  HB_STRIDED(HYLE_B200_E4M3, HYLE_B200_F32);
  HB_STRIDED(HYLE_B200_E4M3, HYLE_B200_BF16);
  HB_STRIDED(HYLE_B200_E4M3, HYLE_B200_F16);
  HB_STRIDED(HYLE_B200_E5M2, HYLE_B200_BF16);
  HB_STRIDED(HYLE_B200_E5M2, HYLE_B200_E4M3);
#undef HB_STRIDED
  return HYLE_B200_NOT_SUPPORTED;
}

extern "C" int hyle_b200_strided_scatter(hyle_b200_stream_t stream, int dtype, const void *in, void *out, uint32_t rank,
                                         const int64_t *dims, const int64_t *byte_strides) {
  const int width = element_bytes(dtype);
  if (width == 0) return HYLE_B200_NOT_SUPPORTED;
  if (rank > 8 || (rank != 0 && (dims == nullptr || byte_strides == nullptr))) return HYLE_B200_INVALID_VALUE;
  uint64_t count = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    if (dims[d] < 0 || byte_strides[d] % width != 0) return HYLE_B200_INVALID_VALUE;
    if (dims[d] > 1 && byte_strides[d] == 0) return HYLE_B200_INVALID_VALUE;  // two elements at one address
    if (dims[d] != 0 && count > 0xffffffffffffffffull / static_cast<uint64_t>(dims[d])) return HYLE_B200_INVALID_VALUE;
    count *= static_cast<uint64_t>(dims[d]);
  }
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr || !aligned_to(in, width) || !aligned_to(out, width)) return HYLE_B200_INVALID_VALUE;
  View view = merged_view(rank, dims, byte_strides);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (view.rank == 0 || (view.rank == 1 && view.strides[0] == width))
    return static_cast<int>(cudaMemcpyAsync(out, in, count * width, cudaMemcpyDeviceToDevice, s));
  // A destination that is dense in a PERMUTED axis order (a transposed layout without gaps) is the same
  // move seen from the other side: its storage, walked in its own order, reads the dense source through
  // permuted strides -- the gathering kernels above, with their shared-memory tiles for transpositions.
  {
    uint32_t order[8];
    for (uint32_t d = 0; d < view.rank; ++d) order[d] = d;
    for (uint32_t a = 1; a < view.rank; ++a)  // insertion sort, largest destination stride first
      for (uint32_t b = a; b > 0 && view.strides[order[b]] > view.strides[order[b - 1]]; --b) {
        const uint32_t t = order[b];
        order[b] = order[b - 1];
        order[b - 1] = t;
      }
    bool permutation = view.strides[order[view.rank - 1]] == width;
    for (uint32_t a = 0; permutation && a + 1 < view.rank; ++a)
      permutation = view.strides[order[a]] == view.strides[order[a + 1]] * static_cast<int64_t>(view.dims[order[a + 1]]);
    if (permutation) {
      int64_t source_stride[8];  // of the dense source, per axis of the merged view
      int64_t running = width;
      for (int d = static_cast<int>(view.rank) - 1; d >= 0; --d) {
        source_stride[d] = running;
        running *= static_cast<int64_t>(view.dims[d]);
      }
      int64_t turned_dims[8], turned_strides[8];
      for (uint32_t a = 0; a < view.rank; ++a) {
        turned_dims[a] = static_cast<int64_t>(view.dims[order[a]]);
        turned_strides[a] = source_stride[order[a]];
      }
      return copy_from_view(s, width, in, out, count, merged_view(view.rank, turned_dims, turned_strides));
    }
  }
  // Contiguous innermost runs of whole, aligned 16-byte groups move as uint4.
  const uint32_t last = view.rank - 1;
  bool wide = view.strides[last] == width && (view.dims[last] * width) % 16 == 0 && aligned_to(in, 16) && aligned_to(out, 16);
  for (uint32_t d = 0; d < last; ++d) wide = wide && view.strides[d] % 16 == 0;
  if (wide) {
    view.dims[last] = view.dims[last] * width / 16;
    view.strides[last] = 16;
    return launch_scatter<uint4>(s, in, out, count * width / 16, view);
  }
  if (width == 4) return launch_scatter<uint32_t>(s, in, out, count, view);
  if (width == 2) return launch_scatter<uint16_t>(s, in, out, count, view);
  return launch_scatter<uint8_t>(s, in, out, count, view);
}

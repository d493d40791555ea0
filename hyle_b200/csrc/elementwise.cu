// Streaming elementwise operators: Unary{13 kinds}, Binary{all six kinds} with trailing-axis broadcast,
// GatedActivation{kSilu} (SwiGLU) and Cast{f32->bf16}.  All are HBM-bound: every thread keeps
// several independent 16-byte loads in flight, computes in f32 and writes 16-byte vectors.
#include "common.cuh"

namespace hb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;       // independent 16-byte vectors in flight per thread and operand
constexpr int kCtasPerSm = 8;    // 8 x 256 threads fill an SM

// ---- element math --------------------------------------------------------------------------------
template <int kKind>
__device__ __forceinline__ float binary_op(float a, float b) {
  if constexpr (kKind == HYLE_B200_BINARY_ADD) return __fadd_rn(a, b);
  if constexpr (kKind == HYLE_B200_BINARY_MULTIPLY) return __fmul_rn(a, b);
  if constexpr (kKind == HYLE_B200_BINARY_SUBTRACT) return __fsub_rn(a, b);
  if constexpr (kKind == HYLE_B200_BINARY_DIVIDE) return __fdiv_rn(a, b);
  // Number minimum / maximum.  fminf / fmaxf return the other operand for one NaN; for two zeros
  // the sign is fixed by hand: OR of the sign bits for the minimum, AND for the maximum.
  if constexpr (kKind == HYLE_B200_BINARY_MINIMUM) {
    const float r = fminf(a, b);
    return (a == 0.0f && b == 0.0f) ? __uint_as_float(__float_as_uint(a) | __float_as_uint(b)) : r;
  }
  const float r = fmaxf(a, b);
  return (a == 0.0f && b == 0.0f) ? __uint_as_float(__float_as_uint(a) & __float_as_uint(b)) : r;
}

template <int kKind>
__device__ __forceinline__ float4 binary_vec(float4 a, float4 b) {
  return make_float4(binary_op<kKind>(a.x, b.x), binary_op<kKind>(a.y, b.y),
                     binary_op<kKind>(a.z, b.z), binary_op<kKind>(a.w, b.w));
}

template <int kDtype>
__device__ __forceinline__ float narrow_lo(uint32_t w) {
  if constexpr (kDtype == HYLE_B200_BF16) return bf16_lo(w);
  return f16_to_f32(static_cast<unsigned short>(w & 0xffffu));
}
template <int kDtype>
__device__ __forceinline__ float narrow_hi(uint32_t w) {
  if constexpr (kDtype == HYLE_B200_BF16) return bf16_hi(w);
  return f16_to_f32(static_cast<unsigned short>(w >> 16));
}
template <int kDtype>
__device__ __forceinline__ uint32_t narrow_pack(float lo, float hi) {
  if constexpr (kDtype == HYLE_B200_BF16) return pack_bf16x2(lo, hi);
  return pack_f16x2(lo, hi);
}
template <int kDtype>
__device__ __forceinline__ float narrow_scalar(unsigned short s) {
  if constexpr (kDtype == HYLE_B200_BF16) return bf16_to_f32(s);
  return f16_to_f32(s);
}
template <int kDtype>
__device__ __forceinline__ unsigned short narrow_store(float v) {
  if constexpr (kDtype == HYLE_B200_BF16) return f32_to_bf16(v);
  return f32_to_f16(v);
}

// f32 operation on packed 16-bit pairs, one rounding back to storage (docs/user/compute.md:358-359).
template <int kKind, int kDtype>
__device__ __forceinline__ uint32_t binary_pair(uint32_t a, uint32_t b) {
  return narrow_pack<kDtype>(binary_op<kKind>(narrow_lo<kDtype>(a), narrow_lo<kDtype>(b)),
                             binary_op<kKind>(narrow_hi<kDtype>(a), narrow_hi<kDtype>(b)));
}
template <int kKind, int kDtype>
__device__ __forceinline__ uint4 binary_vec(uint4 a, uint4 b) {
  return make_uint4(binary_pair<kKind, kDtype>(a.x, b.x), binary_pair<kKind, kDtype>(a.y, b.y),
                    binary_pair<kKind, kDtype>(a.z, b.z), binary_pair<kKind, kDtype>(a.w, b.w));
}

template <int kKind, int kDtype, class Vec>
__device__ __forceinline__ Vec apply_vec(Vec a, Vec b) {
  if constexpr (kDtype == HYLE_B200_F32) {
    return binary_vec<kKind>(a, b);
  } else {
    return binary_vec<kKind, kDtype>(a, b);
  }
}

template <int kDtype> struct Storage { using Vec = uint4; using Scalar = unsigned short; };
template <> struct Storage<HYLE_B200_F32> { using Vec = float4; using Scalar = float; };

// ---- Binary, same shape: flat stream over 16-byte vectors ------------------------------------------
template <int kKind, int kDtype>
__global__ void __launch_bounds__(kThreads)
binary_flat_kernel(const typename Storage<kDtype>::Vec *lhs,
                   const typename Storage<kDtype>::Vec *__restrict__ rhs,
                   typename Storage<kDtype>::Vec *out, uint64_t vectors) {
  grid_dependency_sync();
  using Vec = typename Storage<kDtype>::Vec;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < vectors; i += kUnroll * stride) {
    Vec a[kUnroll], b[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      a[k] = ld_stream(lhs + i + k * stride);
      b[k] = ld_stream(rhs + i + k * stride);
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k)
      st_stream(out + i + k * stride, apply_vec<kKind, kDtype>(a[k], b[k]));
  }
  for (; i < vectors; i += stride)
    st_stream(out + i, apply_vec<kKind, kDtype>(ld_stream(lhs + i), ld_stream(rhs + i)));
}

// ---- Binary, right operand is one row repeated (bias over rows) -----------------------------------
// The grid is (column tiles, row groups).  A thread owns one 16-byte column slot: the bias vector is
// read once into registers and reused for every row the CTA walks, so the only HBM streams are lhs
// and out, and no per-element index arithmetic remains.
template <int kKind, int kDtype>
__global__ void __launch_bounds__(kThreads)
binary_rowvec_kernel(const typename Storage<kDtype>::Vec *lhs,
                     const typename Storage<kDtype>::Vec *__restrict__ rhs,
                     typename Storage<kDtype>::Vec *out, uint64_t rows,
                     uint32_t row_vectors) {
  grid_dependency_sync();
  using Vec = typename Storage<kDtype>::Vec;
  const uint32_t column = blockIdx.x * kThreads + threadIdx.x;
  if (column >= row_vectors) return;
  const Vec bias = __ldg(rhs + column);
  const uint64_t step = gridDim.y;
  uint64_t row = blockIdx.y;
  for (; row + (kUnroll - 1) * step < rows; row += kUnroll * step) {
    Vec a[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) a[k] = ld_stream(lhs + (row + k * step) * row_vectors + column);
#pragma unroll
    for (int k = 0; k < kUnroll; ++k)
      st_stream(out + (row + k * step) * row_vectors + column, apply_vec<kKind, kDtype>(a[k], bias));
  }
  for (; row < rows; row += step)
    st_stream(out + row * row_vectors + column,
              apply_vec<kKind, kDtype>(ld_stream(lhs + row * row_vectors + column), bias));
}

// ---- Binary, any period / any alignment: one element per thread-iteration --------------------------
template <int kKind, int kDtype>
__global__ void __launch_bounds__(kThreads)
binary_scalar_kernel(const typename Storage<kDtype>::Scalar *lhs,
                     const typename Storage<kDtype>::Scalar *__restrict__ rhs,
                     typename Storage<kDtype>::Scalar *out, uint64_t count,
                     uint64_t period) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count;
       i += stride) {
    const uint64_t j = period == count ? i : (count <= 0xffffffffull
                                                  ? static_cast<uint32_t>(i) % static_cast<uint32_t>(period)
                                                  : i % period);
    if constexpr (kDtype == HYLE_B200_F32) {
      out[i] = binary_op<kKind>(lhs[i], rhs[j]);
    } else {
      out[i] = narrow_store<kDtype>(
          binary_op<kKind>(narrow_scalar<kDtype>(lhs[i]), narrow_scalar<kDtype>(rhs[j])));
    }
  }
}

template <int kKind, int kDtype>
int launch_binary(cudaStream_t stream, const void *lhs, const void *rhs, void *out, uint64_t count,
                  uint64_t period) {
  using Vec = typename Storage<kDtype>::Vec;
  using Scalar = typename Storage<kDtype>::Scalar;
  constexpr uint64_t kLanes = sizeof(Vec) / sizeof(Scalar);
  const bool vector_ok = aligned_to(lhs, 16) && aligned_to(rhs, 16) && aligned_to(out, 16) &&
                         count % kLanes == 0 && period % kLanes == 0;
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  if (vector_ok && period == count) {
    const uint64_t vectors = count / kLanes;
    const unsigned grid = clamp_grid((vectors + kThreads * kUnroll - 1) / (kThreads * kUnroll), resident);
    return launch(binary_flat_kernel<kKind, kDtype>, dim3(grid), dim3(kThreads), 0, stream, 
        static_cast<const Vec *>(lhs), static_cast<const Vec *>(rhs), static_cast<Vec *>(out), vectors);
  }
  const uint64_t row_vectors = period / kLanes;
  if (vector_ok && row_vectors >= 64 && row_vectors <= 0x7fffffffull) {
    const uint64_t rows = count / period;
    const unsigned tiles = static_cast<unsigned>((row_vectors + kThreads - 1) / kThreads);
    // Enough row groups to fill the machine, never more than rows/unroll so the main loop runs.
    uint64_t groups = (resident + tiles - 1) / tiles;
    const uint64_t useful = (rows + kUnroll - 1) / kUnroll;
    if (groups > useful) groups = useful;
    if (groups > 65535) groups = 65535;
    if (groups < 1) groups = 1;
    return launch(binary_rowvec_kernel<kKind, kDtype>, dim3(dim3(tiles, static_cast<unsigned>(groups))), dim3(kThreads), 0, stream, 
        static_cast<const Vec *>(lhs), static_cast<const Vec *>(rhs), static_cast<Vec *>(out), rows,
        static_cast<uint32_t>(row_vectors));
  }
  const unsigned grid = clamp_grid((count + kThreads - 1) / kThreads, resident);
  return launch(binary_scalar_kernel<kKind, kDtype>, dim3(grid), dim3(kThreads), 0, stream, 
      static_cast<const Scalar *>(lhs), static_cast<const Scalar *>(rhs), static_cast<Scalar *>(out),
      count, period);
}

// ---- Unary ---------------------------------------------------------------------------------------
// Element math follows the scalar route of the reference: libm calls for Exp/Log/Sqrt/Tanh,
// 1.0f / sqrt(x) for Rsqrt (src/compute_provider_native/elementwise.cc:30-55), the overflow-free
// sigmoid and the GELU / SiLU definitions of src/simd/math/activations.cc:21-47 (silu(-inf) =
// gelu(-inf) = 0, NaN propagates), ReLU keeping NaN (:49-52), Softplus = log1p(exp(x)) with the
// identity above 20 (src/compute_provider_native/aten_cpu_provider.cc:627-628).  Abs, Neg, Sqrt,
// Rsqrt and ReLU are bit-exact; the transcendental ones use CUDA's full-accuracy single-precision
// functions (1-2 ulp), well inside the 1e-5 relative bound of the parity tests.
__device__ __forceinline__ float sigmoid_exact(float x) {
  const float e = expf(-fabsf(x));
  return x < 0.0f ? __fdiv_rn(e, 1.0f + e) : __fdiv_rn(1.0f, 1.0f + e);  // NaN falls through both compares
}

// sigmoid to about 1e-6 relative in five instructions, for results that are rounded to 16-bit storage
// anyway: sigmoid(x) = 1 / (1 + 2^-t), t = x log2 e, evaluated as 2^-16 / (2^-16 + 2^(-t - 16)).  The
// bias of 2^-16 keeps the exponential finite down to t = -144, so the quotient still resolves the
// sigmoid where the CPU's expf underflows gradually (a 16-bit result of x * sigmoid(x) is zero below
// that), and no branch or select separates the two signs of x.  Returns r with sigmoid(x) = r * 2^-16
// (a sigmoid below 2^-126 is an f32 subnormal with fewer bits, still more than the 16-bit result keeps).
// NaN propagates; -inf gives r = 0, +inf gives r = 2^16.
constexpr float kSigmoidUnbias = 1.52587890625e-05f;  // 2^-16
__device__ __forceinline__ float sigmoid_reciprocal(float x) {
  constexpr float kLog2e = 1.4426950408889634f;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(x, -kLog2e, -16.0f)));
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fadd_rn(e, kSigmoidUnbias)));
  return r;
}
__device__ __forceinline__ float sigmoid_fast(float x) { return __fmul_rn(sigmoid_reciprocal(x), kSigmoidUnbias); }
// x * sigmoid(x) with silu(-inf) = 0: the argument is held at -150 from below (max.NaN keeps a NaN), where
// the sigmoid is zero already, so -inf * 0 never forms and no select is needed.
__device__ __forceinline__ float silu_fast(float x) {
  const float held = max_nan(x, -150.0f);
  return __fmul_rn(held, sigmoid_fast(held));
}

// kFast (16-bit storage): the sigmoid-shaped kinds go through sigmoid_reciprocal.  tanh(|x|) = 2 s(2|x|) - 1
// cancels near zero, where the odd series takes over; gelu_tanh = x s(2 inner) needs no 1 + tanh.
template <int kKind, bool kFast>
__device__ __forceinline__ float unary_op(float x) {
  if constexpr (kFast && kKind == HYLE_B200_UNARY_SIGMOID) return sigmoid_fast(x);
  if constexpr (kFast && kKind == HYLE_B200_UNARY_SILU) return silu_fast(x);
  if constexpr (kFast && kKind == HYLE_B200_UNARY_GELU_TANH) {
    // 2 inner = 2 * 0.7978845608 * x * (1 + 0.044715 x^2) = x * (c1 + c2 x^2); the argument is held at -1e4
    // from below, where the sigmoid is zero already (gelu(-inf) = 0 without a select)
    const float held = max_nan(x, -1.0e4f);
    const float twice_inner = __fmul_rn(held, fmaf(0.07135481627f, __fmul_rn(held, held), 1.59576912161f));
    return __fmul_rn(held, sigmoid_fast(twice_inner));
  }
  if constexpr (kFast && kKind == HYLE_B200_UNARY_TANH) {
    const float a = fabsf(x), a2 = a * a;
    const float series = a * fmaf(a2, fmaf(a2, 0.13333333333f, -0.33333333333f), 1.0f);
    const float large = fmaf(2.0f, sigmoid_fast(2.0f * a), -1.0f);
    return copysignf(a < 0.04f ? series : large, x);  // NaN: both candidates are NaN
  }
  if constexpr (kKind == HYLE_B200_UNARY_ABS) return fabsf(x);
  if constexpr (kKind == HYLE_B200_UNARY_NEG) return -x;
  if constexpr (kKind == HYLE_B200_UNARY_EXP) return expf(x);
  if constexpr (kKind == HYLE_B200_UNARY_LOG) return logf(x);
  if constexpr (kKind == HYLE_B200_UNARY_SQRT) return __fsqrt_rn(x);
  if constexpr (kKind == HYLE_B200_UNARY_RSQRT) return __fdiv_rn(1.0f, __fsqrt_rn(x));
  if constexpr (kKind == HYLE_B200_UNARY_TANH) return tanhf(x);
  if constexpr (kKind == HYLE_B200_UNARY_SIGMOID) return sigmoid_exact(x);
  if constexpr (kKind == HYLE_B200_UNARY_RELU) return x != x ? x : (x > 0.0f ? x : 0.0f);
  if constexpr (kKind == HYLE_B200_UNARY_GELU)
    return x == -INFINITY ? 0.0f : 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  if constexpr (kKind == HYLE_B200_UNARY_GELU_TANH) {
    if (x == -INFINITY) return 0.0f;
    const float inner = 0.79788456080286535588f * x * fmaf(0.044715f, x * x, 1.0f);
    return 0.5f * x * (1.0f + tanhf(inner));
  }
  if constexpr (kKind == HYLE_B200_UNARY_SILU) return x == -INFINITY ? 0.0f : x * sigmoid_exact(x);
  return x > 20.0f ? x : log1pf(expf(x));  // Softplus; NaN compares false and propagates through expf
}

template <int kKind, int kDtype, class Vec>
__device__ __forceinline__ Vec unary_vec(Vec a) {
  if constexpr (kDtype == HYLE_B200_F32) {
    return make_float4(unary_op<kKind, false>(a.x), unary_op<kKind, false>(a.y), unary_op<kKind, false>(a.z), unary_op<kKind, false>(a.w));
  } else {
    auto pair = [](uint32_t w) {
      return narrow_pack<kDtype>(unary_op<kKind, true>(narrow_lo<kDtype>(w)), unary_op<kKind, true>(narrow_hi<kDtype>(w)));
    };
    return make_uint4(pair(a.x), pair(a.y), pair(a.z), pair(a.w));
  }
}

template <int kKind, int kDtype>
__global__ void __launch_bounds__(kThreads)
unary_flat_kernel(const typename Storage<kDtype>::Vec *in, typename Storage<kDtype>::Vec *out, uint64_t vectors) {
  grid_dependency_sync();
  using Vec = typename Storage<kDtype>::Vec;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < vectors; i += kUnroll * stride) {
    Vec a[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) a[k] = ld_stream(in + i + k * stride);
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) st_stream(out + i + k * stride, unary_vec<kKind, kDtype>(a[k]));
  }
  for (; i < vectors; i += stride) st_stream(out + i, unary_vec<kKind, kDtype>(ld_stream(in + i)));
}

// Unaligned tensors and the tail behind the last whole vector.
template <int kKind, int kDtype>
__global__ void __launch_bounds__(kThreads)
unary_scalar_kernel(const typename Storage<kDtype>::Scalar *in, typename Storage<kDtype>::Scalar *out, uint64_t count) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride) {
    if constexpr (kDtype == HYLE_B200_F32) out[i] = unary_op<kKind, false>(in[i]);
    else out[i] = narrow_store<kDtype>(unary_op<kKind, true>(narrow_scalar<kDtype>(in[i])));
  }
}

template <int kKind, int kDtype>
int launch_unary(cudaStream_t stream, const void *in, void *out, uint64_t count) {
  using Vec = typename Storage<kDtype>::Vec;
  using Scalar = typename Storage<kDtype>::Scalar;
  constexpr uint64_t kLanes = sizeof(Vec) / sizeof(Scalar);
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  const bool vector_ok = aligned_to(in, 16) && aligned_to(out, 16);
  const uint64_t vectors = vector_ok ? count / kLanes : 0;
  if (vectors != 0) {
    const unsigned grid = clamp_grid((vectors + kThreads * kUnroll - 1) / (kThreads * kUnroll), resident);
    const int status = launch(unary_flat_kernel<kKind, kDtype>, dim3(grid), dim3(kThreads), 0, stream,
                              static_cast<const Vec *>(in), static_cast<Vec *>(out), vectors);
    if (status != HYLE_B200_OK) return status;
  }
  const uint64_t done = vectors * kLanes;
  if (done == count) return HYLE_B200_OK;
  const unsigned grid = clamp_grid((count - done + kThreads - 1) / kThreads, resident);
  return launch(unary_scalar_kernel<kKind, kDtype>, dim3(grid), dim3(kThreads), 0, stream,
                static_cast<const Scalar *>(in) + done, static_cast<Scalar *>(out) + done, count - done);
}

// ---- SwiGLU --------------------------------------------------------------------------------------
// silu(x) = x * sigmoid(x) with the overflow-free sigmoid of src/simd/math/activations.cc:21-25:
// e = exp(-|x|); sigmoid = x < 0 ? e/(1+e) : 1/(1+e); silu(-inf) = 0 (:44-47).
//
// About ten instructions per element, two of them on the special-function unit: see sigmoid_reciprocal
// above.  Accuracy: about 1e-6 relative, i.e. the result differs from the checker only when the bf16
// rounding is within that distance of a tie.
__device__ __forceinline__ float silu(float x) { return silu_fast(x); }

// GatedActivation{activation}: out = storage(act(f32 gate) * f32 up), one rounding
// (src/compute_provider_native/aten_cpu_provider.cc:414-445,654-665).  With kRoundGate the activated
// gate is first rounded to the storage type, which makes the result that of Unary{activation}
// followed by Binary{kMultiply} on 16-bit tensors (two roundings): the form a graph region takes when
// it fuses those two nodes without changing what they compute.
template <int kAct>
__device__ __forceinline__ float gate_activation(float x) {
  if constexpr (kAct == HYLE_B200_GATE_SILU) return silu(x);
  if constexpr (kAct == HYLE_B200_GATE_GELU) return unary_op<HYLE_B200_UNARY_GELU, true>(x);
  return unary_op<HYLE_B200_UNARY_GELU_TANH, true>(x);
}
template <int kAct, int kDtype, bool kRoundGate>
__device__ __forceinline__ float gated_value(float g, float u) {
  float a = gate_activation<kAct>(g);
  if constexpr (kRoundGate) a = narrow_scalar<kDtype>(narrow_store<kDtype>(a));
  return __fmul_rn(a, u);
}
template <int kAct, int kDtype, bool kRoundGate>
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t g, uint32_t u) {
  return narrow_pack<kDtype>(gated_value<kAct, kDtype, kRoundGate>(narrow_lo<kDtype>(g), narrow_lo<kDtype>(u)),
                             gated_value<kAct, kDtype, kRoundGate>(narrow_hi<kDtype>(g), narrow_hi<kDtype>(u)));
}
template <int kAct, int kDtype, bool kRoundGate>
__device__ __forceinline__ uint4 swiglu_vec(uint4 g, uint4 u) {
  return make_uint4(swiglu_pair<kAct, kDtype, kRoundGate>(g.x, u.x), swiglu_pair<kAct, kDtype, kRoundGate>(g.y, u.y),
                    swiglu_pair<kAct, kDtype, kRoundGate>(g.z, u.z), swiglu_pair<kAct, kDtype, kRoundGate>(g.w, u.w));
}

// Dense separate gate/up: one flat stream.
template <int kAct, int kDtype, bool kRoundGate>
__global__ void __launch_bounds__(kThreads)
swiglu_flat_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ up,
                   uint4 *__restrict__ out, uint64_t vectors) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < vectors; i += kUnroll * stride) {
    uint4 g[kUnroll], u[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      g[k] = ld_stream(gate + i + k * stride);
      u[k] = ld_stream(up + i + k * stride);
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) st_stream(out + i + k * stride, swiglu_vec<kAct, kDtype, kRoundGate>(g[k], u[k]));
  }
  for (; i < vectors; i += stride)
    st_stream(out + i, swiglu_vec<kAct, kDtype, kRoundGate>(ld_stream(gate + i), ld_stream(up + i)));
}

// Row-strided operands (the packed-halves layout): grid = (column tiles, row groups).
template <int kAct, int kDtype, bool kRoundGate>
__global__ void __launch_bounds__(kThreads)
swiglu_rows_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ up,
                   uint4 *__restrict__ out, uint64_t rows, uint32_t row_vectors,
                   uint64_t gate_stride_vectors, uint64_t up_stride_vectors) {
  grid_dependency_sync();
  const uint32_t column = blockIdx.x * kThreads + threadIdx.x;
  if (column >= row_vectors) return;
  const uint64_t step = gridDim.y;
  uint64_t row = blockIdx.y;
  for (; row + (kUnroll - 1) * step < rows; row += kUnroll * step) {
    uint4 g[kUnroll], u[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      g[k] = ld_stream(gate + (row + k * step) * gate_stride_vectors + column);
      u[k] = ld_stream(up + (row + k * step) * up_stride_vectors + column);
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k)
      st_stream(out + (row + k * step) * row_vectors + column, swiglu_vec<kAct, kDtype, kRoundGate>(g[k], u[k]));
  }
  for (; row < rows; row += step)
    st_stream(out + row * row_vectors + column,
              swiglu_vec<kAct, kDtype, kRoundGate>(ld_stream(gate + row * gate_stride_vectors + column),
                                                   ld_stream(up + row * up_stride_vectors + column)));
}

// Any width / alignment.
template <int kAct, int kDtype, bool kRoundGate>
__global__ void __launch_bounds__(kThreads)
swiglu_scalar_kernel(const unsigned short *__restrict__ gate, const unsigned short *__restrict__ up,
                     unsigned short *__restrict__ out, uint64_t rows, uint64_t cols,
                     uint64_t gate_stride, uint64_t up_stride) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  const uint64_t count = rows * cols;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count;
       i += stride) {
    const uint64_t row = i / cols, column = i - row * cols;
    const float g = narrow_scalar<kDtype>(gate[row * gate_stride + column]);
    const float u = narrow_scalar<kDtype>(up[row * up_stride + column]);
    out[i] = narrow_store<kDtype>(gated_value<kAct, kDtype, kRoundGate>(g, u));
  }
}

// ---- Cast f32 -> bf16 -----------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
cast_f32_bf16_kernel(const float4 *__restrict__ in, uint4 *__restrict__ out, uint64_t vectors) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < vectors; i += kUnroll * stride) {
    float4 a[kUnroll], b[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      a[k] = ld_stream(in + 2 * (i + k * stride));
      b[k] = ld_stream(in + 2 * (i + k * stride) + 1);
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k)
      st_stream(out + i + k * stride,
                make_uint4(pack_bf16x2(a[k].x, a[k].y), pack_bf16x2(a[k].z, a[k].w),
                           pack_bf16x2(b[k].x, b[k].y), pack_bf16x2(b[k].z, b[k].w)));
  }
  for (; i < vectors; i += stride) {
    const float4 a = ld_stream(in + 2 * i), b = ld_stream(in + 2 * i + 1);
    st_stream(out + i, make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w),
                                  pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w)));
  }
}

__global__ void __launch_bounds__(kThreads)
cast_f32_bf16_scalar_kernel(const float *__restrict__ in, unsigned short *__restrict__ out,
                            uint64_t count) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride)
    out[i] = f32_to_bf16(in[i]);
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" int hyle_b200_binary(hyle_b200_stream_t stream, int kind, int dtype, const void *lhs,
                                const void *rhs, void *out, uint64_t count, uint64_t rhs_period) {
  if (count == 0) return HYLE_B200_OK;
  if (lhs == nullptr || rhs == nullptr || out == nullptr || rhs_period == 0 ||
      count % rhs_period != 0)
    return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
#define HB_BINARY_CASE(K, D) \
  if (kind == K && dtype == D) return launch_binary<K, D>(s, lhs, rhs, out, count, rhs_period)
#define HB_BINARY_KIND(K) \
  HB_BINARY_CASE(K, HYLE_B200_F32); \
  HB_BINARY_CASE(K, HYLE_B200_BF16); \
  HB_BINARY_CASE(K, HYLE_B200_F16)
  HB_BINARY_KIND(HYLE_B200_BINARY_ADD);
  HB_BINARY_KIND(HYLE_B200_BINARY_MULTIPLY);
  HB_BINARY_KIND(HYLE_B200_BINARY_SUBTRACT);
  HB_BINARY_KIND(HYLE_B200_BINARY_DIVIDE);
  HB_BINARY_KIND(HYLE_B200_BINARY_MINIMUM);
  HB_BINARY_KIND(HYLE_B200_BINARY_MAXIMUM);
#undef HB_BINARY_KIND
#undef HB_BINARY_CASE
  return HYLE_B200_INVALID_VALUE;
}

namespace hb {
namespace {
template <int kAct, int kDtype, bool kRoundGate>
int launch_gated(cudaStream_t s, const void *gate, const void *up, void *out, uint64_t rows, uint64_t cols,
                 uint64_t gate_row_stride, uint64_t up_row_stride) {
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  const bool vector_ok = aligned_to(gate, 16) && aligned_to(up, 16) && aligned_to(out, 16) &&
                         cols % 8 == 0 && gate_row_stride % 8 == 0 && up_row_stride % 8 == 0;
  if (vector_ok && gate_row_stride == cols && up_row_stride == cols) {
    const uint64_t vectors = rows * cols / 8;
    const unsigned grid = clamp_grid((vectors + kThreads * kUnroll - 1) / (kThreads * kUnroll), resident);
    return launch(swiglu_flat_kernel<kAct, kDtype, kRoundGate>, dim3(grid), dim3(kThreads), 0, s,
                  static_cast<const uint4 *>(gate), static_cast<const uint4 *>(up), static_cast<uint4 *>(out), vectors);
  }
  if (vector_ok && cols / 8 <= 0x7fffffffull) {
    const uint64_t row_vectors = cols / 8;
    const unsigned tiles = static_cast<unsigned>((row_vectors + kThreads - 1) / kThreads);
    uint64_t groups = (resident + tiles - 1) / tiles;
    const uint64_t useful = (rows + kUnroll - 1) / kUnroll;
    if (groups > useful) groups = useful;
    if (groups > 65535) groups = 65535;
    if (groups < 1) groups = 1;
    return launch(swiglu_rows_kernel<kAct, kDtype, kRoundGate>, dim3(dim3(tiles, static_cast<unsigned>(groups))), dim3(kThreads), 0, s,
                  static_cast<const uint4 *>(gate), static_cast<const uint4 *>(up), static_cast<uint4 *>(out), rows,
                  static_cast<uint32_t>(row_vectors), gate_row_stride / 8, up_row_stride / 8);
  }
  const unsigned grid = clamp_grid((rows * cols + kThreads - 1) / kThreads, resident);
  return launch(swiglu_scalar_kernel<kAct, kDtype, kRoundGate>, dim3(grid), dim3(kThreads), 0, s,
                static_cast<const unsigned short *>(gate), static_cast<const unsigned short *>(up),
                static_cast<unsigned short *>(out), rows, cols, gate_row_stride, up_row_stride);
}

template <int kAct, int kDtype>
int launch_gated_rounding(cudaStream_t s, int round_gate, const void *gate, const void *up, void *out, uint64_t rows,
                          uint64_t cols, uint64_t gate_row_stride, uint64_t up_row_stride) {
  return round_gate ? launch_gated<kAct, kDtype, true>(s, gate, up, out, rows, cols, gate_row_stride, up_row_stride)
                    : launch_gated<kAct, kDtype, false>(s, gate, up, out, rows, cols, gate_row_stride, up_row_stride);
}
template <int kDtype>
int launch_gated_kind(cudaStream_t s, int activation, int round_gate, const void *gate, const void *up, void *out,
                      uint64_t rows, uint64_t cols, uint64_t gate_row_stride, uint64_t up_row_stride) {
  switch (activation) {
    case HYLE_B200_GATE_SILU:
      return launch_gated_rounding<HYLE_B200_GATE_SILU, kDtype>(s, round_gate, gate, up, out, rows, cols, gate_row_stride, up_row_stride);
    case HYLE_B200_GATE_GELU:
      return launch_gated_rounding<HYLE_B200_GATE_GELU, kDtype>(s, round_gate, gate, up, out, rows, cols, gate_row_stride, up_row_stride);
    case HYLE_B200_GATE_GELU_TANH:
      return launch_gated_rounding<HYLE_B200_GATE_GELU_TANH, kDtype>(s, round_gate, gate, up, out, rows, cols, gate_row_stride, up_row_stride);
    default: return HYLE_B200_INVALID_VALUE;
  }
}
}  // namespace
}  // namespace hb

extern "C" int hyle_b200_gated_activation(hyle_b200_stream_t stream, int activation, int dtype, int round_gate,
                                          const void *gate, const void *up, void *out, uint64_t rows, uint64_t cols,
                                          uint64_t gate_row_stride, uint64_t up_row_stride) {
  if (activation < HYLE_B200_GATE_SILU || activation > HYLE_B200_GATE_GELU_TANH) return HYLE_B200_INVALID_VALUE;
  if (dtype != HYLE_B200_BF16 && dtype != HYLE_B200_F16) return HYLE_B200_NOT_SUPPORTED;
  if (rows == 0 || cols == 0) return HYLE_B200_OK;
  if (gate == nullptr || up == nullptr || out == nullptr || gate_row_stride < cols || up_row_stride < cols)
    return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == HYLE_B200_BF16)
    return hb::launch_gated_kind<HYLE_B200_BF16>(s, activation, round_gate, gate, up, out, rows, cols, gate_row_stride, up_row_stride);
  return hb::launch_gated_kind<HYLE_B200_F16>(s, activation, round_gate, gate, up, out, rows, cols, gate_row_stride, up_row_stride);
}

extern "C" int hyle_b200_swiglu_bf16(hyle_b200_stream_t stream, const void *gate, const void *up,
                                     void *out, uint64_t rows, uint64_t cols,
                                     uint64_t gate_row_stride, uint64_t up_row_stride) {
  return hyle_b200_gated_activation(stream, HYLE_B200_GATE_SILU, HYLE_B200_BF16, 0, gate, up, out, rows, cols,
                                    gate_row_stride, up_row_stride);
}

extern "C" int hyle_b200_unary(hyle_b200_stream_t stream, int kind, int dtype, const void *in, void *out,
                               uint64_t count) {
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr) return HYLE_B200_INVALID_VALUE;
  const size_t width = dtype == HYLE_B200_F32 ? 4 : 2;
  if (!aligned_to(in, width) || !aligned_to(out, width)) return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
#define HB_UNARY_CASE(K) \
  if (kind == K) { \
    if (dtype == HYLE_B200_F32) return launch_unary<K, HYLE_B200_F32>(s, in, out, count); \
    if (dtype == HYLE_B200_BF16) return launch_unary<K, HYLE_B200_BF16>(s, in, out, count); \
    if (dtype == HYLE_B200_F16) return launch_unary<K, HYLE_B200_F16>(s, in, out, count); \
    return HYLE_B200_INVALID_VALUE; \
  }
  HB_UNARY_CASE(HYLE_B200_UNARY_ABS)
  HB_UNARY_CASE(HYLE_B200_UNARY_NEG)
  HB_UNARY_CASE(HYLE_B200_UNARY_EXP)
  HB_UNARY_CASE(HYLE_B200_UNARY_LOG)
  HB_UNARY_CASE(HYLE_B200_UNARY_SQRT)
  HB_UNARY_CASE(HYLE_B200_UNARY_RSQRT)
  HB_UNARY_CASE(HYLE_B200_UNARY_TANH)
  HB_UNARY_CASE(HYLE_B200_UNARY_SIGMOID)
  HB_UNARY_CASE(HYLE_B200_UNARY_RELU)
  HB_UNARY_CASE(HYLE_B200_UNARY_GELU)
  HB_UNARY_CASE(HYLE_B200_UNARY_GELU_TANH)
  HB_UNARY_CASE(HYLE_B200_UNARY_SILU)
  HB_UNARY_CASE(HYLE_B200_UNARY_SOFTPLUS)
#undef HB_UNARY_CASE
  return HYLE_B200_INVALID_VALUE;
}

extern "C" int hyle_b200_cast_f32_to_bf16(hyle_b200_stream_t stream, const float *in,
                                          void *out_bf16, uint64_t count) {
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || out_bf16 == nullptr) return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * kCtasPerSm;
  if (aligned_to(in, 16) && aligned_to(out_bf16, 16) && count % 8 == 0) {
    const uint64_t vectors = count / 8;
    const unsigned grid = clamp_grid((vectors + kThreads * kUnroll - 1) / (kThreads * kUnroll), resident);
    return launch(cast_f32_bf16_kernel, dim3(grid), dim3(kThreads), 0, s, reinterpret_cast<const float4 *>(in),
                                                   static_cast<uint4 *>(out_bf16), vectors);
  }
  const unsigned grid = clamp_grid((count + kThreads - 1) / kThreads, resident);
  return launch(cast_f32_bf16_scalar_kernel, dim3(grid), dim3(kThreads), 0, s, in, static_cast<unsigned short *>(out_bf16), count);
}

// Row-wise operators: Reduce{kSum|kMean|kMinimum|kMaximum} over the last axis of f32 rows, its
// fusion with a bias add (one read of A, one write of C, reductions from registers), and bf16
// RmsNorm with the optional fused residual add.  Each row is read from HBM exactly once.
#include "common.cuh"

#include <math_constants.h>
#include <type_traits>

namespace hb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / kWarpSize;

// ================================================================================================
// f32 rows: optional op with a row vector, optional store, row sum / max / min.
// One CTA owns one row at a time.  Column slot (k, t) = four columns starting at (k*256 + t)*4; a
// thread adds its columns in (k, lane-of-vector) order, warps combine by xor butterfly, the eight
// warp partials are added in warp order.  The order does not depend on the grid, on alignment or on
// which outputs are requested, so a fused launch and separate launches agree bit for bit.
// ================================================================================================
constexpr int kOpNone = -1;

struct RowF32Params {
  const float *a;
  const float *rhs;  // one row, or nullptr
  float *c;          // elementwise output or nullptr
  float *row_sum;    // nullptr to skip
  float *row_max;
  float *row_min;
  uint64_t rows;
  uint64_t cols;
  int mean;          // row_sum receives sum / cols
};

template <int kOp>
__device__ __forceinline__ float row_op(float a, float b) {
  if constexpr (kOp == HYLE_B200_BINARY_ADD) return __fadd_rn(a, b);
  if constexpr (kOp == HYLE_B200_BINARY_MULTIPLY) return __fmul_rn(a, b);
  return a;
}

struct RowAcc {
  float sum, mx, mn;
  __device__ __forceinline__ RowAcc() : sum(0.0f), mx(-INFINITY), mn(INFINITY) {}
  __device__ __forceinline__ void add(float v) {
    sum = __fadd_rn(sum, v);
    mx = max_nan(mx, v);
    mn = min_nan(mn, v);
  }
};

// kSlots > 0: cols == kSlots*1024 exactly, 16-byte aligned pointers, bias kept in registers.
// kSlots == 0: any cols; kVec selects 16-byte accesses for full slots (needs cols % 4 == 0 and
// aligned pointers), scalar accesses otherwise.
template <int kSlots, bool kVec, int kOp>
__global__ void __launch_bounds__(kThreads) row_f32_kernel(const RowF32Params p) {
  grid_dependency_sync();
  __shared__ float s_sum[2][kWarps], s_max[2][kWarps], s_min[2][kWarps];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint64_t cols = p.cols;

  float4 bias[kSlots > 0 ? kSlots : 1];
  if constexpr (kSlots > 0 && kOp != kOpNone) {
#pragma unroll
    for (int k = 0; k < kSlots; ++k) bias[k] = __ldg(reinterpret_cast<const float4 *>(p.rhs) + k * kThreads + t);
  }

  int parity = 0;
  for (uint64_t row = blockIdx.x; row < p.rows; row += gridDim.x, parity ^= 1) {
    const float *a_row = p.a + row * cols;
    float *c_row = p.c != nullptr ? p.c + row * cols : nullptr;
    RowAcc acc;
    if constexpr (kSlots > 0) {
      float4 x[kSlots];
#pragma unroll
      for (int k = 0; k < kSlots; ++k) x[k] = ld_stream(reinterpret_cast<const float4 *>(a_row) + k * kThreads + t);
#pragma unroll
      for (int k = 0; k < kSlots; ++k) {
        x[k] = make_float4(row_op<kOp>(x[k].x, bias[k].x), row_op<kOp>(x[k].y, bias[k].y),
                           row_op<kOp>(x[k].z, bias[k].z), row_op<kOp>(x[k].w, bias[k].w));
        if (c_row != nullptr) st_stream(reinterpret_cast<float4 *>(c_row) + k * kThreads + t, x[k]);
        acc.add(x[k].x); acc.add(x[k].y); acc.add(x[k].z); acc.add(x[k].w);
      }
    } else {
      for (uint64_t base = static_cast<uint64_t>(t) * 4; base < cols; base += kThreads * 4) {
        if (kVec && base + 4 <= cols) {
          float4 x = ld_stream(reinterpret_cast<const float4 *>(a_row + base));
          if constexpr (kOp != kOpNone) {
            const float4 b = __ldg(reinterpret_cast<const float4 *>(p.rhs + base));
            x = make_float4(row_op<kOp>(x.x, b.x), row_op<kOp>(x.y, b.y), row_op<kOp>(x.z, b.z),
                            row_op<kOp>(x.w, b.w));
          }
          if (c_row != nullptr) st_stream(reinterpret_cast<float4 *>(c_row + base), x);
          acc.add(x.x); acc.add(x.y); acc.add(x.z); acc.add(x.w);
        } else {
          for (uint64_t col = base; col < base + 4 && col < cols; ++col) {
            float x = ld_stream(a_row + col);
            if constexpr (kOp != kOpNone) x = row_op<kOp>(x, __ldg(p.rhs + col));
            if (c_row != nullptr) st_stream(c_row + col, x);
            acc.add(x);
          }
        }
      }
    }
    const float sum = warp_sum(acc.sum);
    const float mx = warp_max_nan(acc.mx);
    const float mn = warp_min_nan(acc.mn);
    if (lane == 0) {
      s_sum[parity][warp] = sum;
      s_max[parity][warp] = mx;
      s_min[parity][warp] = mn;
    }
    // One barrier per row: the partials are double buffered, and the barrier of the next row
    // orders this row's read by thread 0 before the row after next overwrites the slot.
    __syncthreads();
    if (t == 0) {
      float total = s_sum[parity][0], hi = s_max[parity][0], lo = s_min[parity][0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) {
        total = __fadd_rn(total, s_sum[parity][w]);
        hi = max_nan(hi, s_max[parity][w]);
        lo = min_nan(lo, s_min[parity][w]);
      }
      if (p.row_sum != nullptr)
        p.row_sum[row] = p.mean ? __fdiv_rn(total, static_cast<float>(cols)) : total;
      if (p.row_max != nullptr) p.row_max[row] = hi;
      if (p.row_min != nullptr) p.row_min[row] = lo;
    }
  }
}

template <int kOp>
int launch_row_f32(cudaStream_t stream, const RowF32Params &p) {
  if (p.rows == 0) return HYLE_B200_OK;
  const bool aligned = aligned_to(p.a, 16) && (p.rhs == nullptr || aligned_to(p.rhs, 16)) &&
                       (p.c == nullptr || aligned_to(p.c, 16)) && p.cols % 4 == 0;
  // 48-64 registers per thread: five to eight CTAs share an SM.
  const unsigned grid = clamp_grid(p.rows, static_cast<uint64_t>(sm_count()) * 8);
  int launch_status = HYLE_B200_OK;
  if (aligned && p.cols == 1024) launch_status = launch(row_f32_kernel<1, true, kOp>, dim3(grid), dim3(kThreads), 0, stream, p);
  else if (aligned && p.cols == 2048) launch_status = launch(row_f32_kernel<2, true, kOp>, dim3(grid), dim3(kThreads), 0, stream, p);
  else if (aligned && p.cols == 4096) launch_status = launch(row_f32_kernel<4, true, kOp>, dim3(grid), dim3(kThreads), 0, stream, p);
  else if (aligned && p.cols == 8192) launch_status = launch(row_f32_kernel<8, true, kOp>, dim3(grid), dim3(kThreads), 0, stream, p);
  else if (aligned) launch_status = launch(row_f32_kernel<0, true, kOp>, dim3(grid), dim3(kThreads), 0, stream, p);
  else launch_status = launch(row_f32_kernel<0, false, kOp>, dim3(grid), dim3(kThreads), 0, stream, p);
  return launch_status;
}

// ================================================================================================
// bf16 RmsNorm, optional fused residual add.
//   h = kResidual ? bf16_rne(f32 x + f32 r) : x;  ss = sum f32(h)^2 (fma, f32);
//   inverse = 1.0f / sqrtf(ss / hidden + eps);     y = bf16_rne((f32(h) * inverse) * w)
// (src/simd/math/activations.cc:124-146).  kWeight: 0 none, 1 bf16, 2 f32.
// ================================================================================================
__device__ __forceinline__ float inverse_rms(float sum_squares, uint32_t hidden, float eps) {
  const float mean = __fdiv_rn(sum_squares, static_cast<float>(hidden));
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

__device__ __forceinline__ uint32_t add_pair(uint32_t a, uint32_t b) {
  return pack_bf16x2(__fadd_rn(bf16_lo(a), bf16_lo(b)), __fadd_rn(bf16_hi(a), bf16_hi(b)));
}
__device__ __forceinline__ uint4 add_vec(uint4 a, uint4 b) {
  return make_uint4(add_pair(a.x, b.x), add_pair(a.y, b.y), add_pair(a.z, b.z), add_pair(a.w, b.w));
}
__device__ __forceinline__ float squares(uint32_t w, float acc) {
  const float lo = bf16_lo(w), hi = bf16_hi(w);
  return fmaf(hi, hi, fmaf(lo, lo, acc));
}
__device__ __forceinline__ float squares(uint4 v, float acc) {
  return squares(v.w, squares(v.z, squares(v.y, squares(v.x, acc))));
}

// Scale eight packed bf16 values by inverse and the weight vector at element offset `element`.
template <int kWeight>
__device__ __forceinline__ uint4 scale_vec(uint4 h, float inverse, const void *weight, uint64_t element) {
  float v[8] = {bf16_lo(h.x), bf16_hi(h.x), bf16_lo(h.y), bf16_hi(h.y),
                bf16_lo(h.z), bf16_hi(h.z), bf16_lo(h.w), bf16_hi(h.w)};
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], inverse);
  if constexpr (kWeight == 1) {
    const uint4 w = __ldg(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(weight) + element));
    const float f[8] = {bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y),
                        bf16_lo(w.z), bf16_hi(w.z), bf16_lo(w.w), bf16_hi(w.w)};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], f[i]);
  } else if constexpr (kWeight == 2) {
    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(weight) + element));
    const float4 w1 = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(weight) + element) + 1);
    const float f[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], f[i]);
  }
  return make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                    pack_bf16x2(v[6], v[7]));
}

// One warp per row, the whole row in registers: hidden == kVectors*256.  No barrier, no shared
// memory; every lane has 2*kVectors independent 16-byte loads in flight.
template <int kVectors, bool kResidual, int kWeight>
__global__ void __launch_bounds__(kThreads)
rms_warp_kernel(const uint4 *x, const uint4 *residual, const void *__restrict__ weight, uint4 *y,
                uint4 *h_out, uint64_t rows, float eps) {
  grid_dependency_sync();
  constexpr uint32_t kHidden = kVectors * 256;
  const int lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x >> 5);
  for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
       row < rows; row += warps) {
    const uint64_t base = row * (kHidden / 8);
    uint4 h[kVectors];
    if constexpr (kResidual) {
      uint4 r[kVectors];
#pragma unroll
      for (int k = 0; k < kVectors; ++k) {
        h[k] = ld_stream(x + base + k * 32 + lane);
        r[k] = ld_stream(residual + base + k * 32 + lane);
      }
#pragma unroll
      for (int k = 0; k < kVectors; ++k) {
        h[k] = add_vec(h[k], r[k]);
        st_stream(h_out + base + k * 32 + lane, h[k]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < kVectors; ++k) h[k] = ld_stream(x + base + k * 32 + lane);
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kVectors; ++k) ss = squares(h[k], ss);
    ss = warp_sum(ss);
    const float inverse = inverse_rms(ss, kHidden, eps);
#pragma unroll
    for (int k = 0; k < kVectors; ++k)
      st_stream(y + base + k * 32 + lane,
                scale_vec<kWeight>(h[k], inverse, weight, static_cast<uint64_t>(k * 32 + lane) * 8));
  }
}

// One CTA per row, the row staged in shared memory as bf16: any hidden up to kMaxStagedHidden.
constexpr uint32_t kMaxStagedHidden = 32768;

template <bool kVec, bool kResidual, int kWeight>
__global__ void __launch_bounds__(kThreads)
rms_cta_kernel(const unsigned short *x, const unsigned short *residual,
               const void *__restrict__ weight, unsigned short *y, unsigned short *h_out,
               uint64_t rows, uint32_t hidden, float eps) {
  grid_dependency_sync();
  extern __shared__ __align__(16) unsigned char staged_bytes[];
  __shared__ float s_partial[2][kWarps];
  unsigned short *staged = reinterpret_cast<unsigned short *>(staged_bytes);
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  int parity = 0;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const uint64_t base = row * hidden;
    float ss = 0.0f;
    if constexpr (kVec) {
      for (uint32_t v = t; v < hidden / 8; v += kThreads) {
        uint4 h = ld_stream(reinterpret_cast<const uint4 *>(x + base) + v);
        if constexpr (kResidual) {
          h = add_vec(h, ld_stream(reinterpret_cast<const uint4 *>(residual + base) + v));
          st_stream(reinterpret_cast<uint4 *>(h_out + base) + v, h);
        }
        reinterpret_cast<uint4 *>(staged)[v] = h;
        ss = squares(h, ss);
      }
    } else {
      for (uint32_t i = t; i < hidden; i += kThreads) {
        unsigned short h = x[base + i];
        if constexpr (kResidual) {
          h = f32_to_bf16(__fadd_rn(bf16_to_f32(h), bf16_to_f32(residual[base + i])));
          h_out[base + i] = h;
        }
        staged[i] = h;
        const float f = bf16_to_f32(h);
        ss = fmaf(f, f, ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) s_partial[parity][warp] = ss;
    __syncthreads();  // also publishes the staged row
    float total = s_partial[parity][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total = __fadd_rn(total, s_partial[parity][w]);
    const float inverse = inverse_rms(total, hidden, eps);
    if constexpr (kVec) {
      for (uint32_t v = t; v < hidden / 8; v += kThreads)
        st_stream(reinterpret_cast<uint4 *>(y + base) + v,
                  scale_vec<kWeight>(reinterpret_cast<const uint4 *>(staged)[v], inverse, weight,
                                     static_cast<uint64_t>(v) * 8));
    } else {
      for (uint32_t i = t; i < hidden; i += kThreads) {
        float v = __fmul_rn(bf16_to_f32(staged[i]), inverse);
        if constexpr (kWeight == 1) v = __fmul_rn(v, bf16_to_f32(static_cast<const unsigned short *>(weight)[i]));
        if constexpr (kWeight == 2) v = __fmul_rn(v, static_cast<const float *>(weight)[i]);
        y[base + i] = f32_to_bf16(v);
      }
    }
    __syncthreads();  // the staged row is rewritten by the next iteration
  }
}

template <bool kResidual, int kWeight>
int launch_rms(cudaStream_t stream, const void *x, const void *residual, const void *weight, void *y,
               void *h, uint64_t rows, uint64_t hidden, float eps) {
  const bool aligned = aligned_to(x, 16) && aligned_to(y, 16) && (weight == nullptr || aligned_to(weight, 16)) &&
                       (!kResidual || (aligned_to(residual, 16) && aligned_to(h, 16))) && hidden % 8 == 0;
  const int sms = sm_count();
  auto warp_launch = [&](auto vectors_tag) {
    constexpr int kVectors = decltype(vectors_tag)::value;
    // Two rows per CTA: many small CTAs keep the tail of the grid short (the hardware hands a freed
    // slot to the next CTA), and small row counts still spread over all SMs.
    int warps_per_cta = 2;
    if (rows < static_cast<uint64_t>(sms) * 2) warps_per_cta = 1;
    const uint64_t ctas = (rows + warps_per_cta - 1) / warps_per_cta;
    const unsigned grid = clamp_grid(ctas, 1u << 20);
    return launch(rms_warp_kernel<kVectors, kResidual, kWeight>, dim3(grid), dim3(warps_per_cta * 32), 0, stream, 
        static_cast<const uint4 *>(x), static_cast<const uint4 *>(residual), weight,
        static_cast<uint4 *>(y), static_cast<uint4 *>(h), rows, eps);
  };
  if (aligned && hidden == 256) return warp_launch(std::integral_constant<int, 1>{});
  if (aligned && hidden == 512) return warp_launch(std::integral_constant<int, 2>{});
  if (aligned && hidden == 1024) return warp_launch(std::integral_constant<int, 4>{});
  if (aligned && hidden == 2048) return warp_launch(std::integral_constant<int, 8>{});
  if (hidden > kMaxStagedHidden) return HYLE_B200_NOT_SUPPORTED;
  const size_t staged = (static_cast<size_t>(hidden) * 2 + 15) & ~static_cast<size_t>(15);
  const unsigned grid = clamp_grid(rows, static_cast<uint64_t>(sms) * 4);
  int launch_status = HYLE_B200_OK;
  if (aligned) {
    auto kernel = rms_cta_kernel<true, kResidual, kWeight>;
    if (staged > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    launch_status = launch(kernel, dim3(grid), dim3(kThreads), staged, stream, 
        static_cast<const unsigned short *>(x), static_cast<const unsigned short *>(residual), weight,
        static_cast<unsigned short *>(y), static_cast<unsigned short *>(h), rows,
        static_cast<uint32_t>(hidden), eps);
  } else {
    auto kernel = rms_cta_kernel<false, kResidual, kWeight>;
    if (staged > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    launch_status = launch(kernel, dim3(grid), dim3(kThreads), staged, stream, 
        static_cast<const unsigned short *>(x), static_cast<const unsigned short *>(residual), weight,
        static_cast<unsigned short *>(y), static_cast<unsigned short *>(h), rows,
        static_cast<uint32_t>(hidden), eps);
  }
  return launch_status;
}

// ------------------------------------------------------------------------------------------------
// RmsNorm on f16 and f32 rows (the other two storages of the CPU route,
// src/compute_provider_native/normalization.cc:41-80,219-234): the same formula with the storage's own
// load and a single rounding at the store; the weight has the row's type or is f32.
// Rows of at most 8 KB: one warp per row, second read from L1.  Longer rows: one CTA per row, the row
// staged in shared memory in its own storage.
// ------------------------------------------------------------------------------------------------
template <int kDtype>
struct Stored {
  static constexpr int kBytes = kDtype == HYLE_B200_F32 ? 4 : 2;
  static __device__ __forceinline__ float load1(const void *base, uint64_t i) {
    if constexpr (kDtype == HYLE_B200_F32) return static_cast<const float *>(base)[i];
    else if constexpr (kDtype == HYLE_B200_BF16) return bf16_to_f32(static_cast<const unsigned short *>(base)[i]);
    else return f16_to_f32(static_cast<const unsigned short *>(base)[i]);
  }
  static __device__ __forceinline__ void store1(void *base, uint64_t i, float v) {
    if constexpr (kDtype == HYLE_B200_F32) static_cast<float *>(base)[i] = v;
    else if constexpr (kDtype == HYLE_B200_BF16) static_cast<unsigned short *>(base)[i] = f32_to_bf16(v);
    else static_cast<unsigned short *>(base)[i] = f32_to_f16(v);
  }
  // eight consecutive elements starting at element 8 * vec (16-byte aligned storage)
  static __device__ __forceinline__ void load8(const void *base, uint64_t vec, float (&v)[8]) {
    if constexpr (kDtype == HYLE_B200_F32) {
      const float4 a = static_cast<const float4 *>(base)[2 * vec], b = static_cast<const float4 *>(base)[2 * vec + 1];
      v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
      const uint4 w = static_cast<const uint4 *>(base)[vec];
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const unsigned short narrow = static_cast<unsigned short>(e & 1 ? words[e / 2] >> 16 : words[e / 2] & 0xffffu);
        v[e] = kDtype == HYLE_B200_BF16 ? bf16_to_f32(narrow) : f16_to_f32(narrow);
      }
    }
  }
  static __device__ __forceinline__ void store8(void *base, uint64_t vec, const float (&v)[8]) {
    if constexpr (kDtype == HYLE_B200_F32) {
      static_cast<float4 *>(base)[2 * vec] = make_float4(v[0], v[1], v[2], v[3]);
      static_cast<float4 *>(base)[2 * vec + 1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint32_t words[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        words[e] = kDtype == HYLE_B200_BF16
                       ? pack_bf16x2(v[2 * e], v[2 * e + 1])
                       : pack_f16x2(v[2 * e], v[2 * e + 1]);
      static_cast<uint4 *>(base)[vec] = make_uint4(words[0], words[1], words[2], words[3]);
    }
  }
};

// y[8] = (x[8] * inverse) * w[8]; kWeight: -1 none, else the weight's dtype
template <int kWeight>
__device__ __forceinline__ void scale8(float (&v)[8], float inverse, const void *weight, uint64_t vec) {
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], inverse);
  if constexpr (kWeight >= 0) {
    float w[8];
    Stored<kWeight>::load8(weight, vec, w);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], w[e]);
  }
}

// kKeep > 0: rows of at most kKeep * 256 values (vector path) stay in registers between the two passes,
// kKeep groups of eight values per lane, all loads in flight at once; the row is read once.
template <int kDtype, int kWeight, bool kVec, int kKeep = 0>
__global__ void __launch_bounds__(kThreads)
rms_stored_warp_kernel(const void *x, const void *weight, void *y, uint64_t rows, uint32_t hidden, float eps) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x >> 5);
  for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    const char *in = static_cast<const char *>(x) + row * hidden * Stored<kDtype>::kBytes;
    char *out = static_cast<char *>(y) + row * hidden * Stored<kDtype>::kBytes;
    float ss = 0.0f;
    if constexpr (kVec && kKeep > 0) {
      float f[kKeep][8];
      const uint32_t vectors = hidden / 8;
#pragma unroll
      for (int k = 0; k < kKeep; ++k) {
        const uint32_t v = k * 32 + lane;
        if (v < vectors) {
          Stored<kDtype>::load8(in, v, f[k]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[k][e] = 0.0f;
        }
      }
#pragma unroll
      for (int k = 0; k < kKeep; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[k][e], f[k][e], ss);
      const float inverse = inverse_rms(warp_sum(ss), hidden, eps);
#pragma unroll
      for (int k = 0; k < kKeep; ++k) {
        const uint32_t v = k * 32 + lane;
        if (v < vectors) {
          scale8<kWeight>(f[k], inverse, weight, v);
          Stored<kDtype>::store8(out, v, f[k]);
        }
      }
      continue;
    }
    if constexpr (kVec) {
      for (uint32_t v = lane; v < hidden / 8; v += 32) {
        float f[8];
        Stored<kDtype>::load8(in, v, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
      }
    } else {
      for (uint32_t i = lane; i < hidden; i += 32) {
        const float f = Stored<kDtype>::load1(in, i);
        ss = fmaf(f, f, ss);
      }
    }
    // every lane has read its part of the row before the sum is known: y may be x
    const float inverse = inverse_rms(warp_sum(ss), hidden, eps);
    if constexpr (kVec) {
      for (uint32_t v = lane; v < hidden / 8; v += 32) {
        float f[8];
        Stored<kDtype>::load8(in, v, f);
        scale8<kWeight>(f, inverse, weight, v);
        Stored<kDtype>::store8(out, v, f);
      }
    } else {
      for (uint32_t i = lane; i < hidden; i += 32) {
        float f = __fmul_rn(Stored<kDtype>::load1(in, i), inverse);
        if constexpr (kWeight >= 0) f = __fmul_rn(f, Stored<kWeight < 0 ? kDtype : kWeight>::load1(weight, i));
        Stored<kDtype>::store1(out, i, f);
      }
    }
  }
}

constexpr uint32_t kMaxStoredRowBytes = 64 * 1024;

template <int kDtype, int kWeight, bool kVec>
__global__ void __launch_bounds__(kThreads)
rms_stored_cta_kernel(const void *x, const void *weight, void *y, uint64_t rows, uint32_t hidden, float eps) {
  grid_dependency_sync();
  extern __shared__ __align__(16) unsigned char staged_bytes[];
  __shared__ float s_partial[2][kWarps];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  int parity = 0;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const char *in = static_cast<const char *>(x) + row * hidden * Stored<kDtype>::kBytes;
    char *out = static_cast<char *>(y) + row * hidden * Stored<kDtype>::kBytes;
    float ss = 0.0f;
    if constexpr (kVec) {
      for (uint32_t v = t; v < hidden / 8; v += kThreads) {
        float f[8];
        Stored<kDtype>::load8(in, v, f);
        Stored<kDtype>::store8(staged_bytes, v, f);  // decode and encode are exact inverses: the stored bits
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
      }
    } else {
      for (uint32_t i = t; i < hidden; i += kThreads) {
        const float f = Stored<kDtype>::load1(in, i);
        Stored<kDtype>::store1(staged_bytes, i, f);
        ss = fmaf(f, f, ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) s_partial[parity][warp] = ss;
    __syncthreads();  // also publishes the staged row
    float total = s_partial[parity][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total = __fadd_rn(total, s_partial[parity][w]);
    const float inverse = inverse_rms(total, hidden, eps);
    if constexpr (kVec) {
      for (uint32_t v = t; v < hidden / 8; v += kThreads) {
        float f[8];
        Stored<kDtype>::load8(staged_bytes, v, f);
        scale8<kWeight>(f, inverse, weight, v);
        Stored<kDtype>::store8(out, v, f);
      }
    } else {
      for (uint32_t i = t; i < hidden; i += kThreads) {
        float f = __fmul_rn(Stored<kDtype>::load1(staged_bytes, i), inverse);
        if constexpr (kWeight >= 0) f = __fmul_rn(f, Stored<kWeight < 0 ? kDtype : kWeight>::load1(weight, i));
        Stored<kDtype>::store1(out, i, f);
      }
    }
    __syncthreads();  // the staged row is rewritten by the next iteration
  }
}

template <int kDtype, int kWeight, bool kVec>
int launch_rms_stored(cudaStream_t stream, const void *x, const void *weight, void *y, uint64_t rows, uint64_t hidden, float eps) {
  const uint64_t row_bytes = hidden * Stored<kDtype>::kBytes;
  const int sms = sm_count();
  if (row_bytes <= 8 * 1024) {
    const unsigned grid = clamp_grid((rows + kWarps - 1) / kWarps, static_cast<uint64_t>(sms) * 8);
    auto go = [&](auto keep_tag) {
      return launch(rms_stored_warp_kernel<kDtype, kWeight, kVec, decltype(keep_tag)::value>, dim3(grid), dim3(kThreads), 0, stream,
                    x, weight, y, rows, static_cast<uint32_t>(hidden), eps);
    };
    if constexpr (kVec) {
      if (hidden <= 512) return go(std::integral_constant<int, 2>{});
      if (hidden <= 1024) return go(std::integral_constant<int, 4>{});
      if (hidden <= 2048) return go(std::integral_constant<int, 8>{});
    }
    return go(std::integral_constant<int, 0>{});
  }
  if (row_bytes > kMaxStoredRowBytes) return HYLE_B200_NOT_SUPPORTED;
  const size_t staged = (static_cast<size_t>(row_bytes) + 15) & ~static_cast<size_t>(15);
  auto kernel = rms_stored_cta_kernel<kDtype, kWeight, kVec>;
  if (staged > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMaxStoredRowBytes));
  return launch(kernel, dim3(clamp_grid(rows, static_cast<uint64_t>(sms) * 4)), dim3(kThreads), staged, stream, x, weight, y, rows,
                static_cast<uint32_t>(hidden), eps);
}

template <int kDtype>
int dispatch_rms_stored(cudaStream_t stream, const void *x, const void *weight, int weight_dtype, void *y, uint64_t rows,
                        uint64_t hidden, float eps) {
  if (rows == 0 || hidden == 0) return HYLE_B200_OK;
  const int element = Stored<kDtype>::kBytes;
  if (x == nullptr || y == nullptr || !aligned_to(x, element) || !aligned_to(y, element) ||
      (weight != nullptr && weight_dtype != kDtype && weight_dtype != HYLE_B200_F32))
    return HYLE_B200_INVALID_VALUE;
  const bool vec = hidden % 8 == 0 && aligned_to(x, 16) && aligned_to(y, 16) && (weight == nullptr || aligned_to(weight, 16));
  if (weight != nullptr && !aligned_to(weight, weight_dtype == HYLE_B200_F32 ? 4 : 2)) return HYLE_B200_INVALID_VALUE;
  auto go = [&](auto weight_tag) {
    constexpr int kWeight = decltype(weight_tag)::value;
    return vec ? launch_rms_stored<kDtype, kWeight, true>(stream, x, weight, y, rows, hidden, eps)
               : launch_rms_stored<kDtype, kWeight, false>(stream, x, weight, y, rows, hidden, eps);
  };
  if (weight == nullptr) return go(std::integral_constant<int, -1>{});
  if (weight_dtype == HYLE_B200_F32) return go(std::integral_constant<int, HYLE_B200_F32>{});
  return go(std::integral_constant<int, kDtype>{});
}

// ------------------------------------------------------------------------------------------------
// Reduce{kMinimum | kMaximum} over the last axis of bf16 / f16 rows, the result in the rows' own type
// (the narrow Min/Max the CPU route keeps, src/compute_provider_native/reduction.cc:203-223).  The
// comparison runs on the exactly converted f32 values under the f32 kernel's rules (NaN wins, -0 < +0,
// an empty row gives the identity), and an extremum converts back without rounding.
// kCta: one CTA per row (long rows); else one warp per row.
// ------------------------------------------------------------------------------------------------
template <int kDtype, bool kMaximum, bool kVec, bool kCta>
__global__ void __launch_bounds__(kThreads)
narrow_extremum_kernel(const void *in, void *out, uint64_t rows, uint64_t cols) {
  grid_dependency_sync();
  __shared__ float s_partial[2][kWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t width = kCta ? kThreads : 32, position = kCta ? threadIdx.x : lane;
  const uint64_t stride = kCta ? gridDim.x : static_cast<uint64_t>(gridDim.x) * kWarps;
  auto combine = [](float a, float b) { return kMaximum ? max_nan(a, b) : min_nan(a, b); };
  int parity = 0;
  for (uint64_t row = kCta ? blockIdx.x : static_cast<uint64_t>(blockIdx.x) * kWarps + warp; row < rows; row += stride, parity ^= 1) {
    const char *base = static_cast<const char *>(in) + row * cols * Stored<kDtype>::kBytes;
    float best = kMaximum ? -CUDART_INF_F : CUDART_INF_F;
    if constexpr (kVec) {
      const uint64_t vectors = cols / 8;
      uint64_t v = position;
      for (; v + width < vectors; v += 2 * width) {  // two 16-byte loads in flight per thread
        float a[8], b[8];
        Stored<kDtype>::load8(base, v, a);
        Stored<kDtype>::load8(base, v + width, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) best = combine(best, combine(a[e], b[e]));
      }
      if (v < vectors) {
        float a[8];
        Stored<kDtype>::load8(base, v, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) best = combine(best, a[e]);
      }
    } else {
      for (uint64_t i = position; i < cols; i += width) best = combine(best, Stored<kDtype>::load1(base, i));
    }
    best = kMaximum ? warp_max_nan(best) : warp_min_nan(best);
    if constexpr (kCta) {
      if (lane == 0) s_partial[parity][warp] = best;
      __syncthreads();  // double-buffered partials: one barrier per row
      if (threadIdx.x == 0) {
        float total = s_partial[parity][0];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) total = combine(total, s_partial[parity][w]);
        Stored<kDtype>::store1(out, row, total);
      }
    } else {
      if (lane == 0) Stored<kDtype>::store1(out, row, best);
    }
  }
}

template <int kDtype, bool kMaximum>
int launch_narrow_extremum(cudaStream_t stream, const void *in, void *out, uint64_t rows, uint64_t cols) {
  const bool vec = cols % 8 == 0 && aligned_to(in, 16);
  const int sms = sm_count();
  // a warp covers a row of up to 16 KB well; beyond that, or when there are too few rows to give every SM
  // eight warps, a CTA per row
  const bool cta = cols > 8192 || rows < static_cast<uint64_t>(sms) * kWarps;
  const unsigned grid = clamp_grid(cta ? rows : (rows + kWarps - 1) / kWarps, static_cast<uint64_t>(sms) * 8);
  auto go = [&](auto vec_tag, auto cta_tag) {
    return launch(narrow_extremum_kernel<kDtype, kMaximum, decltype(vec_tag)::value, decltype(cta_tag)::value>, dim3(grid),
                  dim3(kThreads), 0, stream, in, out, rows, cols);
  };
  if (vec) return cta ? go(std::true_type{}, std::true_type{}) : go(std::true_type{}, std::false_type{});
  return cta ? go(std::false_type{}, std::true_type{}) : go(std::false_type{}, std::false_type{});
}

template <bool kResidual>
int dispatch_rms(cudaStream_t stream, const void *x, const void *residual, const void *weight,
                 int weight_dtype, void *y, void *h, uint64_t rows, uint64_t hidden, float eps) {
  if (rows == 0 || hidden == 0) return HYLE_B200_OK;
  if (x == nullptr || y == nullptr || (kResidual && (residual == nullptr || h == nullptr)))
    return HYLE_B200_INVALID_VALUE;
  if (weight == nullptr) return launch_rms<kResidual, 0>(stream, x, residual, nullptr, y, h, rows, hidden, eps);
  if (weight_dtype == HYLE_B200_BF16) return launch_rms<kResidual, 1>(stream, x, residual, weight, y, h, rows, hidden, eps);
  if (weight_dtype == HYLE_B200_F32) return launch_rms<kResidual, 2>(stream, x, residual, weight, y, h, rows, hidden, eps);
  return HYLE_B200_INVALID_VALUE;
}

// ================================================================================================
// bf16 LayerNorm with optional bf16 scale and bias (both or neither).
//   mean = (sum f32(x)) / hidden;  ss = sum (f32(x) - mean)^2 (fma, f32);
//   inverse = 1.0f / sqrtf(ss / hidden + eps);
//   y = bf16_rne(fma((f32(x) - mean) * inverse, scale, bias))         without scale: no fma
// (src/simd/math/activations.cc:148-174).  Both sums run over values the warp / CTA already holds,
// so HBM sees the row once in and once out.
// ================================================================================================
__device__ __forceinline__ float sum_vec(uint4 v, float acc) {
  acc = __fadd_rn(acc, __fadd_rn(bf16_lo(v.x), bf16_hi(v.x)));
  acc = __fadd_rn(acc, __fadd_rn(bf16_lo(v.y), bf16_hi(v.y)));
  acc = __fadd_rn(acc, __fadd_rn(bf16_lo(v.z), bf16_hi(v.z)));
  return __fadd_rn(acc, __fadd_rn(bf16_lo(v.w), bf16_hi(v.w)));
}
__device__ __forceinline__ float centered_squares(uint4 v, float mean, float acc) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = __fsub_rn(bf16_lo(w[i]), mean), hi = __fsub_rn(bf16_hi(w[i]), mean);
    acc = fmaf(hi, hi, fmaf(lo, lo, acc));
  }
  return acc;
}
__device__ __forceinline__ float layer_value(float x, float mean, float inverse, bool affine, float scale, float bias) {
  const float normalized = __fmul_rn(__fsub_rn(x, mean), inverse);
  return affine ? fmaf(normalized, scale, bias) : normalized;
}
template <bool kAffine>
__device__ __forceinline__ uint4 layer_vec(uint4 h, float mean, float inverse, const unsigned short *scale,
                                           const unsigned short *bias, uint64_t element) {
  uint4 s = make_uint4(0, 0, 0, 0), b = s;
  if constexpr (kAffine) {
    s = __ldg(reinterpret_cast<const uint4 *>(scale + element));
    b = __ldg(reinterpret_cast<const uint4 *>(bias + element));
  }
  const uint32_t hw[4] = {h.x, h.y, h.z, h.w}, sw[4] = {s.x, s.y, s.z, s.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    out[i] = pack_bf16x2(layer_value(bf16_lo(hw[i]), mean, inverse, kAffine, bf16_lo(sw[i]), bf16_lo(bw[i])),
                         layer_value(bf16_hi(hw[i]), mean, inverse, kAffine, bf16_hi(sw[i]), bf16_hi(bw[i])));
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// One warp per row, the row in registers: hidden == kVectors * 256.
template <int kVectors, bool kAffine>
__global__ void __launch_bounds__(kThreads)
layer_norm_warp_kernel(const uint4 *x, const unsigned short *__restrict__ scale, const unsigned short *__restrict__ bias,
                       uint4 *y, uint64_t rows, float eps) {
  grid_dependency_sync();
  constexpr uint32_t kHidden = kVectors * 256;
  const int lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x >> 5);
  for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps) {
    const uint64_t base = row * (kHidden / 8);
    uint4 h[kVectors];
#pragma unroll
    for (int k = 0; k < kVectors; ++k) h[k] = ld_stream(x + base + k * 32 + lane);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < kVectors; ++k) sum = sum_vec(h[k], sum);
    const float mean = __fdiv_rn(warp_sum(sum), static_cast<float>(kHidden));
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kVectors; ++k) ss = centered_squares(h[k], mean, ss);
    const float inverse = inverse_rms(warp_sum(ss), kHidden, eps);
#pragma unroll
    for (int k = 0; k < kVectors; ++k)
      st_stream(y + base + k * 32 + lane,
                layer_vec<kAffine>(h[k], mean, inverse, scale, bias, static_cast<uint64_t>(k * 32 + lane) * 8));
  }
}

// One CTA per row, the row staged in shared memory: any hidden up to kMaxStagedHidden.
template <bool kAffine>
__global__ void __launch_bounds__(kThreads)
layer_norm_cta_kernel(const unsigned short *x, const unsigned short *__restrict__ scale,
                      const unsigned short *__restrict__ bias, unsigned short *y, uint64_t rows, uint32_t hidden,
                      float eps) {
  grid_dependency_sync();
  extern __shared__ __align__(16) unsigned char staged_bytes[];
  __shared__ float s_partial[2][kWarps];
  unsigned short *staged = reinterpret_cast<unsigned short *>(staged_bytes);
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  auto cta_sum = [&](float v, int slot) {
    v = warp_sum(v);
    if (lane == 0) s_partial[slot][warp] = v;
    __syncthreads();
    float total = s_partial[slot][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total = __fadd_rn(total, s_partial[slot][w]);
    return total;
  };
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint64_t base = row * hidden;
    float sum = 0.0f;
    for (uint32_t i = t; i < hidden; i += kThreads) {
      const unsigned short h = x[base + i];
      staged[i] = h;
      sum = __fadd_rn(sum, bf16_to_f32(h));
    }
    const float mean = __fdiv_rn(cta_sum(sum, 0), static_cast<float>(hidden));
    float ss = 0.0f;
    for (uint32_t i = t; i < hidden; i += kThreads) {
      const float c = __fsub_rn(bf16_to_f32(staged[i]), mean);
      ss = fmaf(c, c, ss);
    }
    const float inverse = inverse_rms(cta_sum(ss, 1), hidden, eps);
    for (uint32_t i = t; i < hidden; i += kThreads)
      y[base + i] = f32_to_bf16(layer_value(bf16_to_f32(staged[i]), mean, inverse, kAffine,
                                            kAffine ? bf16_to_f32(scale[i]) : 0.0f, kAffine ? bf16_to_f32(bias[i]) : 0.0f));
    __syncthreads();  // the staged row and the partial slots are rewritten by the next iteration
  }
}

template <bool kAffine>
int launch_layer_norm(cudaStream_t stream, const void *x, const void *scale, const void *bias, void *y, uint64_t rows,
                      uint64_t hidden, float eps) {
  const bool aligned = aligned_to(x, 16) && aligned_to(y, 16) && (!kAffine || (aligned_to(scale, 16) && aligned_to(bias, 16)));
  const int sms = sm_count();
  auto warp_launch = [&](auto vectors_tag) {
    constexpr int kVectors = decltype(vectors_tag)::value;
    int warps_per_cta = 2;
    if (rows < static_cast<uint64_t>(sms) * 2) warps_per_cta = 1;
    const unsigned grid = clamp_grid((rows + warps_per_cta - 1) / warps_per_cta, 1u << 20);
    return launch(layer_norm_warp_kernel<kVectors, kAffine>, dim3(grid), dim3(warps_per_cta * 32), 0, stream,
                  static_cast<const uint4 *>(x), static_cast<const unsigned short *>(scale),
                  static_cast<const unsigned short *>(bias), static_cast<uint4 *>(y), rows, eps);
  };
  if (aligned && hidden == 256) return warp_launch(std::integral_constant<int, 1>{});
  if (aligned && hidden == 512) return warp_launch(std::integral_constant<int, 2>{});
  if (aligned && hidden == 1024) return warp_launch(std::integral_constant<int, 4>{});
  if (aligned && hidden == 2048) return warp_launch(std::integral_constant<int, 8>{});
  if (hidden > kMaxStagedHidden) return HYLE_B200_NOT_SUPPORTED;
  const size_t staged = (static_cast<size_t>(hidden) * 2 + 15) & ~static_cast<size_t>(15);
  auto kernel = layer_norm_cta_kernel<kAffine>;
  if (staged > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  return launch(kernel, dim3(clamp_grid(rows, static_cast<uint64_t>(sms) * 4)), dim3(kThreads), staged, stream,
                static_cast<const unsigned short *>(x), static_cast<const unsigned short *>(scale),
                static_cast<const unsigned short *>(bias), static_cast<unsigned short *>(y), rows,
                static_cast<uint32_t>(hidden), eps);
}

// ================================================================================================
// Softmax{kSoftmax, scale, mask = kBoolean} on f16 rows, the attention-score form the CPU route
// keeps (src/compute_provider_native/transformer.cc:44-57,228-275):
//   v = f32(x) * scale;  v = -inf where the mask byte is 0;  y = f16_rne(softmax_f32(v))
// with softmax_f32 as in src/simd/math/activations.cc:301-317 (f32 exp of v - max, multiply by
// float(1 / sum); a row with NaN or +inf, or with every element masked, is all NaN).
// One CTA per row; the row stays in registers (16 values per thread) up to 4096 columns and is
// re-read from L1/L2 beyond that.  The mask has the tensor's shape or repeats over the leading
// axes with a period that is a multiple of the row length.
// kAdditive: Softmax{mask = kAdditive} (include/hyle/compute/operation.h:122-126), the mask an f16
// tensor added after the scaling, v = f32(x) * scale + f32(mask), as the reference's CUDA kernel forms
// it (src/compute_provider_cuda/reduction_kernel.cu:131-146); -inf entries mask, a row left without a
// finite maximum (or holding NaN / +inf) is all NaN as above.
// ================================================================================================
// One masked value: the Boolean form selects, the additive form adds.
template <bool kAdditive>
__device__ __forceinline__ float masked_score(float scaled, uint32_t mask_word) {
  if constexpr (kAdditive) return __fadd_rn(scaled, f16_to_f32(static_cast<unsigned short>(mask_word)));
  else return mask_word == 0 ? -CUDART_INF_F : scaled;
}
// Mask element e (0..7) of one 8-element step: a byte of a uint2, or a half of a uint4.
template <bool kAdditive> struct MaskVector { using Type = uint2; };
template <> struct MaskVector<true> { using Type = uint4; };
template <bool kAdditive>
__device__ __forceinline__ uint32_t mask_element(const typename MaskVector<kAdditive>::Type &m, int e) {
  if constexpr (kAdditive) {
    const uint32_t words[4] = {m.x, m.y, m.z, m.w};
    return e & 1 ? words[e / 2] >> 16 : words[e / 2] & 0xffffu;
  } else {
    return ((e < 4 ? m.x : m.y) >> (8 * (e & 3))) & 0xffu;
  }
}
template <bool kAdditive>
__device__ __forceinline__ typename MaskVector<kAdditive>::Type masked_padding() {
  // padding slots must not count: Boolean 0 = masked; additive -inf (0xfc00 in both halves)
  if constexpr (kAdditive) return make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);
  else return make_uint2(0, 0);
}
constexpr int kScoreSlots = 16;

template <bool kAdditive>
__global__ void __launch_bounds__(kThreads)
masked_softmax_f16_kernel(const unsigned short *x, const void *__restrict__ mask_storage, unsigned short *y, uint64_t rows,
                          uint32_t cols, uint64_t mask_rows, float scale) {
  using MaskWord = typename std::conditional<kAdditive, unsigned short, unsigned char>::type;
  const MaskWord *mask = static_cast<const MaskWord *>(mask_storage);
  grid_dependency_sync();
  __shared__ float s_part[2][kWarps];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const bool resident = cols <= kThreads * kScoreSlots;
  auto value_at = [&](const unsigned short *row, const MaskWord *row_mask, uint32_t i) {
    return masked_score<kAdditive>(__fmul_rn(f16_to_f32(row[i]), scale), row_mask[i]);
  };
  auto cta_reduce = [&](float v, int slot, bool maximum) {
    v = maximum ? warp_max_nan(v) : warp_sum(v);
    if (lane == 0) s_part[slot][warp] = v;
    __syncthreads();
    float total = s_part[slot][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total = maximum ? max_nan(total, s_part[slot][w]) : __fadd_rn(total, s_part[slot][w]);
    return total;
  };
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const unsigned short *in = x + row * cols;
    const MaskWord *row_mask = mask + (row % mask_rows) * cols;
    unsigned short *out = y + row * cols;
    float v[kScoreSlots];
    float peak = -CUDART_INF_F;
    if (resident) {
#pragma unroll
      for (int k = 0; k < kScoreSlots; ++k) {
        const uint32_t i = k * kThreads + t;
        v[k] = i < cols ? value_at(in, row_mask, i) : -CUDART_INF_F;
        peak = max_nan(peak, v[k]);
      }
    } else {
      for (uint32_t i = t; i < cols; i += kThreads) peak = max_nan(peak, value_at(in, row_mask, i));
    }
    peak = cta_reduce(peak, 0, true);
    const bool valid = peak > -CUDART_INF_F && peak < CUDART_INF_F;  // false for NaN too
    float sum = 0.0f;
    if (resident) {
#pragma unroll
      for (int k = 0; k < kScoreSlots; ++k) {
        v[k] = expf(v[k] - peak);  // exp(-inf) = 0 for masked and padding slots
        sum += v[k];
      }
    } else {
      for (uint32_t i = t; i < cols; i += kThreads) sum += expf(value_at(in, row_mask, i) - peak);
    }
    sum = cta_reduce(sum, 1, false);
    const float inverse = valid ? __fdiv_rn(1.0f, sum) : CUDART_NAN_F;
    if (resident) {
#pragma unroll
      for (int k = 0; k < kScoreSlots; ++k) {
        const uint32_t i = k * kThreads + t;
        if (i < cols) out[i] = f32_to_f16(valid ? __fmul_rn(v[k], inverse) : CUDART_NAN_F);
      }
    } else {
      for (uint32_t i = t; i < cols; i += kThreads)
        out[i] = f32_to_f16(valid ? __fmul_rn(expf(value_at(in, row_mask, i) - peak), inverse) : CUDART_NAN_F);
    }
    __syncthreads();  // the partial slots are rewritten by the next row
  }
}

// Rows of 1024-4096 values whose length is a multiple of 8, 16-byte aligned: eight values per
// thread-step (one 16-byte load of scores, one 8-byte load of mask bytes, one 16-byte store), the row
// resident in registers, exp as ex2.approx of the scaled difference (relative error about 1e-6, far
// inside the f16 step the result is rounded to).
constexpr int kVectorSlots = 2;

template <bool kAdditive>
__global__ void __launch_bounds__(kThreads)
masked_softmax_f16_vector_kernel(const uint4 *__restrict__ x, const typename MaskVector<kAdditive>::Type *__restrict__ mask,
                                 uint4 *__restrict__ y, uint64_t rows, uint32_t vectors, uint64_t mask_rows, float scale) {
  grid_dependency_sync();
  __shared__ float s_part[2][kWarps];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  auto cta_reduce = [&](float v, int slot, bool maximum) {
    v = maximum ? warp_max_nan(v) : warp_sum(v);
    if (lane == 0) s_part[slot][warp] = v;
    __syncthreads();
    float total = s_part[slot][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total = maximum ? max_nan(total, s_part[slot][w]) : __fadd_rn(total, s_part[slot][w]);
    return total;
  };
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4 *in = x + row * vectors;
    const typename MaskVector<kAdditive>::Type *row_mask = mask + (row % mask_rows) * vectors;
    float v[kVectorSlots][8];
    float peak = -CUDART_INF_F;
#pragma unroll
    for (int k = 0; k < kVectorSlots; ++k) {
      const uint32_t i = k * kThreads + t;
      if (i < vectors) {
        const uint4 w = ld_stream(in + i);
        const auto m = __ldg(row_mask + i);
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const unsigned short half = static_cast<unsigned short>(e & 1 ? words[e / 2] >> 16 : words[e / 2] & 0xffffu);
          v[k][e] = masked_score<kAdditive>(__fmul_rn(f16_to_f32(half), scale), mask_element<kAdditive>(m, e));
          peak = max_nan(peak, v[k][e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[k][e] = -CUDART_INF_F;
      }
    }
    peak = cta_reduce(peak, 0, true);
    const bool valid = peak > -CUDART_INF_F && peak < CUDART_INF_F;  // false for NaN too
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < kVectorSlots; ++k) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float weight;  // exp(v - peak); masked and padding slots give ex2(-inf) = 0
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(weight) : "f"(__fmul_rn(__fsub_rn(v[k][e], peak), 1.4426950408889634f)));
        v[k][e] = weight;
        sum += weight;
      }
    }
    sum = cta_reduce(sum, 1, false);
    const float inverse = valid ? __fdiv_rn(1.0f, sum) : CUDART_NAN_F;
#pragma unroll
    for (int k = 0; k < kVectorSlots; ++k) {
      const uint32_t i = k * kThreads + t;
      if (i < vectors) {
        uint32_t words[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)  // inverse is NaN for an invalid row, and NaN times any weight is NaN
          words[e] = pack_f16x2(__fmul_rn(v[k][2 * e], inverse), __fmul_rn(v[k][2 * e + 1], inverse));
        st_stream(y + row * vectors + i, make_uint4(words[0], words[1], words[2], words[3]));
      }
    }
    __syncthreads();  // the partial slots are rewritten by the next row
  }
}

// Rows of up to 2048 values (a multiple of 8): one WARP per row, the row in registers (up to eight
// 16-byte loads in flight per lane), shuffles only -- no barrier between the three phases of a row.
// The kernel is bound by instruction issue and by the XU pipe (exponentials and conversions), not by
// HBM alone, so the per-value work is kept short.  Always: an invalid row multiplies by inverse = NaN,
// which needs no select, and two results leave in one packed f32 -> f16x2 conversion.  kFast, for
// |scale| <= 32 (every attention scale):
//   - the weight is ex2(fma(v, log2e, -c)) with c = RN(peak * log2e) instead of ex2((v - peak) * log2e).
//     c differs from peak * log2e by at most half an ulp of c, which is 2^-3 for the values an f16 score
//     times 32 (plus an f16 addend) can reach, and every exponent of the row is off by that same amount:
//     it cancels in the normalisation.  (For larger scales half an ulp of c could overflow the exponential
//     of the maximum itself; they keep the exact subtraction.)
//   - Boolean masks with a positive scale fold it into the same fma, ex2(fma(x, scale * log2e, -c)), the
//     maximum taken over the unscaled values (a positive scale keeps the order, NaN and the infinities); a
//     masked value is -inf before and after;
//   - the additive form makes v = fma(x, scale, addend) (one rounding where the reference's kernel has two:
//     an f32 ulp, against an f16 result).
template <int kSlots, bool kAdditive, bool kFast>
__global__ void __launch_bounds__(128)
masked_softmax_f16_warp_kernel(const uint4 *__restrict__ x, const typename MaskVector<kAdditive>::Type *__restrict__ mask,
                               uint4 *__restrict__ y, uint64_t rows, uint32_t vectors, uint64_t mask_rows, float scale) {
  grid_dependency_sync();
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr bool kFold = kFast && !kAdditive;
  const int lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x / 32);
  const float factor = kFold ? __fmul_rn(scale, kLog2e) : kLog2e;  // of the stored value v in the exponent
  for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; row < rows; row += warps) {
    const uint4 *in = x + row * vectors;
    const typename MaskVector<kAdditive>::Type *row_mask = mask + (row % mask_rows) * vectors;
    uint4 w[kSlots];
    typename MaskVector<kAdditive>::Type m[kSlots];
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
      const uint32_t i = k * 32 + lane;
      w[k] = i < vectors ? ld_stream(in + i) : make_uint4(0, 0, 0, 0);
      m[k] = i < vectors ? __ldg(row_mask + i) : masked_padding<kAdditive>();  // padding counts as masked
    }
    float v[kSlots][8];
    float peak = -CUDART_INF_F;
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
      const uint32_t words[4] = {w[k].x, w[k].y, w[k].z, w[k].w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const unsigned short half = static_cast<unsigned short>(e & 1 ? words[e / 2] >> 16 : words[e / 2] & 0xffffu);
        const uint32_t mask_word = mask_element<kAdditive>(m[k], e);
        if constexpr (kFold) v[k][e] = mask_word == 0 ? -CUDART_INF_F : f16_to_f32(half);
        else if constexpr (kFast) v[k][e] = __fmaf_rn(f16_to_f32(half), scale, f16_to_f32(static_cast<unsigned short>(mask_word)));
        else v[k][e] = masked_score<kAdditive>(__fmul_rn(f16_to_f32(half), scale), mask_word);
        peak = max_nan(peak, v[k][e]);
      }
    }
    peak = warp_max_nan(peak);
    const bool valid = peak > -CUDART_INF_F && peak < CUDART_INF_F;  // false for NaN too
    const float neg_c = valid ? -__fmul_rn(peak, factor) : 0.0f;
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float exponent = kFast ? __fmaf_rn(v[k][e], factor, neg_c) : __fmul_rn(__fsub_rn(v[k][e], peak), kLog2e);
        float weight;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(weight) : "f"(exponent));
        v[k][e] = weight;
        sum += weight;
      }
    }
    sum = warp_sum(sum);
    const float inverse = valid ? __fdiv_rn(1.0f, sum) : CUDART_NAN_F;  // NaN times any weight is NaN
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
      const uint32_t i = k * 32 + lane;
      if (i < vectors) {
        uint32_t words[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) words[e] = pack_f16x2(__fmul_rn(v[k][2 * e], inverse), __fmul_rn(v[k][2 * e + 1], inverse));
        st_stream(y + row * vectors + i, make_uint4(words[0], words[1], words[2], words[3]));
      }
    }
  }
}

template <int kSlots, bool kAdditive>
int launch_masked_softmax_warp(cudaStream_t stream, const void *in, const void *mask, void *out, uint64_t rows,
                               uint32_t vectors, uint64_t mask_rows, float scale) {
  const unsigned grid = clamp_grid((rows + 3) / 4, static_cast<uint64_t>(sm_count()) * 16);
  const bool fast = kAdditive ? (scale >= -32.0f && scale <= 32.0f) : (scale > 0.0f && scale <= 32.0f);  // false for NaN
  return launch(fast ? masked_softmax_f16_warp_kernel<kSlots, kAdditive, true> : masked_softmax_f16_warp_kernel<kSlots, kAdditive, false>,
                dim3(grid), dim3(128), 0, stream, static_cast<const uint4 *>(in),
                static_cast<const typename MaskVector<kAdditive>::Type *>(mask), static_cast<uint4 *>(out), rows, vectors, mask_rows,
                scale);
}

template <bool kAdditive>
int launch_masked_softmax(cudaStream_t s, const void *in, const void *mask, uint64_t mask_count, float scale, void *out, uint64_t rows,
                          uint64_t cols) {
  const unsigned grid = clamp_grid(rows, static_cast<uint64_t>(sm_count()) * 8);
  const bool vector_ok = cols % 8 == 0 && aligned_to(in, 16) && aligned_to(out, 16) && aligned_to(mask, kAdditive ? 16 : 8);
  const uint64_t mask_rows = mask_count / cols;
  if (vector_ok && cols <= 2048) {
    const uint32_t vectors = static_cast<uint32_t>(cols / 8);
    if (vectors <= 32) return launch_masked_softmax_warp<1, kAdditive>(s, in, mask, out, rows, vectors, mask_rows, scale);
    if (vectors <= 64) return launch_masked_softmax_warp<2, kAdditive>(s, in, mask, out, rows, vectors, mask_rows, scale);
    if (vectors <= 128) return launch_masked_softmax_warp<4, kAdditive>(s, in, mask, out, rows, vectors, mask_rows, scale);
    return launch_masked_softmax_warp<8, kAdditive>(s, in, mask, out, rows, vectors, mask_rows, scale);
  }
  if (vector_ok && cols <= static_cast<uint64_t>(kThreads) * 8 * kVectorSlots)
    return launch(masked_softmax_f16_vector_kernel<kAdditive>, dim3(grid), dim3(kThreads), 0, s, static_cast<const uint4 *>(in),
                  static_cast<const typename MaskVector<kAdditive>::Type *>(mask), static_cast<uint4 *>(out), rows,
                  static_cast<uint32_t>(cols / 8), mask_rows, scale);
  return launch(masked_softmax_f16_kernel<kAdditive>, dim3(grid), dim3(kThreads), 0, s, static_cast<const unsigned short *>(in), mask,
                static_cast<unsigned short *>(out), rows, static_cast<uint32_t>(cols), mask_rows, scale);
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" int hyle_b200_reduce_rows_f32(hyle_b200_stream_t stream, int kind, const float *in,
                                         float *out, uint64_t rows, uint64_t cols) {
  if (rows == 0) return HYLE_B200_OK;
  if (out == nullptr || (in == nullptr && cols != 0) || kind < HYLE_B200_REDUCE_SUM ||
      kind > HYLE_B200_REDUCE_MAXIMUM)
    return HYLE_B200_INVALID_VALUE;
  RowF32Params p{};
  p.a = in;
  p.rows = rows;
  p.cols = cols;
  p.mean = kind == HYLE_B200_REDUCE_MEAN;
  if (kind == HYLE_B200_REDUCE_SUM || kind == HYLE_B200_REDUCE_MEAN) p.row_sum = out;
  if (kind == HYLE_B200_REDUCE_MAXIMUM) p.row_max = out;
  if (kind == HYLE_B200_REDUCE_MINIMUM) p.row_min = out;
  return launch_row_f32<kOpNone>(reinterpret_cast<cudaStream_t>(stream), p);
}

extern "C" int hyle_b200_reduce_rows_extremum(hyle_b200_stream_t stream, int kind, int dtype, const void *in, void *out,
                                              uint64_t rows, uint64_t cols) {
  if (rows == 0) return HYLE_B200_OK;
  if (out == nullptr || (in == nullptr && cols != 0) || (kind != HYLE_B200_REDUCE_MINIMUM && kind != HYLE_B200_REDUCE_MAXIMUM) ||
      (dtype != HYLE_B200_BF16 && dtype != HYLE_B200_F16) || !aligned_to(in, 2) || !aligned_to(out, 2))
    return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const bool maximum = kind == HYLE_B200_REDUCE_MAXIMUM;
  if (dtype == HYLE_B200_BF16)
    return maximum ? launch_narrow_extremum<HYLE_B200_BF16, true>(s, in, out, rows, cols)
                   : launch_narrow_extremum<HYLE_B200_BF16, false>(s, in, out, rows, cols);
  return maximum ? launch_narrow_extremum<HYLE_B200_F16, true>(s, in, out, rows, cols)
                 : launch_narrow_extremum<HYLE_B200_F16, false>(s, in, out, rows, cols);
}

extern "C" int hyle_b200_add_bias_row_sum_max_f32(hyle_b200_stream_t stream, const float *a,
                                                  const float *bias, float *c, float *row_sum,
                                                  float *row_max, uint64_t rows, uint64_t cols) {
  if (rows == 0) return HYLE_B200_OK;
  if ((a == nullptr || bias == nullptr) && cols != 0) return HYLE_B200_INVALID_VALUE;
  RowF32Params p{};
  p.a = a;
  p.rhs = bias;
  p.c = c;
  p.row_sum = row_sum;
  p.row_max = row_max;
  p.rows = rows;
  p.cols = cols;
  return launch_row_f32<HYLE_B200_BINARY_ADD>(reinterpret_cast<cudaStream_t>(stream), p);
}

extern "C" int hyle_b200_rms_norm_bf16(hyle_b200_stream_t stream, const void *x, const void *weight,
                                       int weight_dtype, void *y, uint64_t rows, uint64_t hidden,
                                       float epsilon) {
  return dispatch_rms<false>(reinterpret_cast<cudaStream_t>(stream), x, nullptr, weight, weight_dtype,
                             y, nullptr, rows, hidden, epsilon);
}

extern "C" int hyle_b200_rms_norm(hyle_b200_stream_t stream, int dtype, const void *x, const void *weight, int weight_dtype,
                                  void *y, uint64_t rows, uint64_t hidden, float epsilon) {
  auto s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case HYLE_B200_BF16: return dispatch_rms<false>(s, x, nullptr, weight, weight_dtype, y, nullptr, rows, hidden, epsilon);
    case HYLE_B200_F16: return dispatch_rms_stored<HYLE_B200_F16>(s, x, weight, weight_dtype, y, rows, hidden, epsilon);
    case HYLE_B200_F32: return dispatch_rms_stored<HYLE_B200_F32>(s, x, weight, weight_dtype, y, rows, hidden, epsilon);
    default: return HYLE_B200_INVALID_VALUE;
  }
}

extern "C" int hyle_b200_add_rms_norm_bf16(hyle_b200_stream_t stream, const void *x,
                                           const void *residual, const void *weight,
                                           int weight_dtype, void *y, void *h, uint64_t rows,
                                           uint64_t hidden, float epsilon) {
  return dispatch_rms<true>(reinterpret_cast<cudaStream_t>(stream), x, residual, weight, weight_dtype,
                            y, h, rows, hidden, epsilon);
}

extern "C" int hyle_b200_layer_norm_bf16(hyle_b200_stream_t stream, const void *x, const void *scale,
                                         const void *bias, void *y, uint64_t rows, uint64_t hidden,
                                         float epsilon) {
  if (rows == 0 || hidden == 0) return HYLE_B200_OK;
  if (x == nullptr || y == nullptr || (scale == nullptr) != (bias == nullptr)) return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (scale == nullptr) return launch_layer_norm<false>(s, x, nullptr, nullptr, y, rows, hidden, epsilon);
  return launch_layer_norm<true>(s, x, scale, bias, y, rows, hidden, epsilon);
}

extern "C" int hyle_b200_masked_softmax_f16(hyle_b200_stream_t stream, const void *in, const unsigned char *mask,
                                            uint64_t mask_count, float scale, void *out, uint64_t rows,
                                            uint64_t cols) {
  if (rows == 0 || cols == 0) return HYLE_B200_OK;
  if (in == nullptr || mask == nullptr || out == nullptr || cols > 0x7fffffffull || mask_count == 0 ||
      mask_count % cols != 0 || (rows * cols) % mask_count != 0 || !aligned_to(in, 2) || !aligned_to(out, 2))
    return HYLE_B200_INVALID_VALUE;
  return launch_masked_softmax<false>(reinterpret_cast<cudaStream_t>(stream), in, mask, mask_count, scale, out, rows, cols);
}

extern "C" int hyle_b200_additive_masked_softmax_f16(hyle_b200_stream_t stream, const void *in, const void *mask_f16,
                                                     uint64_t mask_count, float scale, void *out, uint64_t rows,
                                                     uint64_t cols) {
  if (rows == 0 || cols == 0) return HYLE_B200_OK;
  if (in == nullptr || mask_f16 == nullptr || out == nullptr || cols > 0x7fffffffull || mask_count == 0 ||
      mask_count % cols != 0 || (rows * cols) % mask_count != 0 || !aligned_to(in, 2) || !aligned_to(out, 2) ||
      !aligned_to(mask_f16, 2))
    return HYLE_B200_INVALID_VALUE;
  return launch_masked_softmax<true>(reinterpret_cast<cudaStream_t>(stream), in, mask_f16, mask_count, scale, out, rows, cols);
}

// Device helpers shared by the sm_100a kernels: streaming vector loads/stores, bf16/f16 storage
// conversions with the reference's rounding (include/hyle/simd/dtype.h:55-121), NaN-propagating
// extrema and fixed-order warp/CTA reductions.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "hyle_b200.h"

namespace hb {

constexpr int kWarpSize = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// ---- argument checks shared by the entry points ----------------------------------------------
inline bool aligned_to(const void *p, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0;
}

// Number of SMs of the current device, cached per device (a host-side query, no allocation).
int sm_count();

// ---- streaming global memory access ----------------------------------------------------------
// Every operand of these operators is touched once per launch, so loads and stores carry the
// evict-first hint and leave L2 to the small reused vectors (bias, norm weight).
__device__ __forceinline__ uint4 ld_stream(const uint4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4 *p, uint4 v) { __stcs(p, v); }
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ uint2 ld_stream(const uint2 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint2 *p, uint2 v) { __stcs(p, v); }
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float *p, float v) { __stcs(p, v); }
__device__ __forceinline__ unsigned short ld_stream(const unsigned short *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(unsigned short *p, unsigned short v) { __stcs(p, v); }

// ---- bf16 / f16 storage ------------------------------------------------------------------------
// bf16 is the top half of an f32 (include/hyle/simd/dtype.h:105-107).
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float bf16_to_f32(unsigned short b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
// Two f32 -> packed bf16 pair, round to nearest even (dtype.h:114-121).  NaN becomes the canonical
// quiet NaN 0x7fff where the reference keeps the payload; both are NaN.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ unsigned short f32_to_bf16(float v) {
  return static_cast<unsigned short>(pack_bf16x2(v, 0.0f) & 0xffffu);
}
__device__ __forceinline__ float f16_to_f32(unsigned short h) {
  float r;
  asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(h));
  return r;
}
// Two f32 -> packed f16 pair, round to nearest even, one conversion instruction for both.
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ unsigned short f32_to_f16(float v) {
  unsigned short r;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
  return r;
}

// ---- extrema -----------------------------------------------------------------------------------
// NaN-propagating maximum/minimum with -0 < +0: the Reduce{kMaximum|kMinimum} rule
// (src/compute_provider_native/reduction.cc:34-47, docs/user/compute.md:384-388).
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// ---- warp reductions (xor butterfly: every lane ends with the same value, fixed order) ---------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_nan(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max_nan(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}
__device__ __forceinline__ float warp_min_nan(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min_nan(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

// ---- launch helpers ----------------------------------------------------------------------------
inline int launch_result() { return static_cast<int>(cudaPeekAtLastError()); }

// Programmatic dependent launch.  Most of these operators run for 10-30 us, where the few
// microseconds between the end of one grid and the first CTA of the next are a visible fraction.
// Every kernel is launched with programmatic stream serialisation allowed and begins with
// grid_dependency_sync(): the CTAs of the next grid in the stream may be placed on SMs while the
// previous grid drains, but none of them touches global memory before the previous grid has
// completed and flushed (griddepcontrol.wait).  With a predecessor that never signals, or without
// the launch attribute, both instructions do nothing, so stream order is unchanged in every case.
__device__ __forceinline__ void grid_dependency_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <class... Params, class... Args>
inline int launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                  Args &&...args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...));
}

inline unsigned clamp_grid(uint64_t blocks, uint64_t limit) {
  if (blocks < 1) blocks = 1;
  return static_cast<unsigned>(blocks < limit ? blocks : limit);
}

}  // namespace hb

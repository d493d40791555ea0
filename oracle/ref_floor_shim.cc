// extern "C" doorway onto the reference's own scalar floor -- TEST INFRASTRUCTURE.
//
// This translation unit contains no arithmetic of its own.  It is compiled together with the
// reference's Highway-free sources, in place from the mounted reference tree (oracle/Makefile):
//   src/simd/math/activations.cc   swiglu_bf16_scalar, rms_norm_bf16_scalar, softmax_f32_scalar,
//                                  log_softmax_f32_scalar, {sigmoid,gelu,gelu_tanh,silu,relu}_f32_scalar, layer_norm_bf16_scalar
//   src/simd/sort/top_k.cc         top_k_f32
//   third_party/random123_counter/philox.h   word (the counter generator behind RandomBits)
//   include/hyle/simd/dtype.h      f32_to_bf16, bf16_to_f32, f32_to_f16, f16_to_f32, f32_to_f8e4m3, f8e4m3_to_f32,
//                                  f32_to_f8e5m2, f8e5m2_to_f32
// and only forwards row by row, so tests can pin oracle/hyle_oracle.c against the reference's code
// and the benchmark can time the reference's code on the host cores.  Rows are split over threads
// in contiguous ranges like the reference's parallel_for_ranges
// (src/compute_provider_native/native_plan.h:94-111).
#include <cstddef>
#include <cstdint>

#include "hyle/simd/dtype.h"
#include "hyle/simd/sort.h"
#include "src/simd/math/kernels.h"
#include "third_party/random123_counter/philox.h"

#ifdef _OPENMP
#include <omp.h>
#endif

namespace simd = hyle::simd;

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void hyle_ref_set_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
}

REF_API uint16_t hyle_ref_f32_to_bf16(float v) { return simd::f32_to_bf16(v).bits; }
REF_API float hyle_ref_bf16_to_f32(uint16_t v) { return simd::bf16_to_f32(simd::bfloat16_t::from_bits(v)); }
REF_API uint16_t hyle_ref_f32_to_f16(float v) { return simd::f32_to_f16(v).bits; }
REF_API float hyle_ref_f16_to_f32(uint16_t v) { return simd::f16_to_f32(simd::float16_t::from_bits(v)); }

REF_API uint8_t hyle_ref_f32_to_e4m3(float v) { return simd::f32_to_f8e4m3(v).bits; }
REF_API float hyle_ref_e4m3_to_f32(uint8_t v) { return simd::f8e4m3_to_f32(simd::float8_e4m3_t::from_bits(v)); }
REF_API uint8_t hyle_ref_f32_to_e5m2(float v) { return simd::f32_to_f8e5m2(v).bits; }
REF_API float hyle_ref_e5m2_to_f32(uint8_t v) { return simd::f8e5m2_to_f32(simd::float8_e5m2_t::from_bits(v)); }

// word `index` of the counter stream of one identity (third_party/random123_counter/philox.h)
REF_API uint32_t hyle_ref_random_word(const uint32_t *identity, uint64_t index) {
  return hyle::borrowed::random123_counter::word(identity, index);
}

REF_API void hyle_ref_swiglu_bf16(const uint16_t *gate, const uint16_t *up, uint16_t *out, uint64_t rows,
                                  uint64_t cols, uint64_t gate_stride, uint64_t up_stride) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r)
    simd::detail::swiglu_bf16_scalar(reinterpret_cast<const simd::bfloat16_t *>(gate + r * gate_stride),
                                     reinterpret_cast<const simd::bfloat16_t *>(up + r * up_stride),
                                     reinterpret_cast<simd::bfloat16_t *>(out + r * cols), cols);
}

REF_API void hyle_ref_rms_norm_bf16(const uint16_t *x, const uint16_t *weight, uint16_t *y, uint64_t rows,
                                    uint64_t hidden, float eps) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r)
    simd::detail::rms_norm_bf16_scalar(reinterpret_cast<const simd::bfloat16_t *>(x + r * hidden),
                                       reinterpret_cast<const simd::bfloat16_t *>(weight),
                                       reinterpret_cast<simd::bfloat16_t *>(y + r * hidden), hidden, eps);
}

REF_API void hyle_ref_layer_norm_bf16(const uint16_t *x, const uint16_t *scale, const uint16_t *bias, uint16_t *y,
                                      uint64_t rows, uint64_t hidden, float eps) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r)
    simd::detail::layer_norm_bf16_scalar(reinterpret_cast<const simd::bfloat16_t *>(x + r * hidden),
                                         reinterpret_cast<const simd::bfloat16_t *>(scale),
                                         reinterpret_cast<const simd::bfloat16_t *>(bias),
                                         reinterpret_cast<simd::bfloat16_t *>(y + r * hidden), hidden, eps);
}

// kind: 7 sigmoid, 8 relu, 9 gelu, 10 gelu_tanh, 11 silu (the numbering of hyle::compute::UnaryKind)
REF_API int hyle_ref_activation_f32(int kind, const float *in, float *out, uint64_t count) {
  switch (kind) {
    case 7: simd::detail::sigmoid_f32_scalar(in, out, count); return 0;
    case 8: simd::detail::relu_f32_scalar(in, out, count); return 0;
    case 9: simd::detail::gelu_f32_scalar(in, out, count); return 0;
    case 10: simd::detail::gelu_tanh_f32_scalar(in, out, count); return 0;
    case 11: simd::detail::silu_f32_scalar(in, out, count); return 0;
    default: return 1;
  }
}

REF_API void hyle_ref_softmax_f32(int log_kind, const float *in, float *out, uint64_t rows, uint64_t cols) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    if (log_kind) simd::detail::log_softmax_f32_scalar(in + r * cols, out + r * cols, cols);
    else simd::detail::softmax_f32_scalar(in + r * cols, out + r * cols, cols);
  }
}

REF_API void hyle_ref_argmax_f32(const float *in, int32_t *index, float *value, uint64_t rows, uint64_t cols) {
#pragma omp parallel for schedule(static)
  for (uint64_t r = 0; r < rows; ++r) {
    simd::ScoredIndexF32 best{};
    simd::top_k_f32(in + r * cols, cols, &best, 1);
    if (index) index[r] = static_cast<int32_t>(best.index);
    if (value) value[r] = best.score;
  }
}

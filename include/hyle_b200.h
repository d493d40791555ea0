/*
 * hyle_b200 -- C ABI of the B200 (sm_100a) kernel library for HYLE's elementwise, broadcast and
 * reduction operators.
 *
 * HYLE has no native FFI; its extension seam is the typed custom-kernel API
 * (include/hyle/compute/custom_kernel.h:302-360) and the model for a kernel library behind it is
 * the sample's `launch_affine(cudaStream_t, pointers, count, parameters) noexcept -> cudaError_t`
 * (samples/package/graph/custom_kernel/cuda_kernel.h:16-19): "no HYLE runtime or provider SPI
 * lives in this image".  Every operator entry point below has that shape (the four
 * hyle_b200_exchange_* helpers at the end are set-up code: they allocate and map memory):
 *
 *   - plain device pointers, element counts and scalars; no C++ or framework types;
 *   - stream-ordered: work is recorded on `stream` and the call returns without synchronising;
 *   - no allocation, no host synchronisation, no printing, safe under stream capture; scratch
 *     memory is passed in by the caller and sized by the
 *     matching *_workspace_bytes() query, the way a HYLE provider declares a caller-owned
 *     WorkspaceRequirement (include/hyle/compute/custom_kernel.h:39-52);
 *   - the return value is a cudaError_t-compatible int: 0 launched, 1 (cudaErrorInvalidValue)
 *     for arguments outside the documented domain, 801 (cudaErrorNotSupported) for a shape this
 *     library declines (the provider turns that into Status::Unimplemented so another provider
 *     can take the request), anything else is the CUDA launch error;
 *   - numeric problems found on the device are OR-ed into a caller-zeroed device status word,
 *     the protocol of src/compute_backend_cuda/device_status_kernel.h:7-13.
 *
 * All tensors are dense row-major.  bf16/f16 values are passed as 16-bit storage words.
 */
#ifndef HYLE_B200_H_
#define HYLE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(HYLE_B200_BUILD)
#define HYLE_B200_API __attribute__((visibility("default")))
#else
#define HYLE_B200_API
#endif

/* Same object as cudaStream_t; spelled out so C callers need no CUDA header. */
typedef struct CUstream_st *hyle_b200_stream_t;

#define HYLE_B200_ABI_VERSION 20

enum hyle_b200_result {
  HYLE_B200_OK = 0,
  HYLE_B200_INVALID_VALUE = 1,   /* cudaErrorInvalidValue */
  HYLE_B200_NOT_SUPPORTED = 801, /* cudaErrorNotSupported */
  /* hyle_b200_q8_0_roundtrip_bf16_static: count is above HYLE_B200_STATIC_MAX_VALUES. */
  HYLE_B200_STATIC_SCRATCH_EXCEEDED = 100001,
  /* hyle_b200_file_stream_*: the file cannot be opened, the range is not inside it, or a read failed. */
  HYLE_B200_IO_ERROR = 100002
};

/* Storage types, numbered independently of hyle::compute::DataType. */
enum hyle_b200_dtype {
  HYLE_B200_F32 = 0,
  HYLE_B200_BF16 = 1,
  HYLE_B200_F16 = 2,
  /* the remaining types are accepted by hyle_b200_cast only */
  HYLE_B200_E4M3 = 3, /* DataType::kFloat8E4M3FN: bias 7, no infinity, NaN 0x7F, largest normal 448 */
  HYLE_B200_E5M2 = 4, /* DataType::kFloat8E5M2: bias 15, IEEE-like */
  HYLE_B200_BOOL = 5, /* one byte, any non-zero value is true */
  HYLE_B200_I32 = 6
};

/* hyle::compute::BinaryKind (include/hyle/compute/operation.h:75-82); numbered independently. */
enum hyle_b200_binary_kind {
  HYLE_B200_BINARY_ADD = 0,
  HYLE_B200_BINARY_MULTIPLY = 1,
  HYLE_B200_BINARY_SUBTRACT = 2,
  HYLE_B200_BINARY_DIVIDE = 3,
  /* Number minimum / maximum: a NaN operand yields the other operand (NaN only if both are);
   * zeros of opposite sign give -0 for the minimum and +0 for the maximum whatever the operand
   * order (src/simd/ops/kernel_impl.h:256-267, include/hyle/simd/ops.h:77-79). */
  HYLE_B200_BINARY_MINIMUM = 4,
  HYLE_B200_BINARY_MAXIMUM = 5
};

/* hyle::compute::UnaryKind, same order (include/hyle/compute/operation.h:57-73). */
enum hyle_b200_unary_kind {
  HYLE_B200_UNARY_ABS = 0,
  HYLE_B200_UNARY_NEG = 1,
  HYLE_B200_UNARY_EXP = 2,
  HYLE_B200_UNARY_LOG = 3,
  HYLE_B200_UNARY_SQRT = 4,
  HYLE_B200_UNARY_RSQRT = 5, /* 1.0f / sqrt(x), not an approximation */
  HYLE_B200_UNARY_TANH = 6,
  HYLE_B200_UNARY_SIGMOID = 7,
  HYLE_B200_UNARY_RELU = 8,  /* NaN stays NaN */
  HYLE_B200_UNARY_GELU = 9,  /* erf form; gelu(-inf) = 0 */
  HYLE_B200_UNARY_GELU_TANH = 10,
  HYLE_B200_UNARY_SILU = 11, /* silu(-inf) = 0 */
  HYLE_B200_UNARY_SOFTPLUS = 12 /* log1p(exp(x)), x above 20 returned unchanged; softplus(-inf) = +0 */
};

/* hyle::compute::ReductionKind (include/hyle/compute/operation.h:84-89). */
enum hyle_b200_reduce_kind {
  HYLE_B200_REDUCE_SUM = 0,
  HYLE_B200_REDUCE_MEAN = 1,
  HYLE_B200_REDUCE_MINIMUM = 2,
  HYLE_B200_REDUCE_MAXIMUM = 3
};

/* hyle::compute::SoftmaxKind (include/hyle/compute/operation.h:117-120). */
enum hyle_b200_softmax_kind {
  HYLE_B200_SOFTMAX = 0,
  HYLE_B200_LOG_SOFTMAX = 1
};

/* Bits of the device status word. */
enum hyle_b200_status_bits {
  /* Q8_0 encode met a non-finite value or |x| > 65504*127; that block was written as 34 zero
   * bytes (src/compute_provider_ggml/ggml_cpu_provider.cc:596-608). */
  HYLE_B200_STATUS_INVALID_Q8_INPUT = 1u,
  /* hyle_b200_q8_0_roundtrip_bf16_exchange: a peer's sum did not arrive within poll_limit polls;
   * *sum_squares_out is NaN. */
  HYLE_B200_STATUS_EXCHANGE_TIMEOUT = 2u,
  /* hyle_b200_fp8_e4m3_encode met a non-finite value; that byte was written as 0
   * (src/compute_provider_ggml/ggml_cpu_provider.cc:591-594). */
  HYLE_B200_STATUS_INVALID_FP8_INPUT = 4u,
  /* hyle_b200_categorical met a row with NaN, +inf or no finite value; its index is -1. */
  HYLE_B200_STATUS_INVALID_CATEGORICAL_ROW = 8u,
  /* hyle_b200_scan on i32: a prefix left the int32 range; no output was written
   * (src/compute_provider_ggml/standard_index.cc:127-134). */
  HYLE_B200_STATUS_SCAN_OVERFLOW = 16u,
  /* hyle_b200_logits_reduce_f32 / hyle_b200_softmax_f32, streaming kernel: a second-pass task gave up
   * waiting for a row's first-pass partials (the launch did not get the co-resident CTAs it was sized
   * for) or a bulk copy never landed; the affected rows are NaN. */
  HYLE_B200_STATUS_STREAM_WAIT_TIMEOUT = 32u
};

HYLE_B200_API int hyle_b200_abi_version(void);
/* Static string for a result code; never NULL. */
HYLE_B200_API const char *hyle_b200_result_string(int result);

/* ---------------------------------------------------------------------------------------------
 * Binary{kAdd|kSubtract|kMultiply|kDivide|kMinimum|kMaximum} with NumPy trailing-axis broadcast of
 * the right operand.
 * Replaces: Binary schema include/hyle/compute/operation.h:301-303, broadcast inference
 * src/compute_ops/operation.cc:480-491, CPU route src/compute_provider_native/elementwise.cc:116-133
 * (one dense call per broadcast chunk, :333-348,540-571).
 * out[i] = lhs[i] (op) rhs[i % rhs_period] for i in [0,count).  rhs_period == count means no
 * broadcast; rhs_period == last-axes extent is the bias-over-rows case; count % rhs_period == 0.
 * f32: one IEEE operation per element (bit-exact).  bf16/f16: f32 operation, one RNE rounding.
 * out may alias lhs exactly.
 */
HYLE_B200_API int hyle_b200_binary(hyle_b200_stream_t stream, int kind, int dtype,
                                   const void *lhs, const void *rhs, void *out,
                                   uint64_t count, uint64_t rhs_period);

/* ---------------------------------------------------------------------------------------------
 * Unary{kind} on a dense tensor of f32 / bf16 / f16 (16-bit types: f32 math, one RNE rounding).
 * Replaces: Unary schema include/hyle/compute/operation.h:57-73, CPU route
 * src/compute_provider_native/elementwise.cc:30-100 (Neg, Exp, Log, Sqrt, Rsqrt, Tanh, Relu, Silu),
 * activation definitions src/simd/math/activations.cc:21-52 (Sigmoid, Gelu, GeluTanh, Silu, Relu),
 * Softplus src/compute_provider_native/aten_cpu_provider.cc:627-628.
 * Abs, Neg, Sqrt, Rsqrt, Relu are bit-exact; the others within 1e-5 relative in f32 and one
 * storage step in bf16 / f16.  out may alias in exactly.
 */
HYLE_B200_API int hyle_b200_unary(hyle_b200_stream_t stream, int kind, int dtype, const void *in,
                                  void *out, uint64_t count);

/* ---------------------------------------------------------------------------------------------
 * Reduce{kind, axes={-1}} over dense f32 rows.
 * Replaces: Reduce schema include/hyle/compute/operation.h:307-312, inference
 * src/compute_ops/operation.cc:1345-1394, CPU route src/compute_provider_native/reduction.cc:34-110.
 * Minimum/Maximum propagate NaN and order -0 < +0; empty rows give Sum=0, Mean=NaN,
 * Minimum=+inf, Maximum=-inf.  Sum/Mean use a fixed summation order (deterministic).
 */
HYLE_B200_API int hyle_b200_reduce_rows_f32(hyle_b200_stream_t stream, int kind,
                                            const float *in, float *out, uint64_t rows,
                                            uint64_t cols);

/* Fusion of Binary{kAdd}(A, bias[cols]) -> Reduce{kSum} and Reduce{kMaximum} over the last axis:
 * one read of A, one write of C, both row reductions taken from registers.  Results equal the
 * three separate calls above bit for bit (same summation order).  Any of c/row_sum/row_max may be
 * NULL to skip that output.
 */
/* Reduce{kMinimum | kMaximum, axes={-1}} over dense bf16 or f16 rows, the result in the rows' type:
 * the narrow Min/Max of the CPU route (src/compute_provider_native/reduction.cc:203-223: f16 both
 * kinds, bf16 the maximum; bf16 minimum is taken here as well).  Exact: the rules of
 * hyle_b200_reduce_rows_f32 on the converted values, and an extremum converts back unchanged. */
HYLE_B200_API int hyle_b200_reduce_rows_extremum(hyle_b200_stream_t stream, int kind, int dtype,
                                                 const void *in, void *out, uint64_t rows,
                                                 uint64_t cols);

HYLE_B200_API int hyle_b200_add_bias_row_sum_max_f32(hyle_b200_stream_t stream, const float *a,
                                                     const float *bias, float *c,
                                                     float *row_sum, float *row_max,
                                                     uint64_t rows, uint64_t cols);

/* ---------------------------------------------------------------------------------------------
 * RmsNorm{epsilon, accumulation=f32} on bf16 rows, weight bf16 or f32 (weight_dtype) or NULL.
 * Replaces: RmsNorm schema include/hyle/compute/operation.h:323-328, CPU route
 * src/compute_provider_native/normalization.cc:42-80 and the scalar floor
 * src/simd/math/activations.cc:124-146:
 *   inverse = 1.0f / sqrtf(sum(x*x)/hidden + epsilon);  y = bf16_rne((x * inverse) * w).
 * y may alias x exactly.
 */
HYLE_B200_API int hyle_b200_rms_norm_bf16(hyle_b200_stream_t stream, const void *x,
                                          const void *weight, int weight_dtype, void *y,
                                          uint64_t rows, uint64_t hidden, float epsilon);

/* RmsNorm on rows stored as dtype (HYLE_B200_BF16: the entry above; HYLE_B200_F16 and HYLE_B200_F32:
 * the other two storages the CPU route takes, src/compute_provider_native/normalization.cc:219-234),
 * same formula, the result rounded once to dtype.  weight: NULL, or [hidden] stored as dtype or as
 * f32 (weight_dtype).  Rows of more than 64 KB (f16, f32) are HYLE_B200_NOT_SUPPORTED.  y may alias
 * x exactly. */
HYLE_B200_API int hyle_b200_rms_norm(hyle_b200_stream_t stream, int dtype, const void *x,
                                     const void *weight, int weight_dtype, void *y, uint64_t rows,
                                     uint64_t hidden, float epsilon);

/* Fusion of Binary{kAdd} (bf16: f32 add, one RNE) with the RmsNorm above:
 *   h = bf16_rne(f32(x) + f32(residual));  y = RmsNorm(h)   -- the norm reads the ROUNDED h, so
 * the pair equals the unfused composition bit for bit.  h may alias residual or x; y may alias x.
 */
HYLE_B200_API int hyle_b200_add_rms_norm_bf16(hyle_b200_stream_t stream, const void *x,
                                              const void *residual, const void *weight,
                                              int weight_dtype, void *y, void *h,
                                              uint64_t rows, uint64_t hidden, float epsilon);

/* ---------------------------------------------------------------------------------------------
 * LayerNorm{epsilon, accumulation=f32} over the last axis of a bf16 tensor, with a bf16 scale and
 * bias of [hidden] (both or neither).
 * Replaces: LayerNorm schema include/hyle/compute/operation.h:330-333, scalar floor
 * src/simd/math/activations.cc:148-174:
 *   mean = sum(x) / hidden; inverse = 1.0f / sqrt(sum((x - mean)^2) / hidden + epsilon);
 *   y = bf16_rne(fma((x - mean) * inverse, scale, bias)).
 * hidden <= 32768.  The sums are taken in a fixed (tree) order; y is within one bf16 step of the
 * sequential-order result.
 */
HYLE_B200_API int hyle_b200_layer_norm_bf16(hyle_b200_stream_t stream, const void *x,
                                            const void *scale, const void *bias, void *y,
                                            uint64_t rows, uint64_t hidden, float epsilon);

/* ---------------------------------------------------------------------------------------------
 * GatedActivation{kSilu}: out = bf16_rne(silu(f32 gate) * f32 up), silu(-inf) = 0.
 * Replaces: GatedActivation schema include/hyle/compute/operation.h:91-100,362-365 and the scalar
 * floor src/simd/math/activations.cc:21-25,44-47,114-122.
 * Row strides are in elements: kSeparate passes gate/up with stride cols; kPackedHalves passes
 * gate = packed, up = packed + cols, both strides 2*cols.
 */
HYLE_B200_API int hyle_b200_swiglu_bf16(hyle_b200_stream_t stream, const void *gate,
                                        const void *up, void *out, uint64_t rows, uint64_t cols,
                                        uint64_t gate_row_stride, uint64_t up_row_stride);

/* hyle::compute::GatedActivationKind (include/hyle/compute/operation.h:91-95). */
enum hyle_b200_gate_kind {
  HYLE_B200_GATE_SILU = 0,
  HYLE_B200_GATE_GELU = 1,       /* 0.5 x (1 + erf(x / sqrt 2)) */
  HYLE_B200_GATE_GELU_TANH = 2   /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
};
/* GatedActivation{activation} on bf16 or f16 tensors (f16 separate is the form the native CPU route
 * keeps, src/compute_provider_native/elementwise.cc:660-704):
 *   out = storage_rne(activation(f32 gate) * f32 up), activation(-inf) = 0.
 * round_gate != 0 rounds activation(gate) to the storage type before the product: exactly
 * Unary{activation} followed by Binary{kMultiply} on 16-bit tensors, in one pass.  That is how a graph
 * region fuses those two nodes (engine/models/qwen35/block_graph.h:27-40 emits them for 16-bit
 * activations) without changing their result.  Strides as for hyle_b200_swiglu_bf16. */
HYLE_B200_API int hyle_b200_gated_activation(hyle_b200_stream_t stream, int activation, int dtype,
                                             int round_gate, const void *gate, const void *up,
                                             void *out, uint64_t rows, uint64_t cols,
                                             uint64_t gate_row_stride, uint64_t up_row_stride);

/* ---------------------------------------------------------------------------------------------
 * Logits reduction: per row of f32 logits, in one pass over HBM,
 *   lse[row]          = max + float(log(double sum exp(x - max)))      (the LogSoftmax shift)
 *   probs[row, :]     = bf16_rne(exp(x - max) * float(1 / sum))        (Softmax then Cast{bf16})
 *   argmax_index[row] = lowest index of the maximum, NaN ordered last  (TopK{count=1})
 *   argmax_value[row] = that element
 * Replaces: Softmax include/hyle/compute/operation.h:403-409 with src/simd/math/activations.cc:301-334,
 * Cast include/hyle/compute/operation.h:289-295, TopK include/hyle/compute/operation.h:411-417 with
 * src/simd/sort/top_k.cc:17-27,51-69.
 * Rows holding NaN or +inf, or only -inf, get NaN lse and NaN probs (include/hyle/simd/math.h:307-311);
 * argmax is still defined for them.  Any output pointer may be NULL.
 * Domain: finite logits below 2^27 (1.3e8) in magnitude.  The kernels subtract one constant,
 * RN(max * log2 e), from every exponent inside the multiplication; its rounding (half an ulp, at most 8
 * in that domain) cancels between a weight and the sum and is taken back out of the lse.  Larger
 * magnitudes (the CPU route subtracts the maximum itself and takes any finite value) are outside what
 * this entry point computes correctly.
 *
 * Two kernels.  Without a workspace, or for fewer than 64 rows, a thread-block cluster keeps each
 * row in registers / shared memory (rows too wide for that return NOT_SUPPORTED).  With a
 * workspace of hyle_b200_logits_workspace_bytes(rows, cols) bytes (16-byte aligned, zero-filled
 * once after allocation; each launch leaves it re-armed; stream-ordered launches only) and an
 * output tensor, batches of 64 rows or more take a two-pass streaming kernel whose second pass
 * reads the row back from L2: HBM traffic is the same, throughput is higher.
 *
 * status_word (device memory, may be NULL): the streaming kernel ORs
 * HYLE_B200_STATUS_STREAM_WAIT_TIMEOUT into it when a row could not be completed (its outputs are NaN).
 * That needs a lost store or a bulk copy that never lands: a second-pass task whose first-pass
 * partials are missing reduces the missing chunks itself instead of waiting for another CTA, so the
 * kernel completes with right results however many of its CTAs are resident at once.
 */
HYLE_B200_API uint64_t hyle_b200_logits_workspace_bytes(uint64_t rows, uint64_t cols);
HYLE_B200_API int hyle_b200_logits_reduce_f32(hyle_b200_stream_t stream, const float *logits,
                                              uint64_t rows, uint64_t cols, float *lse,
                                              void *probs_bf16, int32_t *argmax_index,
                                              float *argmax_value, void *workspace,
                                              uint64_t workspace_bytes, uint32_t *status_word);

/* Schedule of the streaming kernel.  Zero fields of a tuning mean "choose"; the defaults are the
 * measured best for the shape.  For tuning sweeps and for tests that force the rare paths (a window
 * of one row with help_after_polls = 1 makes second-pass tasks reduce their own partials). */
typedef struct hyle_b200_stream_tuning {
  int32_t chunk_vectors;      /* float4 per thread and task: 10 (10240-value chunks), the one size built */
  uint32_t window_rows;       /* rows between a row's first and second pass */
  uint32_t help_after_polls;  /* polls before a waiting warp reduces a missing chunk itself */
  int32_t ctas_per_sm;        /* at most what the kernel was built for (4) and what fits */
} hyle_b200_stream_tuning;
typedef struct hyle_b200_stream_plan {
  int32_t chunk_vectors;
  uint32_t chunks_per_row;
  uint32_t chunk_values;
  uint32_t window_rows;
  uint32_t fixed_tasks_per_cta;  /* tasks taken by CTA position; always inside the first-pass head */
  int32_t ctas_per_sm;
  uint32_t grid;
  uint32_t help_after_polls;
} hyle_b200_stream_plan;
/* hyle_b200_logits_reduce_f32 with an explicit schedule; INVALID_VALUE when the shape does not take
 * the streaming kernel (no workspace, fewer than 64 rows, unaligned) or the tuning is inconsistent. */
HYLE_B200_API int hyle_b200_logits_reduce_f32_tuned(hyle_b200_stream_t stream, const float *logits,
                                                    uint64_t rows, uint64_t cols, float *lse,
                                                    void *probs_bf16, int32_t *argmax_index,
                                                    float *argmax_value, void *workspace,
                                                    uint64_t workspace_bytes, uint32_t *status_word,
                                                    const hyle_b200_stream_tuning *tuning);
/* Host-side only: the schedule the streaming kernel would use (NOT_SUPPORTED when the shape is not
 * eligible), and the (pass, row, chunk) at a position of its ordered task list (pass 0 = first,
 * 1 = second, 2 = past the end). */
HYLE_B200_API int hyle_b200_logits_stream_plan(uint64_t rows, uint64_t cols,
                                               const hyle_b200_stream_tuning *tuning,
                                               hyle_b200_stream_plan *plan_out);
HYLE_B200_API int hyle_b200_logits_stream_task(uint64_t rows, uint32_t chunks, uint32_t window,
                                               uint64_t task, uint32_t *pass_out, uint64_t *row_out,
                                               uint32_t *chunk_out);

/* Softmax{axis=-1, kind} with f32 output (output dtype = input dtype,
 * src/compute_ops/operation.cc:1619). out may alias in (the cluster kernel is used then).
 * workspace and status_word: as for hyle_b200_logits_reduce_f32, may be NULL. */
HYLE_B200_API int hyle_b200_softmax_f32(hyle_b200_stream_t stream, int kind, const float *in,
                                        float *out, uint64_t rows, uint64_t cols, void *workspace,
                                        uint64_t workspace_bytes, uint32_t *status_word);

/* Stream-ordered clear of a workspace (cudaMemsetAsync): what a caller that receives workspace
 * memory with arbitrary contents records once before the first launch that uses it. */
HYLE_B200_API int hyle_b200_workspace_clear(hyle_b200_stream_t stream, void *workspace, uint64_t bytes);

/* Cast{destination type} (include/hyle/compute/operation.h:289-295) for the pairs of the CPU route
 * (src/compute_provider_native/cast.cc:128-176): f32/bf16/f16 among themselves, i32 -> f32,
 * f32/bf16/f16 <-> bool, f32/bf16/f16 <-> E4M3, E5M2 -> bf16, E5M2 -> E4M3.  Bit-exact:
 * round to nearest even; the 8-bit formats saturate finite overflow to their largest normal
 * (include/hyle/simd/dtype.h:163-213); bool is "magnitude bits non-zero" (cast.cc:78-91).
 * Other pairs return NOT_SUPPORTED. */
HYLE_B200_API int hyle_b200_cast(hyle_b200_stream_t stream, int source_dtype, int destination_dtype,
                                 const void *in, void *out, uint64_t count);

/* Cast -- or a plain copy when the two types are equal -- FROM A STRIDED VIEW into a dense row-major
 * tensor: `in` addresses element (0, ..., 0); element (i0, ..., ik) lies byte_strides[0]*i0 + ... bytes
 * from it (rank <= 8; strides are multiples of the element size and may be zero (broadcast) or
 * negative).  This is how the reference's tensor kernels read every operand
 * (src/compute_provider_cuda/tensor_kernel.cu:70-108); here a non-dense operand is made dense (and
 * cast) in one pass and then feeds any other entry point.  Pairs: those of hyle_b200_cast plus every
 * type onto itself (bits are moved).  A view that is in fact dense takes the dense kernels. */
HYLE_B200_API int hyle_b200_strided_cast(hyle_b200_stream_t stream, int source_dtype,
                                         int destination_dtype, const void *in, void *out,
                                         uint32_t rank, const int64_t *dims,
                                         const int64_t *byte_strides);

/* The mirror for outputs: a dense row-major tensor `in` is placed INTO A STRIDED VIEW `out` of the same
 * element type (bits are moved): element (i0, ..., ik) goes byte_strides[0]*i0 + ... bytes from `out`
 * (rank <= 8; strides are multiples of the element size and may be negative, but not zero on an axis
 * longer than one: two elements would share an address).  The reference's tensor kernels write every
 * output through its byte strides (src/compute_provider_cuda/tensor_kernel.cu:70-108); here an operator
 * writes its dense result and this entry places it, e.g. into a slice of a larger tensor.  Bytes of the
 * destination outside the view are not touched.  The public custom-kernel seam never needs it: for exact
 * shapes the reference's prepare admits only the inferred, dense output description
 * (src/compute/operation.cc:265-296); it serves callers of the C ABI that own a strided destination
 * (a provider bound through the reference's private seam, whose bounded shape domains skip that check).  dtype: any storage type of hyle_b200_cast (only its
 * width matters).  Contiguous innermost runs move 16 bytes per thread when everything is 16-byte
 * aligned; a destination that is dense in a permuted axis order (a transposed layout without gaps) takes
 * the tiled transposition of hyle_b200_strided_cast seen from the destination's side; any other
 * destination whose innermost axis is strided is written element by element. */
HYLE_B200_API int hyle_b200_strided_scatter(hyle_b200_stream_t stream, int dtype, const void *in, void *out,
                                            uint32_t rank, const int64_t *dimensions,
                                            const int64_t *byte_strides);

/* Select (include/hyle/compute/operation.h:305, inference src/compute_ops/operation.cc:1309-1328):
 * out[i] = condition[i] != 0 ? when_true[i % true_period] : when_false[i % false_period]; elements
 * are moved as bits (NaN payloads included).  condition is one byte per element, any non-zero value is
 * true (include/hyle/simd/ops.h:80).  dtype F32 / I32 (4-byte) or BF16 / F16 (2-byte) elements; a
 * period equals count (same shape) or divides it (trailing-axes broadcast; 1 = one scalar). */
HYLE_B200_API int hyle_b200_select(hyle_b200_stream_t stream, int dtype, const void *condition,
                                   const void *when_true, const void *when_false, void *out,
                                   uint64_t count, uint64_t true_period, uint64_t false_period);

/* Scan{axis=-1, exclusive} (include/hyle/compute/operation.h:314-321; CPU route
 * src/compute_provider_ggml/standard_index.cc:113-157): prefix sums along the rows of a dense
 * [rows, cols] tensor, inclusive, or exclusive from zero.  dtype F32: float accumulation in a blocked
 * order (the operator permits reassociation).  dtype I32: exact, int64 accumulation; if any inclusive
 * prefix of any row (the row total included, also for an exclusive scan) does not fit int32,
 * HYLE_B200_STATUS_SCAN_OVERFLOW is set in *status_word and NOTHING is written to out, which takes a
 * checking pass before the writing pass; status_word is required for I32 and must not already carry
 * that bit.  out must not alias in. */
HYLE_B200_API int hyle_b200_scan(hyle_b200_stream_t stream, int dtype, const void *in, void *out,
                                 uint64_t rows, uint64_t cols, int exclusive, uint32_t *status_word);

/* Softmax{axis=-1, kSoftmax, scale, mask=kBoolean} on f16 rows, f32 accumulation: the masked, scaled
 * form of the CPU route (src/compute_provider_native/transformer.cc:44-57,228-275):
 *   v = f32(in) * scale;  v = -inf where the mask byte is 0;  out = f16_rne(softmax(v)).
 * mask: one byte per element, mask_count elements repeating over the leading axes (mask_count is a
 * multiple of cols and divides rows * cols; rows * cols = the tensor's own shape).  A row with NaN
 * or +inf, or with every element masked, is all NaN.  Results within one f16 step of the CPU route. */
HYLE_B200_API int hyle_b200_masked_softmax_f16(hyle_b200_stream_t stream, const void *in,
                                               const unsigned char *mask, uint64_t mask_count,
                                               float scale, void *out, uint64_t rows,
                                               uint64_t cols);

/* Softmax{axis=-1, kSoftmax, scale, mask=kAdditive} on f16 rows (include/hyle/compute/operation.h:122-126;
 * the reference forms the value in src/compute_provider_cuda/reduction_kernel.cu:131-146):
 *   v = f32(in) * scale + f32(mask);  out = f16_rne(softmax(v)),  f32 accumulation.
 * mask_f16: f16 addends (0 keeps, -inf masks, anything finite biases), mask_count of them repeating
 * over the leading axes under the rules of hyle_b200_masked_softmax_f16, whose treatment of NaN,
 * +inf and fully masked rows applies.  Product and sum are rounded to f32 separately (the ATen CPU
 * provider's order, src/compute_provider_native/aten_cpu_provider.cc:500-505, but without its f16
 * rounding of the product); the native CPU route is NOT followed here: it tests the first byte of
 * each addend as if it were a Boolean (src/compute_provider_native/transformer.cc:44-57).  Results
 * within one f16 step of the f32 composition above. */
HYLE_B200_API int hyle_b200_additive_masked_softmax_f16(hyle_b200_stream_t stream, const void *in,
                                                        const void *mask_f16, uint64_t mask_count,
                                                        float scale, void *out, uint64_t rows,
                                                        uint64_t cols);

/* Cast{f32 -> bf16}, round to nearest even (include/hyle/simd/dtype.h:114-121). */
HYLE_B200_API int hyle_b200_cast_f32_to_bf16(hyle_b200_stream_t stream, const float *in,
                                             void *out_bf16, uint64_t count);

/* Verification hook, no counterpart in the reference: the encoder forms a block's scale amax / 127
 * and its reciprocal without the division sequence (a multiplication by RN(1/127) with one fused
 * correction step; the IEEE reciprocal instruction).  This call compares both, bit for bit, with the
 * correctly rounded divisions for EVERY magnitude the encoder accepts (2^31-odd bit patterns, a few
 * milliseconds) and stores the number of disagreements, which must be 0, in *mismatches (device
 * memory, 8 bytes). */
HYLE_B200_API int hyle_b200_selfcheck_q8_0_scale(hyle_b200_stream_t stream,
                                                 unsigned long long *mismatches);

/* ---------------------------------------------------------------------------------------------
 * Q8_0: blocks of 32 values -> 34 bytes {f16 scale (little endian), 32 x int8}
 * (src/compute_ops/low_precision.cc:28-29).
 *
 * Encode replaces model_ops::CacheEncode{CacheStorage::q8_0()} (include/hyle/compute/model_ops.h:207-229),
 * executor src/compute_provider_ggml/ggml_cpu_provider.cc:585-615:
 *   d = amax/127.0f; id = 1.0f/d; q = roundf(x*id) (half away from zero); scale = f16_rne(d);
 *   a block whose f16 scale is zero, or that holds an invalid value, is 34 zero bytes; invalid
 *   values also set HYLE_B200_STATUS_INVALID_Q8_INPUT in *status_word (may be NULL).
 * count must be a multiple of 32.  dtype is the input storage type.
 */
HYLE_B200_API int hyle_b200_q8_0_encode(hyle_b200_stream_t stream, int dtype, const void *in,
                                        uint64_t count, void *blocks_out,
                                        uint32_t *status_word);

/* Decode: out = bf16_rne(f32(f16 scale) * q).  The reference has no standalone operator; the
 * layout and arithmetic are those of the kGgufQ8_0 blocked tensors its MatMul/Gather consume
 * (src/compute_ops/low_precision.cc:269-297). */
HYLE_B200_API int hyle_b200_q8_0_decode_bf16(hyle_b200_stream_t stream, const void *blocks,
                                             uint64_t count, void *out_bf16);

/* model_ops::CacheEncode{CacheStorage::float8(scale)} (include/hyle/compute/model_ops.h:207-229,
 * include/hyle/compute/low_precision.h:94), executor src/compute_provider_ggml/ggml_cpu_provider.cc:589-596:
 *   out[i] = e4m3_satfinite_rne(in[i] / scale), one byte per value; a non-finite input writes 0 and
 *   sets HYLE_B200_STATUS_INVALID_FP8_INPUT in *status_word (may be NULL).
 * dtype = F32 / BF16 / F16 of the input; scale finite and positive. */
HYLE_B200_API int hyle_b200_fp8_e4m3_encode(hyle_b200_stream_t stream, int dtype, const void *in,
                                            uint64_t count, float scale, void *out,
                                            uint32_t *status_word);

/* Paged append: the row mover behind the paged KV cache's append / copy step, the consumer of the
 * rows CacheEncode wrote (launch_paged_append, src/compute_backend_cuda/cuda_paged_append.cu:66-81;
 * wire structs include/hyle/compute/detail/paged_append_wire.h:11-34).  All in device memory:
 *   metadata = {u32 active_count, 0, 0, 0} followed by instruction_capacity instructions of
 *              {u32 source_kind, source_page, source_row, destination_page, destination_row, rows, 0, 0};
 *   source_kind 0 copies `rows` rows from row source_row of input_rows_data (input_rows packed rows),
 *   source_kind 1 from (source_page, source_row) of the arena itself; the destination is row
 *   destination_page * page_rows + destination_row of the arena (physical_pages * page_rows rows).
 * Rows are row_bytes bytes (even), moved bit for bit.  As in the reference kernel
 * (cuda_paged_append.cu:16-45) an episode with active_count > instruction_capacity or non-zero
 * reserved words does nothing, and an instruction with non-zero reserved words, rows == 0, another
 * source kind, or a coordinate outside the arena or the input is skipped.  Instructions of one episode
 * must not write a range another of them reads or writes.  The launch shape depends on the capacities
 * only, so the call can be captured in a CUDA graph and replayed with new metadata contents. */
HYLE_B200_API int hyle_b200_paged_append(hyle_b200_stream_t stream, void *arena,
                                         const void *input_rows_data, const void *metadata,
                                         uint32_t page_rows, uint32_t physical_pages,
                                         uint32_t input_rows, uint32_t instruction_capacity,
                                         uint64_t row_bytes);

/* Paged append with device-resident lengths (launch_device_lengths_paged_append,
 * src/compute_backend_cuda/cuda_paged_append.cu:82-154; records
 * include/hyle/compute/detail/device_lengths_paged_append_wire.h:8-24).  After the 16-byte header
 * {active_count, 0, 0, 0} the metadata holds 32-byte records: a directory {requests, pages, 0 x 6},
 * `requests` bounds {query_rows, minimum_previous_rows, maximum_previous_rows, maximum_kv_rows, 0 x 4}
 * and `pages` dirty pages {request, logical_page, destination_page, initialized_rows, source_page,
 * source_rows, 0 x 2}.  With q = query_lengths[r], kv = kv_lengths[r] (i32, device memory), request r
 * had kv - q rows before and owns the packed new rows [sum of earlier q, + q).  Of a page's
 * initialized rows, those below kv - q are copied from the beginning of source_page (copy on write),
 * those below kv come from the request's new rows, the rest are zeroed.
 * *status_word follows the reference's device status protocol (written only by compare-and-swap from
 * 0): when it is not 0 on entry nothing is done; an episode whose header, directory, bounds or
 * lengths are inconsistent does nothing and reports 4 (invalid sequence offsets); a bad page record
 * is skipped and reports 1 (index out of range) -- which of the OTHER pages are then written is
 * unspecified, here as in the reference.  requests 1..32, input_rows <= INT32_MAX and
 * instruction_capacity >= requests + 2, otherwise NOT_SUPPORTED (cuda_paged_append.cc:110-115). */
HYLE_B200_API int hyle_b200_paged_append_device_lengths(
    hyle_b200_stream_t stream, void *arena, const void *input_rows_data, const void *metadata,
    const int32_t *query_lengths, const int32_t *kv_lengths, uint32_t page_rows,
    uint32_t physical_pages, uint32_t input_rows, uint32_t instruction_capacity, uint64_t row_bytes,
    uint32_t requests, uint32_t *status_word);

/* Scratch for the two kernels below, for a tensor of `count` values: a header (ticket and tile
 * counters), per-CTA partial sums, and for the fused round trip one f64 per tile of 8192 values
 * (count/1024 bytes + 33 KB).  The caller zero-fills it once after
 * allocation; each launch leaves every counter zeroed again, so one workspace serves any number of
 * stream-ordered launches (not concurrent ones), also for smaller counts. */
HYLE_B200_API uint64_t hyle_b200_sum_squares_workspace_bytes(uint64_t count);

/* Reduce{kSum, Axes::all()} of Cast(bf16->f32)^2 (include/hyle/compute/operation.h:232-248):
 * deterministic two-pass sum (fixed per-thread order, fixed-order merge of CTA partials in f64).
 * *sum_out is a device double; its float value is the operator result. */
HYLE_B200_API int hyle_b200_sum_squares_bf16(hyle_b200_stream_t stream, const void *in,
                                             uint64_t count, double *sum_out, void *workspace,
                                             uint64_t workspace_bytes);

/* One pass over a bf16 tensor producing its Q8_0 blocks, the decoded bf16 tensor and the sum of
 * squares of the input: the input is read once (5.0625 bytes of traffic per element).  Tiles are
 * handed to the CTAs dynamically; the sum is built from per-tile sums added in index order, so it is
 * bit-identical from run to run. */
HYLE_B200_API int hyle_b200_q8_0_roundtrip_bf16(hyle_b200_stream_t stream, const void *in,
                                                uint64_t count, void *blocks_out,
                                                void *decoded_bf16, double *sum_squares_out,
                                                uint32_t *status_word, void *workspace,
                                                uint64_t workspace_bytes);

/* ---------------------------------------------------------------------------------------------
 * The same round trip for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its providers always receive caller-owned workspace.)
 *
 * Who needs it: code embedded in a host that owns all device memory through its own pool, a
 * provider whose enqueue path may not allocate and was given no workspace, or a process whose
 * memory budget is fixed at start-up.  Instead of a caller-supplied workspace the kernel's scratch
 * (per-CTA partial sums and a ticket counter, 8256 bytes) is a fixed array inside the library image;
 * every GPU that loads the library holds it until the process exits.  The call performs no
 * cudaMalloc/cudaFree and uses no allocating library routine.
 *
 * Limits and rules:
 *  - at most HYLE_B200_STATIC_MAX_VALUES values per call; more returns
 *    HYLE_B200_STATIC_SCRATCH_EXCEEDED and launches nothing;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *    with that device current); make that first call outside any stream capture;
 *  - all calls on a device share the array: calls that can overlap on the GPU (different
 *    streams without ordering) race on it; stream-ordered calls are safe, each one clears the
 *    counter on its stream before launching.
 *  - the address is cached per device ordinal for the device's PRIMARY context (the one the CUDA
 *    runtime uses); a second driver context on the same device has its own copy of the array and
 *    must not share this cache;
 *  - blocks and decoded values are bit-identical to hyle_b200_q8_0_roundtrip_bf16's.  The sum of
 *    squares is deterministic for one device and launch grid (two calls on the same data return
 *    the same bits) but is added in a different order (per-CTA partials, grid = min(1024,
 *    6 x SMs)), so it agrees with the workspace entry to about 1e-12 relative, not bit for bit.
 * Inputs, outputs and error codes are otherwise those of hyle_b200_q8_0_roundtrip_bf16.
 */
#define HYLE_B200_STATIC_MAX_VALUES (UINT64_C(1) << 31)
HYLE_B200_API int hyle_b200_q8_0_roundtrip_bf16_static(hyle_b200_stream_t stream, const void *in,
                                                       uint64_t count, void *blocks_out,
                                                       void *decoded_bf16, double *sum_squares_out,
                                                       uint32_t *status_word);

/* ---------------------------------------------------------------------------------------------
 * File -> pinned host memory -> device, in chunks, for weight banks that live on disk.
 * Replaces, for this library's one consumer (the Q8_0 decode kernel): the reference's file resource
 * pipeline, include/hyle/compute/cuda_file_stream.h:10-14 over include/hyle/compute/file_stream.h:23-31
 * (`in_flight_slots` staging slots of `staging_bytes_per_slot`; scheduling in
 * src/compute_stream/file_stream.cc).  On-disk GGUF Q8_0 weights are this library's carrier layout: rows
 * of k/32 blocks of 34 bytes (src/compute_ops/low_precision.cc:269-297).
 *
 * open() allocates everything: `slots` pinned staging buffers and `slots` device buffers of
 * chunk_bytes, 2 x slots events, one copy stream, the reader threads; nothing allocates afterwards.
 * Chunk i is read into pinned slot i % slots by `readers` threads at once (a MiB per pread call: one
 * thread copies from the page cache at about a fifth of the host-to-device link), then ONE
 * cudaMemcpyAsync for it is issued on the copy stream.  next() makes the consumer's stream wait (on the device) for that copy and returns
 * the chunk's device address; the address stays valid until the NEXT call of next(), which records on
 * the consumer's stream that the chunk is finished with, so that the copy stream may overwrite its
 * slot.  Chunks arrive in file order; at the end next() returns OK with *chunk_bytes == 0.  A read
 * error or a file shorter than the range makes next() return HYLE_B200_IO_ERROR.  One consumer thread
 * per stream object.  close() waits for the consumer's last recorded use, then frees.
 *
 * A stream opened with bytes == 0 has no sequential reader and no device slots; it serves
 * read_group(): a group of byte ranges of the file, each copied to a device destination of the
 * caller's own (the reference's StreamReadGroup of StreamReadRange{file_offset, destination, bytes},
 * include/hyle/compute/file_stream.h:84-93: how tensors of a weight file reach their buffers).
 * The calling thread reads each range in chunks into the pinned slots, one cudaMemcpyAsync per
 * chunk on the copy stream, reading the next chunk while the previous copy is in flight; on return
 * the consumer's stream has been made to wait for the group's last copy.  Ranges are checked
 * against the file's size before anything is copied (HYLE_B200_IO_ERROR); destinations need no
 * alignment.
 */
typedef struct hyle_b200_file_stream hyle_b200_file_stream;
typedef struct hyle_b200_file_stream_options {
  uint64_t chunk_bytes;    /* 0: 8 MiB */
  uint32_t slots;          /* in-flight chunks, 2..16; 0: 4 */
  uint32_t readers;        /* threads that read one chunk together, 1..16; 0: half the hardware threads, at most 8 */
  uint64_t chunk_granule;  /* chunk_bytes is rounded down to a multiple of this (a record size); 0: 1 */
} hyle_b200_file_stream_options;
typedef struct hyle_b200_file_stream_report {
  uint64_t bytes_read, bytes_copied;  /* so far */
  uint64_t io_calls, copies;          /* pread calls; cudaMemcpyAsync calls (one per chunk) */
  uint64_t staging_bytes, device_bytes, chunk_bytes, chunks;
} hyle_b200_file_stream_report;
HYLE_B200_API int hyle_b200_file_stream_open(const char *path, uint64_t file_offset, uint64_t bytes,
                                             const hyle_b200_file_stream_options *options,
                                             hyle_b200_file_stream **stream_out);
HYLE_B200_API int hyle_b200_file_stream_next(hyle_b200_file_stream *stream, hyle_b200_stream_t consumer,
                                             const void **device_chunk, uint64_t *chunk_bytes,
                                             uint64_t *chunk_offset);
typedef struct hyle_b200_file_range {
  uint64_t file_offset;  /* from the start of the file */
  uint64_t bytes;
  void *destination;     /* device memory */
} hyle_b200_file_range;
HYLE_B200_API int hyle_b200_file_stream_read_group(hyle_b200_file_stream *stream,
                                                   hyle_b200_stream_t consumer,
                                                   const hyle_b200_file_range *ranges, uint32_t count);
HYLE_B200_API int hyle_b200_file_stream_get_report(hyle_b200_file_stream *stream,
                                                   hyle_b200_file_stream_report *report);
HYLE_B200_API int hyle_b200_file_stream_close(hyle_b200_file_stream *stream);
/* The Q8_0 bank of `count` values stored at `file_offset` of `path`, decoded into the device tensor
 * out_bf16 by hyle_b200_q8_0_decode_bf16, one launch per chunk on `consumer`, while later chunks are
 * read and copied.  Returns when every launch is enqueued and the pipeline has been torn down. */
HYLE_B200_API int hyle_b200_q8_0_decode_file_bf16(hyle_b200_stream_t consumer, const char *path,
                                                  uint64_t file_offset, uint64_t count, void *out_bf16,
                                                  const hyle_b200_file_stream_options *options,
                                                  hyle_b200_file_stream_report *report);

/* ---------------------------------------------------------------------------------------------
 * The round trip on a row-sharded tensor, with the cross-GPU sum fused into the kernel.
 *
 * Each of `world` GPUs (one process or thread per GPU) calls this on its own shard, all with the
 * same `epoch`.  The kernel is hyle_b200_q8_0_roundtrip_bf16; where that one stores the shard's
 * sum of squares, this one's finishing CTA writes it into every rank's MAILBOX (peer-mapped
 * device memory, plain 8-byte stores over NVLink), waits for the other ranks' sums in its own
 * mailbox and stores the sum over all ranks, added in rank order: every rank gets the same bits.
 * It replaces kernel + ncclAllReduce(8 bytes) + the launch gaps around it by one kernel.
 * (The reference has no multi-GPU form of this path; the partition is the one its Q8_0 block
 * layout allows: 32-value blocks never cross a row, src/compute_provider_ggml/ggml_cpu_provider.cc:596-608.)
 *
 *  mailboxes   host array of `world` device pointers; mailboxes[r] is rank r's mailbox as THIS GPU
 *              addresses it (for r == rank the local pointer).  A mailbox is
 *              HYLE_B200_EXCHANGE_MAILBOX_BYTES of device memory, zero-filled once at creation,
 *              8-byte aligned, used by no one else.  Between processes, map it with the CUDA IPC
 *              calls (hyle_b200_exchange_* below); within one process, enable peer access and pass
 *              the pointers as they are.
 *  world       2..HYLE_B200_EXCHANGE_MAX_RANKS (1 is accepted and exchanges nothing)
 *  epoch       non-zero, the same on every rank for one collective call, different from the
 *              previous call's by an odd amount (count calls: 1, 2, 3, ...)
 *  poll_limit  polls (about 0.1 us apart at least) before a rank gives up on a peer; then its
 *              *sum_squares_out is NaN and HYLE_B200_STATUS_EXCHANGE_TIMEOUT is set in *status_word.
 *              The kernel never waits longer than that: no rank can hang a GPU.  0 selects the
 *              default of about ten seconds.
 * All ranks must be running the call at the same time on DIFFERENT GPUs (kernels that wait for
 * each other must not share a GPU).  Everything else is as for hyle_b200_q8_0_roundtrip_bf16.
 */
#define HYLE_B200_EXCHANGE_MAX_RANKS 8
#define HYLE_B200_EXCHANGE_MAILBOX_BYTES 256
#define HYLE_B200_EXCHANGE_HANDLE_BYTES 64
HYLE_B200_API int hyle_b200_q8_0_roundtrip_bf16_exchange(
    hyle_b200_stream_t stream, const void *in, uint64_t count, void *blocks_out, void *decoded_bf16,
    double *sum_squares_out, uint32_t *status_word, void *workspace, uint64_t workspace_bytes,
    void *const *mailboxes, uint32_t world, uint32_t rank, uint32_t epoch, uint32_t poll_limit);

/* Mailbox plumbing for one process per GPU, on the current device: create allocates and clears a
 * mailbox and writes the HYLE_B200_EXCHANGE_HANDLE_BYTES handle another process opens (thin
 * wrappers over cudaMalloc / cudaIpcGetMemHandle / cudaIpcOpenMemHandle / cudaIpcCloseMemHandle /
 * cudaFree; these four calls allocate or map memory and belong in set-up code, not in a step). */
HYLE_B200_API int hyle_b200_exchange_create(void **mailbox, unsigned char *handle_out);
HYLE_B200_API int hyle_b200_exchange_open(const unsigned char *handle, void **peer_mailbox);
HYLE_B200_API int hyle_b200_exchange_close(void *peer_mailbox);
HYLE_B200_API int hyle_b200_exchange_destroy(void *mailbox);

/* ---------------------------------------------------------------------------------------------
 * sampling_ops::RandomBits{word_count} (include/hyle/compute/sampling_ops.h:21-34), CPU route
 * src/compute_provider_native/sampling.cc:76-88: out[r, w] = lane w % 4 of Philox-4x32-10 with key
 * identities[r, 0..1] and counter (w / 4, identities[r, 2], identities[r, 3]).  identities is
 * u32[rows, 4], out u32[rows, word_count].  Bit-exact on every backend.
 */
HYLE_B200_API int hyle_b200_random_bits(hyle_b200_stream_t stream, const uint32_t *identities,
                                        uint64_t rows, uint32_t word_count, uint32_t *out);

/* sampling_ops::Categorical{return_log_probability} (include/hyle/compute/sampling_ops.h:36-68),
 * CPU route src/compute_provider_native/sampling.cc:112-181: one index per row of f32 / bf16 / f16
 * log-weights [rows, cols], drawn by inverting the cumulative weights exp(x - max) at
 * u = ((x0 * 2^20 + (x1 >> 12)) + 0.5) * 2^-52 with (x0, x1) from block 0 of the row's identity;
 * -inf has zero mass; log_probability_out (may be NULL) = x[index] - max - log(total).
 * The operator leaves the floating math to each backend (indices of borderline draws need not match
 * another backend's); a row's result here depends only on that row and its identity.
 * A row with NaN, +inf or no finite value gets index -1, NaN log-probability and
 * HYLE_B200_STATUS_INVALID_CATEGORICAL_ROW in *status_word (may be NULL); the adapter turns that into
 * the InvalidArgument completion the CPU route reports.
 */
HYLE_B200_API int hyle_b200_categorical(hyle_b200_stream_t stream, int dtype, const void *log_weights,
                                        const uint32_t *identities, uint64_t rows, uint64_t cols,
                                        int32_t *index_out, float *log_probability_out,
                                        uint32_t *status_word);

#ifdef __cplusplus
}
#endif
#endif /* HYLE_B200_H_ */

// Drives the adapter's cold path (propose / prepare / decline) through the REFERENCE's own
// runtime: Context::create -> compute::prepare -> provider search, on the reference's CPU backend.
// A probe backend stands in for the CUDA one (which needs CUDA >= 13.3): it serves the CPU backend
// id and host memory, and refuses to hand out a stream, so nothing is ever launched -- this program
// checks WHICH requests the provider takes and how it declines, not arithmetic.
//
// Built by tests/provider/Makefile against the reference tree in place; prints one line per
// check and exits non-zero on the first failure.
#include <array>
#include <cstdio>
#include <cstdlib>

#include <hyle/compute/backends/cpu.h>
#include <hyle/compute/device.h>
#include <hyle/compute/prepared_operation.h>
#include <hyle/mem/buffer.h>
#include <hyle/mem/resource.h>

#include <hyle/compute/sampling_ops.h>

#include "b200_paged_append.h"
#include "b200_provider.h"

using namespace hyle::compute;
using hyle::Result;
using hyle::Status;

struct ProbeBackend final {
  static constexpr BackendId id() noexcept { return cpu::kBackendId; }
  static constexpr hyle::mem::MemoryProperty memory() noexcept { return hyle::mem::MemoryProperty::kHostAccessible; }
  static Result<hyle_b200_stream_t> stream(detail::QueueSequence &) noexcept {
    return std::unexpected(Status::Unimplemented("probe backend: no CUDA stream behind a CPU queue"));
  }
  static Result<const void *> pointer(hyle::mem::ConstBufferView) noexcept {
    return std::unexpected(Status::Unimplemented("probe backend"));
  }
  static Result<void *> mutable_pointer(hyle::mem::BufferView) noexcept {
    return std::unexpected(Status::Unimplemented("probe backend"));
  }
  static Status status(int) noexcept { return Status::Internal("probe backend never launches"); }
  static detail::EnqueueResult status_word(detail::QueueSequence &, unsigned **) noexcept {
    return detail::EnqueueResult::rejected(Status::Unimplemented("probe backend"));
  }
};

// The same stand-in under another backend id: a provider made for it must not enter a CPU Context.
struct ForeignBackend final {
  static constexpr BackendId id() noexcept { return BackendId{0x6879'6c65'6232'3030ULL, 0x7e57ULL}; }
  static constexpr hyle::mem::MemoryProperty memory() noexcept { return ProbeBackend::memory(); }
  static Result<hyle_b200_stream_t> stream(detail::QueueSequence &s) noexcept { return ProbeBackend::stream(s); }
  static Result<const void *> pointer(hyle::mem::ConstBufferView v) noexcept { return ProbeBackend::pointer(v); }
  static Result<void *> mutable_pointer(hyle::mem::BufferView v) noexcept { return ProbeBackend::mutable_pointer(v); }
  static Status status(int code) noexcept { return ProbeBackend::status(code); }
  static detail::EnqueueResult status_word(detail::QueueSequence &s, unsigned **word) noexcept {
    return ProbeBackend::status_word(s, word);
  }
};

static int failures = 0;
static void check(bool ok, const char *what) {
  std::printf("%s  %s\n", ok ? "ok  " : "FAIL", what);
  if (!ok) ++failures;
}

template <std::size_t N>
static TensorDesc dense(DataType type, const std::int64_t (&dims)[N]) {
  return TensorDesc::dense(type, std::span<const std::int64_t>(dims, N)).value();
}

// prepare() through the reference runtime with explicit input/output descriptions.
static bool taken(const Context &context, const Operation &op, std::span<const TensorDesc> in,
                  std::span<const TensorDesc> out) {
  auto prepared = prepare(context, op, in, out, hyle::mem::system_resource());
  return prepared.has_value() && prepared->provider().id == b200::kIdentity.id;
}
static bool declined(const Context &context, const Operation &op, std::span<const TensorDesc> in,
                     std::span<const TensorDesc> out) {
  auto prepared = prepare(context, op, in, out, hyle::mem::system_resource());
  return !prepared.has_value() && prepared.error().IsUnimplemented();
}

int main() {
  auto provider = b200::make_provider<ProbeBackend>();
  check(provider.has_value(), "make_custom_provider accepts the factory");
  if (!provider) return 1;
  auto context = Context::create(cpu::device(), std::move(*provider));
  check(context.has_value(), "Context::create with the b200 provider as the only provider");
  if (!context) return 1;

  {  // backend mismatch is Unimplemented at Context creation (src/compute/custom_kernel.cc:64-67)
    auto foreign = b200::make_provider<ForeignBackend>();
    bool refused = foreign.has_value();
    if (refused) {
      auto wrong = Context::create(cpu::device(), std::move(*foreign));
      refused = !wrong.has_value() && wrong.error().IsUnimplemented();
    }
    check(refused, "a provider made for another backend id is refused by a CPU Context: Unimplemented");
  }

  const auto f32_mat = dense(DataType::kFloat32, {64, 4096});
  const auto f32_row = dense(DataType::kFloat32, {4096});
  const auto f32_rows = dense(DataType::kFloat32, {64});
  const auto bf16_mat = dense(DataType::kBFloat16, {64, 2048});
  const auto bf16_w = dense(DataType::kBFloat16, {2048});
  const auto f32_w = dense(DataType::kFloat32, {2048});
  const auto f16_w = dense(DataType::kFloat16, {2048});

  {  // Binary: all six kinds with trailing-axis broadcast are taken, other broadcasts are declined
    const std::array in{f32_mat, f32_row};
    const std::array out{f32_mat};
    check(taken(*context, Operation(Binary{BinaryKind::kAdd}), in, out), "Binary{kAdd} f32 [64,4096] + [4096]");
    check(taken(*context, Operation(Binary{BinaryKind::kMultiply}), in, out), "Binary{kMultiply} f32 broadcast");
    check(taken(*context, Operation(Binary{BinaryKind::kSubtract}), in, out), "Binary{kSubtract} f32 broadcast");
    check(taken(*context, Operation(Binary{BinaryKind::kMinimum}), in, out), "Binary{kMinimum} f32 broadcast");
    const std::array same{bf16_mat, bf16_mat};
    const std::array out16{bf16_mat};
    check(taken(*context, Operation(Binary{BinaryKind::kAdd}), same, out16), "Binary{kAdd} bf16 same shape (residual add)");
  }
  {  // Unary: every kind on the three floating storage types
    const std::array in{f32_mat};
    const std::array out{f32_mat};
    check(taken(*context, Operation(Unary{UnaryKind::kTanh}), in, out), "Unary{kTanh} f32");
    check(taken(*context, Operation(Unary{UnaryKind::kSoftplus}), in, out), "Unary{kSoftplus} f32");
    const std::array in16{bf16_mat};
    const std::array out16{bf16_mat};
    check(taken(*context, Operation(Unary{UnaryKind::kGelu}), in16, out16), "Unary{kGelu} bf16");
  }
  {  // Select: Bool condition, branches of the full shape or of the trailing axes
    const auto mask = dense(DataType::kBool, {64, 4096});
    const std::array in{mask, f32_mat, f32_row};
    const std::array out{f32_mat};
    check(taken(*context, Operation(Select{}), in, out), "Select{} f32, when_false broadcast over rows");
  }
  {  // Reduce over the last axis
    const std::array in{f32_mat};
    const std::array out{f32_rows};
    const std::array<std::int32_t, 1> last{-1};
    Reduce reduce{.kind = ReductionKind::kMaximum, .axes = Axes::from(last).value()};
    check(taken(*context, Operation(reduce), in, out), "Reduce{kMaximum, axes={-1}} f32");
    reduce.kind = ReductionKind::kSum;
    check(taken(*context, Operation(reduce), in, out), "Reduce{kSum, axes={-1}} f32");
    const std::array<std::int32_t, 1> first{0};
    reduce.axes = Axes::from(first).value();
    const std::array out0{f32_row};
    check(declined(*context, Operation(reduce), in, out0), "Reduce over axis 0 declined");
  }
  {  // Scan along the last axis, f32 and checked i32; other axes are left to the next provider
    const std::array in{f32_mat};
    const std::array out{f32_mat};
    check(taken(*context, Operation(Scan{.axis = -1, .exclusive = false}), in, out), "Scan{axis=-1} f32");
    check(taken(*context, Operation(Scan{.axis = 1, .exclusive = true}), in, out), "Scan{axis=1 of 2, exclusive} f32");
    check(declined(*context, Operation(Scan{.axis = 0}), in, out), "Scan over axis 0 declined");
    const auto i32_mat = dense(DataType::kInt32, {4096, 4096});
    const std::array in_i{i32_mat};
    const std::array out_i{i32_mat};
    check(taken(*context, Operation(Scan{}), in_i, out_i), "Scan i32 (overflow reported through the status word)");
  }
  {  // strided inputs are gathered first (a workspace is declared); outputs are always dense
    const auto turned = f32_mat.transposed().value();
    const auto upright = dense(DataType::kFloat32, {4096, 64});
    const std::array in{turned};
    const std::array out{upright};
    check(taken(*context, Operation(Unary{UnaryKind::kExp}), in, out), "Unary f32 on a transposed input view");
    const auto plan = b200::match(Operation(Unary{UnaryKind::kExp}), in, out);
    check(plan && plan->gather_count == 1 && plan->workspace_bytes == 0 && plan->total_workspace_bytes == 64 * 4096 * 4,
          "the plan gathers that input into a workspace of its dense size");
    // Binary under the NumPy rule on both sides: a column vector, a scalar-like [1, 1], a row on the left
    const auto column = dense(DataType::kFloat32, {64, 1}), one = dense(DataType::kFloat32, {1, 1});
    const std::array mat_out{f32_mat};
    const std::array with_column{f32_mat, column};
    const std::array with_one{f32_mat, one};
    const std::array row_left{f32_row, f32_mat};
    check(taken(*context, Operation(Binary{BinaryKind::kMultiply}), with_column, mat_out), "Binary f32 [64,4096] * [64,1] (column broadcast)");
    check(taken(*context, Operation(Binary{BinaryKind::kAdd}), with_one, mat_out), "Binary f32 [64,4096] + [1,1]");
    check(taken(*context, Operation(Binary{BinaryKind::kSubtract}), row_left, mat_out), "Binary f32 [4096] - [64,4096] (left operand broadcast)");
    const auto column_plan = b200::match(Operation(Binary{BinaryKind::kMultiply}), with_column, mat_out);
    check(column_plan && column_plan->gather_count == 1 && column_plan->gathers[0].input == 1 &&
              column_plan->gathers[0].byte_strides[0] == 4 && column_plan->gathers[0].byte_strides[1] == 0,
          "the column is gathered through strides {4, 0}");
    const std::array mismatched{f32_mat, dense(DataType::kFloat32, {32, 1})};
    check(!taken(*context, Operation(Binary{BinaryKind::kMultiply}), mismatched, mat_out), "Binary with an extent that cannot broadcast not taken");
    const std::array dense_in{upright};
    const std::array turned_out{turned};
    // Outputs never arrive strided on this seam: for exact shapes the reference's prepare compares the output
    // description, byte strides included, with the inferred dense one (src/compute/operation.cc:265-296).
    auto refused = prepare(*context, Operation(Unary{UnaryKind::kExp}), dense_in, turned_out, hyle::mem::system_resource());
    check(!refused.has_value() && refused.error().IsInvalidArgument(),
          "Unary f32 into a transposed output: refused by the reference's prepare itself (InvalidArgument), before any provider");
  }
  {  // narrow Reduce: the extrema of bf16 / f16 rows in their own type; sums stay with the f32 kernel
    const auto half_rows = dense(DataType::kFloat16, {64, 2048}), half_col = dense(DataType::kFloat16, {64});
    const auto bf_col = dense(DataType::kBFloat16, {64});
    const std::array half_in{half_rows};
    const std::array half_out{half_col};
    const std::array bf_in{bf16_mat};
    const std::array bf_out{bf_col};
    const std::array<std::int32_t, 1> last{-1};
    const auto last_axis = [&](ReductionKind kind) {
      return Operation(Reduce{.kind = kind, .axes = Axes::from(last).value(), .accumulation_type = DataType::kFloat32});
    };
    check(taken(*context, last_axis(ReductionKind::kMinimum), half_in, half_out), "Reduce{kMinimum} f16 rows");
    check(taken(*context, last_axis(ReductionKind::kMaximum), half_in, half_out), "Reduce{kMaximum} f16 rows");
    check(taken(*context, last_axis(ReductionKind::kMaximum), bf_in, bf_out), "Reduce{kMaximum} bf16 rows");
    check(!taken(*context, last_axis(ReductionKind::kSum), half_in, half_out), "Reduce{kSum} f16 not taken");
  }
  {  // RmsNorm bf16 with bf16 / f32 weight; f16 weight and non-f32 accumulation are declined
    const std::array out{bf16_mat};
    const std::array in16{bf16_mat, bf16_w};
    const std::array in32{bf16_mat, f32_w};
    const std::array inh{bf16_mat, f16_w};
    check(taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), in16, out), "RmsNorm bf16, bf16 weight");
    check(taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), in32, out), "RmsNorm bf16, f32 weight");
    check(!taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), inh, out), "RmsNorm bf16 with f16 weight not taken");
    const auto half_rows = dense(DataType::kFloat16, {64, 2048}), float_rows = dense(DataType::kFloat32, {64, 2048});
    const auto half_w = dense(DataType::kFloat16, {2048}), float_w = dense(DataType::kFloat32, {2048});
    const std::array half_in{half_rows, half_w}, half_wide{half_rows, float_w};
    const std::array float_in{float_rows, float_w}, float_narrow{float_rows, half_w};
    const std::array half_out{half_rows};
    const std::array float_out{float_rows};
    check(taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), half_in, half_out), "RmsNorm f16, f16 weight");
    check(taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), half_wide, half_out), "RmsNorm f16, f32 weight");
    check(taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), float_in, float_out), "RmsNorm f32, f32 weight");
    check(!taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), float_narrow, float_out), "RmsNorm f32 with f16 weight not taken");
    const auto long_rows = dense(DataType::kFloat32, {4, 32768});
    const std::array long_in{long_rows};
    const std::array long_out{long_rows};
    check(!taken(*context, Operation(RmsNorm{.epsilon = 1e-6F}), long_in, long_out), "RmsNorm f32 rows beyond 64 KB not taken");
  }
  {  // LayerNorm bf16: alone, or with bf16 scale and bias
    const std::array out{bf16_mat};
    const std::array plain{bf16_mat};
    const std::array affine{bf16_mat, bf16_w, bf16_w};
    check(taken(*context, Operation(LayerNorm{.epsilon = 1e-5F}), plain, out), "LayerNorm bf16 without parameters");
    check(taken(*context, Operation(LayerNorm{.epsilon = 1e-5F}), affine, out), "LayerNorm bf16, bf16 scale and bias");
  }
  {  // GatedActivation: separate and packed halves
    const auto gate = dense(DataType::kBFloat16, {32, 6144});
    const auto packed = dense(DataType::kBFloat16, {32, 12288});
    const std::array separate{gate, gate};
    const std::array one{packed};
    const std::array out{gate};
    check(taken(*context, Operation(GatedActivation{GatedActivationKind::kSilu, GatedInputKind::kSeparate}), separate, out),
          "GatedActivation{kSilu, kSeparate} bf16");
    check(taken(*context, Operation(GatedActivation{GatedActivationKind::kSilu, GatedInputKind::kPackedHalves}), one, out),
          "GatedActivation{kSilu, kPackedHalves} bf16");
    check(taken(*context, Operation(GatedActivation{GatedActivationKind::kGelu, GatedInputKind::kSeparate}), separate, out),
          "GatedActivation{kGelu, kSeparate} bf16");
    const auto half = dense(DataType::kFloat16, {32, 6144});
    const std::array separate16{half, half};
    const std::array out16{half};
    check(taken(*context, Operation(GatedActivation{GatedActivationKind::kSilu, GatedInputKind::kSeparate}), separate16, out16),
          "GatedActivation{kSilu, kSeparate} f16 (the form the native CPU route keeps)");
    const auto wide = dense(DataType::kFloat32, {32, 6144});
    const std::array separate32{wide, wide};
    const std::array out32{wide};
    check(!taken(*context, Operation(GatedActivation{GatedActivationKind::kSilu, GatedInputKind::kSeparate}), separate32, out32),
          "GatedActivation f32 not taken");
    std::array<TensorDesc, 1> fused_out{};
    check(b200::ActivationMultiply{}.infer_output_descriptions(separate, fused_out).ok() &&
              taken(*context, Operation::custom(b200::ActivationMultiply{.activation = UnaryKind::kGelu}), separate, fused_out),
          "custom b200-activation-multiply{kGelu}");
    check(!taken(*context, Operation::custom(b200::ActivationMultiply{.activation = UnaryKind::kTanh}), separate, fused_out),
          "b200-activation-multiply{kTanh} not taken");
  }
  {  // Softmax / LogSoftmax / Cast / TopK{1}
    const auto logits = dense(DataType::kFloat32, {16, 151936});
    const auto probs16 = dense(DataType::kBFloat16, {16, 151936});
    const auto values = dense(DataType::kFloat32, {16, 1});
    const auto indices = dense(DataType::kInt32, {16, 1});
    const std::array in{logits};
    const std::array out{logits};
    check(taken(*context, Operation(Softmax{}), in, out), "Softmax{axis=-1} f32");
    check(taken(*context, Operation(Softmax{.kind = SoftmaxKind::kLogSoftmax}), in, out), "Softmax{kLogSoftmax} f32");
    check(!taken(*context, Operation(Softmax{.scale = 0.5F}), in, out), "scaled f32 Softmax without a mask not taken");
    const auto scores = dense(DataType::kFloat16, {8, 128, 1024});
    const auto keep = dense(DataType::kBool, {128, 1024});
    const std::array masked_in{scores, keep};
    const std::array masked_out{scores};
    check(taken(*context, Operation(Softmax{.scale = 0.125F, .mask = MaskKind::kBoolean}), masked_in, masked_out),
          "Softmax{scale, Boolean mask} f16 [8,128,1024] with mask [128,1024]");
    const std::array biased_in{scores, dense(DataType::kFloat16, {128, 1024})};
    check(taken(*context, Operation(Softmax{.scale = 0.125F, .mask = MaskKind::kAdditive}), biased_in, masked_out),
          "Softmax{scale, additive mask} f16 [8,128,1024] with f16 addends [128,1024]");
    const std::array wide_in{scores, dense(DataType::kFloat32, {128, 1024})};
    check(!taken(*context, Operation(Softmax{.scale = 0.125F, .mask = MaskKind::kAdditive}), wide_in, masked_out),
          "additive mask of another floating type not taken");
    const std::array cast_out{probs16};
    check(taken(*context, Operation(Cast{DataType::kBFloat16}), in, cast_out), "Cast{f32 -> bf16}");
    const std::array fp8_out{dense(DataType::kFloat8E4M3FN, {16, 151936})};
    check(taken(*context, Operation(Cast{DataType::kFloat8E4M3FN}), in, fp8_out), "Cast{f32 -> E4M3}");
    const std::array half_in{probs16};
    const std::array bool_out{dense(DataType::kBool, {16, 151936})};
    check(taken(*context, Operation(Cast{DataType::kBool}), half_in, bool_out), "Cast{bf16 -> bool}");
    const std::array e5m2_out{dense(DataType::kFloat8E5M2, {16, 151936})};
    check(!taken(*context, Operation(Cast{DataType::kFloat8E5M2}), in, e5m2_out), "Cast{f32 -> E5M2} not taken (no such CPU pair)");
    const std::array top_out{values, indices};
    check(taken(*context, Operation(TopK{.count = 1}), in, top_out), "TopK{count=1} -> values f32, indices i32");
    std::array<TensorDesc, 3> head3{};
    std::array<TensorDesc, 2> head2{};
    check(b200::GreedyHead{}.infer_output_descriptions(in, head3).ok() && head3[1] == values && head3[2] == indices &&
              taken(*context, Operation::custom(b200::GreedyHead{}), in, head3),
          "custom b200-greedy-head -> probabilities bf16, values, indices");
    check(b200::GreedyHead{.values = false}.infer_output_descriptions(in, head2).ok() && head2[1] == indices &&
              taken(*context, Operation::custom(b200::GreedyHead{.values = false}), in, head2),
          "custom b200-greedy-head{values = false} -> probabilities bf16, indices");
  }
  {  // the fused operators and CacheEncode{q8_0}, with inferred outputs
    const std::array in3{bf16_mat, bf16_mat, bf16_w};
    std::array<TensorDesc, 2> out2{};
    check(b200::FusedAddRmsNorm{}.infer_output_descriptions(in3, out2).ok() &&
              taken(*context, Operation::custom(b200::FusedAddRmsNorm{.epsilon = 1e-6F}), in3, out2),
          "custom b200-add-rms-norm");
    const std::array in2{f32_mat, f32_row};
    std::array<TensorDesc, 3> out3{};
    check(b200::BiasRowSumMax{}.infer_output_descriptions(in2, out3).ok() &&
              taken(*context, Operation::custom(b200::BiasRowSumMax{}), in2, out3),
          "custom b200-bias-row-sum-max");
    const auto logits = dense(DataType::kFloat32, {16, 151936});
    const std::array in1{logits};
    std::array<TensorDesc, 4> out4{};
    check(b200::LogitsReduce{}.infer_output_descriptions(in1, out4).ok() &&
              taken(*context, Operation::custom(b200::LogitsReduce{}), in1, out4),
          "custom b200-logits-reduce");
    const auto weights = dense(DataType::kBFloat16, {1024, 8192});
    const std::array inw{weights};
    std::array<TensorDesc, 3> outw{};
    check(b200::Q8_0Roundtrip{}.infer_output_descriptions(inw, outw).ok() && outw[0].dimensions()[1] == 8704,
          "b200-q8_0-roundtrip infers the U8[rows, cols/32*34] carrier");
    auto prepared = prepare(*context, Operation::custom(b200::Q8_0Roundtrip{}), std::span<const TensorDesc>(inw),
                            std::span<const TensorDesc>(outw), hyle::mem::system_resource());
    check(prepared.has_value() && prepared->workspace_requirement().size == hyle_b200_sum_squares_workspace_bytes(1024ull * 8192) &&
              prepared->capture_compatible(),
          "b200-q8_0-roundtrip prepared; caller-owned workspace = hyle_b200_sum_squares_workspace_bytes(count)");
    model_ops::CacheEncode encode{CacheStorage::q8_0().value()};
    std::array<TensorDesc, 1> carrier{};
    check(encode.infer_output_descriptions(inw, carrier).ok() &&
              taken(*context, Operation::custom(encode), inw, carrier),
          "model_ops::CacheEncode{q8_0} bf16");
    model_ops::CacheEncode encode8{CacheStorage::float8(0.25F).value()};
    std::array<TensorDesc, 1> carrier8{};
    check(encode8.infer_output_descriptions(inw, carrier8).ok() &&
              taken(*context, Operation::custom(encode8), inw, carrier8),
          "model_ops::CacheEncode{float8(0.25)} bf16");
  }
  {  // sampling_ops: the counter generator and the categorical draw
    const auto identities = dense(DataType::kUInt32, {16, 4});
    const auto logits = dense(DataType::kFloat32, {16, 151936});
    const std::array bits_in{identities};
    std::array<TensorDesc, 1> bits_out{};
    const sampling_ops::RandomBits bits{8};
    check(bits.infer_output_descriptions(bits_in, bits_out).ok() &&
              taken(*context, Operation::custom(bits), bits_in, bits_out),
          "sampling_ops::RandomBits{8}");
    const std::array draw_in{logits, identities};
    std::array<TensorDesc, 2> draw_out{};
    const sampling_ops::Categorical draw{true};
    check(draw.infer_output_descriptions(draw_in, draw_out).ok() &&
              taken(*context, Operation::custom(draw), draw_in, draw_out),
          "sampling_ops::Categorical{log probability} f32");
  }
  {  // paged append: the launcher shaped like the CUDA backend's own, host-side argument rules only
    detail::PagedAppendNativeSpec spec{16, 64, 32, 0, 8704};
    check(b200::launch_paged_append(nullptr, nullptr, nullptr, spec, nullptr) == HYLE_B200_OK,
          "paged append: an episode of capacity 0 is nothing to launch");
    spec.instruction_capacity = 8;
    alignas(16) static unsigned char arena[16], rows[16], words[16 + 8 * 32];
    spec.row_bytes = 8703;
    check(b200::launch_paged_append(arena, rows, words, spec, nullptr) == HYLE_B200_INVALID_VALUE,
          "paged append: rows are whole 16-bit elements, as prepare_append demands");
    spec.row_bytes = 8704;
    spec.page_rows = 0;
    check(b200::launch_paged_append(arena, rows, words, spec, nullptr) == HYLE_B200_INVALID_VALUE,
          "paged append: empty pages are refused");
    detail::DeviceLengthsPagedAppendSpec lengths{{16, 64, 32, 8, 8704}, 33};
    unsigned status = 0;
    check(b200::launch_device_lengths_paged_append(arena, rows, words, words, words, lengths, &status, nullptr) ==
              HYLE_B200_NOT_SUPPORTED,
          "device-lengths append: more than 32 requests are outside the qualified domain");
    lengths.requests = 7;
    check(b200::launch_device_lengths_paged_append(arena, rows, words, words, words, lengths, &status, nullptr) ==
              HYLE_B200_NOT_SUPPORTED,
          "device-lengths append: the capacity must hold the directory, the bounds and one page");
  }
  {  // Every cold allocation may fail: provider, Context, prepare and create_invocation then end in
     // ResourceExhausted with nothing left allocated, and the next attempt with memory succeeds (the
     // reference checks its own sample the same way: tests/compute/custom_kernel_test.cc:541-581).
    struct Budget final {
      hyle::mem::AllocatorRef backing = hyle::mem::system_allocator();
      std::size_t asked = 0, refuse_at = SIZE_MAX, live = 0;
      static void *take(void *self, std::size_t size, std::size_t alignment) noexcept {
        auto &b = *static_cast<Budget *>(self);
        if (b.asked++ == b.refuse_at) return nullptr;
        void *p = b.backing.allocate(size, alignment);
        if (p != nullptr) ++b.live;
        return p;
      }
      static void give(void *self, void *p, std::size_t size, std::size_t alignment) noexcept {
        auto &b = *static_cast<Budget *>(self);
        if (p != nullptr) --b.live;
        b.backing.deallocate(p, size, alignment);
      }
      static void *resize(void *self, void *p, std::size_t old_size, std::size_t size, std::size_t alignment) noexcept {
        auto &b = *static_cast<Budget *>(self);
        if (size != 0 && b.asked++ == b.refuse_at) return nullptr;
        void *next = b.backing.reallocate(p, old_size, size, alignment);
        if (size == 0) {
          if (p != nullptr) --b.live;
        } else if (next != nullptr && p == nullptr) {
          ++b.live;
        }
        return next;
      }
      hyle::mem::AllocatorRef ref() noexcept { return {&take, &give, &resize, this}; }
    };
    const std::array add_in{f32_mat, f32_row};
    const std::array add_out{f32_mat};
    auto attempt = [&](Budget &budget) -> Status {
      auto made = b200::make_provider<ProbeBackend>(budget.ref());
      if (!made) return std::move(made).error();
      const std::array bindings{ProviderBinding{std::move(*made), 100}};
      auto own = Context::create(cpu::device(), {.metadata_allocator = budget.ref(), .providers = bindings});
      if (!own) return std::move(own).error();
      auto prepared = prepare(*own, Operation(Binary{BinaryKind::kAdd}), add_in, add_out, hyle::mem::system_resource());
      if (!prepared) return std::move(prepared).error();
      if (prepared->provider().id != b200::kIdentity.id) return Status::Internal("another provider was selected");
      auto invocation = prepared->create_invocation();
      if (!invocation) return std::move(invocation).error();
      return Status::Ok();
    };
    Budget budget;
    const bool plain = attempt(budget).ok() && budget.live == 0;
    const std::size_t allocations = budget.asked;
    bool every = plain && allocations > 0;
    for (std::size_t k = 0; every && k < allocations; ++k) {
      budget.asked = 0;
      budget.refuse_at = k;
      every = attempt(budget).IsResourceExhausted() && budget.live == 0;
      budget.asked = 0;
      budget.refuse_at = SIZE_MAX;
      every = every && attempt(budget).ok() && budget.live == 0;
    }
    std::printf("      %zu cold allocations between make_provider and create_invocation\n", allocations);
    check(every, "each cold allocation refused in turn: ResourceExhausted, nothing left allocated, the next attempt succeeds");
  }
  std::printf("%d failure(s)\n", failures);
  return failures == 0 ? 0 : 1;
}

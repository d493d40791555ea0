// HYLE provider adapter for libhyle_b200.so (C++23, against the reference's public headers).
//
// The provider is a custom-kernel Factory/Kernel pair (include/hyle/compute/custom_kernel.h:157-174,
// 302-315) exactly like the reference's CUDA sample (samples/package/graph/custom_kernel/cuda_main.cc:33-126):
// propose()/prepare() match a request against the operators the kernel library implements and
// decline everything else with Status::Unimplemented; enqueue() takes the Queue's stream and the
// tensors' device pointers and makes ONE call through the C ABI (include/hyle_b200.h).  Nothing here
// allocates, synchronises or falls back to another implementation.
//
// The backend is a template parameter because the three things the adapter needs from it -- the
// cudaStream_t of a QueueSequence, the device pointer of a BufferView and the sequence's device
// status word -- come from the CUDA backend the Context was created on.  Two bindings exist:
// `backend::Cuda12Backend` (b200_backend.h, a thin backend built with the CUDA 12.x runtime) and
// `CudaBackend` (below, the reference's own backend, include/hyle/compute/backends/cuda.h, which needs
// CUDA >= 13.3 and is compiled only when that header is usable).  Tests may supply another Backend
// to drive the cold path on the reference's CPU backend.
#pragma once

#include <array>
#include <cstdint>
#include <optional>
#include <span>
#include <utility>

#include <hyle/compute/custom_kernel.h>
#include <hyle/compute/model_ops.h>
#include <hyle/compute/operation.h>

#include <hyle/compute/sampling_ops.h>

#include "b200_ops.h"
#include "b200_trace.h"
#include "hyle_b200.h"

namespace hyle::compute::b200 {

inline constexpr ProviderIdentity kIdentity{{kNamespace, 1}, "hyle-b200", "1"};
inline constexpr ProviderRuntimeProperties kRuntime{.replay_class = ProviderReplayClass::kPrepared,
                                                    .capture_compatible = true};

enum class Entry : std::uint8_t {
  kUnary, kBinary, kSelect, kReduceRows, kScan, kRmsNorm, kLayerNorm, kSwiglu, kSoftmax, kMaskedSoftmax, kCast, kArgmax, kQ8Encode, kFp8Encode, kRandomBits, kCategorical,
  kAddRmsNorm, kBiasRowSumMax, kLogitsReduce, kQ8Roundtrip, kActivationMultiply, kGreedyHead
};
inline constexpr std::size_t kEntryCount = 22;
// Trace zone names, in the order of Entry.
inline constexpr std::array<const char *, kEntryCount> kEnqueueZone{
    "hyle_b200.enqueue.unary", "hyle_b200.enqueue.binary", "hyle_b200.enqueue.select", "hyle_b200.enqueue.reduce_rows",
    "hyle_b200.enqueue.scan", "hyle_b200.enqueue.rms_norm", "hyle_b200.enqueue.layer_norm", "hyle_b200.enqueue.swiglu",
    "hyle_b200.enqueue.softmax", "hyle_b200.enqueue.masked_softmax", "hyle_b200.enqueue.cast", "hyle_b200.enqueue.argmax",
    "hyle_b200.enqueue.q8_0_encode", "hyle_b200.enqueue.fp8_encode", "hyle_b200.enqueue.random_bits",
    "hyle_b200.enqueue.categorical", "hyle_b200.enqueue.add_rms_norm", "hyle_b200.enqueue.bias_row_sum_max",
    "hyle_b200.enqueue.logits_reduce", "hyle_b200.enqueue.q8_0_roundtrip", "hyle_b200.enqueue.activation_multiply",
    "hyle_b200.enqueue.greedy_head"};

// Everything enqueue() needs, frozen at prepare time.  Trivially copyable.
struct Plan final {
  Entry entry{};
  int kind = 0;            // unary / binary / reduce / softmax kind in the C ABI's numbering
  int dtype = 0;           // hyle_b200_dtype of the data (or of the norm weight for the norms)
  int to_dtype = 0;        // Cast: hyle_b200_dtype of the output; RmsNorm: of the rows
  std::uint64_t count = 0; // total elements of input 0
  std::uint64_t rows = 0;
  std::uint64_t cols = 0;
  std::uint64_t rhs_period = 0;
  std::uint64_t gate_stride = 0, up_stride = 0, up_offset = 0;  // SwiGLU layouts, in elements
  float epsilon = 0.0F;    // norm epsilon, the scale of CacheStorage::float8, or the Softmax scale
  bool has_weight = false;
  std::size_t workspace_bytes = 0;  // what the kernel itself needs, at the start of the workspace
  // Strided inputs: each is first made dense in the workspace (behind the kernel's part) by
  // hyle_b200_strided_cast, type onto itself, and the kernel reads the dense temporary.
  struct Gather final {
    std::uint8_t input = 0, rank = 0;
    int dtype = 0;
    std::array<std::int64_t, kMaxTensorRank> dimensions{}, byte_strides{};
    std::size_t offset = 0;  // of the temporary, from the start of the workspace
  };
  std::array<Gather, 4> gathers{};
  std::uint8_t gather_count = 0;
  std::size_t total_workspace_bytes = 0;  // the kernel's part and the temporaries
};

// Storage types hyle_b200_cast knows.
inline std::optional<int> cast_dtype(DataType type) noexcept {
  switch (type) {
    case DataType::kFloat32: return HYLE_B200_F32;
    case DataType::kBFloat16: return HYLE_B200_BF16;
    case DataType::kFloat16: return HYLE_B200_F16;
    case DataType::kFloat8E4M3FN: return HYLE_B200_E4M3;
    case DataType::kFloat8E5M2: return HYLE_B200_E5M2;
    case DataType::kBool: return HYLE_B200_BOOL;
    case DataType::kInt32: return HYLE_B200_I32;
    default: return std::nullopt;
  }
}
// The pairs of src/compute_provider_native/cast.cc:128-176 (and of hyle_b200_cast).
inline bool cast_pair(int from, int to) noexcept {
  const auto wide = [](int t) { return t == HYLE_B200_F32 || t == HYLE_B200_BF16 || t == HYLE_B200_F16; };
  return (wide(from) && wide(to) && from != to) || (from == HYLE_B200_I32 && to == HYLE_B200_F32) ||
         (wide(from) && (to == HYLE_B200_BOOL || to == HYLE_B200_E4M3)) ||
         ((from == HYLE_B200_BOOL || from == HYLE_B200_E4M3) && wide(to)) ||
         (from == HYLE_B200_E5M2 && (to == HYLE_B200_BF16 || to == HYLE_B200_E4M3));
}

inline std::optional<int> abi_dtype(DataType type) noexcept {
  switch (type) {
    case DataType::kFloat32: return HYLE_B200_F32;
    case DataType::kBFloat16: return HYLE_B200_BF16;
    case DataType::kFloat16: return HYLE_B200_F16;
    default: return std::nullopt;
  }
}

inline std::uint64_t elements(const TensorDesc &d) noexcept {
  const auto n = d.element_count();
  return n ? static_cast<std::uint64_t>(*n) : 0;
}
inline std::uint64_t last_extent(const TensorDesc &d) noexcept {
  return d.rank() == 0 ? 1 : static_cast<std::uint64_t>(d.dimensions().back());
}
inline bool all_dense(std::span<const TensorDesc> a, std::span<const TensorDesc> b) noexcept {
  for (const auto &d : a) if (!d.is_dense() || !d.is_plain()) return false;
  for (const auto &d : b) if (!d.is_dense() || !d.is_plain()) return false;
  return true;
}
// rhs equals lhs, or is lhs's trailing axes (NumPy broadcast of a lower-rank right operand).
inline bool trailing_axes(const TensorDesc &lhs, const TensorDesc &rhs) noexcept {
  if (rhs.rank() > lhs.rank()) return false;
  const auto l = lhs.dimensions(), r = rhs.dimensions();
  for (std::size_t i = 0; i < r.size(); ++i)
    if (r[r.size() - 1 - i] != l[l.size() - 1 - i]) return false;
  return true;
}

// The provider's domain.  nullopt = decline (another provider may take the request).
inline std::optional<Plan> match_dense(const Operation &op, std::span<const TensorDesc> in,
                                       std::span<const TensorDesc> out) noexcept {
  if (in.empty() || out.empty() || !all_dense(in, out)) return std::nullopt;
  Plan p{};
  p.count = elements(in[0]);
  p.cols = last_extent(in[0]);
  p.rows = p.cols ? p.count / p.cols : 0;
  const auto type = abi_dtype(in[0].data_type());

  if (const auto *unary = op.get_if<Unary>()) {
    // hyle_b200_unary_kind follows UnaryKind's order (include/hyle/compute/operation.h:57-73)
    if (in.size() != 1 || out.size() != 1 || !type || out[0] != in[0] ||
        static_cast<int>(unary->kind) > HYLE_B200_UNARY_SOFTPLUS)
      return std::nullopt;
    p.entry = Entry::kUnary;
    p.kind = static_cast<int>(unary->kind);
    p.dtype = *type;
    return p;
  }
  if (op.get_if<Select>() != nullptr) {
    // condition Bool of the output's shape; each branch of that shape or of its trailing axes
    if (in.size() != 3 || out.size() != 1 || in[0].data_type() != DataType::kBool || in[1].data_type() != in[2].data_type() ||
        out[0].data_type() != in[1].data_type() || in[0].dimensions().size() != out[0].dimensions().size() ||
        elements(in[0]) != elements(out[0]) || !trailing_axes(out[0], in[1]) || !trailing_axes(out[0], in[2]))
      return std::nullopt;
    const auto branch = cast_dtype(in[1].data_type());
    if (!branch || (*branch != HYLE_B200_F32 && *branch != HYLE_B200_I32 && *branch != HYLE_B200_BF16 && *branch != HYLE_B200_F16))
      return std::nullopt;
    p.entry = Entry::kSelect;
    p.dtype = *branch;
    p.count = elements(out[0]);
    p.rhs_period = elements(in[1]) ? elements(in[1]) : 1;   // period of when_true
    p.gate_stride = elements(in[2]) ? elements(in[2]) : 1;  // period of when_false
    return p;
  }
  if (const auto *binary = op.get_if<Binary>()) {
    if (in.size() != 2 || out.size() != 1 || !type || in[1].data_type() != in[0].data_type() ||
        out[0] != in[0] || !trailing_axes(in[0], in[1]))
      return std::nullopt;
    switch (binary->kind) {
      case BinaryKind::kAdd: p.kind = HYLE_B200_BINARY_ADD; break;
      case BinaryKind::kSubtract: p.kind = HYLE_B200_BINARY_SUBTRACT; break;
      case BinaryKind::kMultiply: p.kind = HYLE_B200_BINARY_MULTIPLY; break;
      case BinaryKind::kDivide: p.kind = HYLE_B200_BINARY_DIVIDE; break;
      case BinaryKind::kMinimum: p.kind = HYLE_B200_BINARY_MINIMUM; break;
      case BinaryKind::kMaximum: p.kind = HYLE_B200_BINARY_MAXIMUM; break;
      default: return std::nullopt;
    }
    p.entry = Entry::kBinary;
    p.dtype = *type;
    p.rhs_period = elements(in[1]) ? elements(in[1]) : 1;
    return p;
  }
  if (const auto *reduce = op.get_if<Reduce>()) {
    // last axis only, dense output without the reduced axis; f32 every kind, bf16 and f16 the extrema
    // (exact in the rows' own type, f32 comparison)
    const bool narrow = type && *type != HYLE_B200_F32;
    if (in.size() != 1 || out.size() != 1 || !type || in[0].rank() == 0 || reduce->keep_dimensions ||
        elements(out[0]) != p.rows || out[0].data_type() != in[0].data_type())
      return std::nullopt;
    if (narrow && ((reduce->kind != ReductionKind::kMinimum && reduce->kind != ReductionKind::kMaximum) ||
                   (reduce->accumulation_type != DataType::kUnknown && reduce->accumulation_type != DataType::kFloat32)))
      return std::nullopt;
    p.dtype = *type;
    const auto axes = reduce->axes.values();
    const auto last = static_cast<int>(in[0].rank()) - 1;
    if (reduce->axes.is_all() ? in[0].rank() != 1 : (axes.size() != 1 || (axes[0] != -1 && axes[0] != last)))
      return std::nullopt;
    switch (reduce->kind) {
      case ReductionKind::kSum: p.kind = HYLE_B200_REDUCE_SUM; break;
      case ReductionKind::kMean: p.kind = HYLE_B200_REDUCE_MEAN; break;
      case ReductionKind::kMinimum: p.kind = HYLE_B200_REDUCE_MINIMUM; break;
      case ReductionKind::kMaximum: p.kind = HYLE_B200_REDUCE_MAXIMUM; break;
      default: return std::nullopt;
    }
    p.entry = Entry::kReduceRows;
    return p;
  }
  if (const auto *scan = op.get_if<Scan>()) {
    // last axis, f32 or i32, same dense description.  The i32 scan reports overflow through the
    // sequence's device status word (OutOfRange at the Completion, nothing written), as
    // src/compute_provider_ggml/standard_index.cc:127-134 does on the host.
    const auto last = static_cast<int>(in.empty() ? 0 : in[0].rank()) - 1;
    const bool f32 = in[0].data_type() == DataType::kFloat32, i32 = in[0].data_type() == DataType::kInt32;
    if (in.size() != 1 || out.size() != 1 || (!f32 && !i32) || in[0].rank() == 0 || out[0] != in[0] ||
        (scan->axis != -1 && scan->axis != last))
      return std::nullopt;
    p.entry = Entry::kScan;
    p.kind = scan->exclusive ? 1 : 0;
    p.dtype = f32 ? HYLE_B200_F32 : HYLE_B200_I32;
    return p;
  }
  if (const auto *norm = op.get_if<RmsNorm>()) {
    // bf16, f16 or f32 rows; the weight of the row's type or f32 (rows beyond 64 KB only as bf16, up to 32768)
    if (in.empty() || in.size() > 2 || out.size() != 1 || !type || out[0] != in[0] ||
        norm->accumulation_type != DataType::kFloat32)
      return std::nullopt;
    if (*type == HYLE_B200_BF16 ? p.cols > 32768 : p.cols * (*type == HYLE_B200_F32 ? 4 : 2) > 65536)
      return std::nullopt;
    p.has_weight = in.size() == 2;
    p.to_dtype = *type;
    p.dtype = *type;
    if (p.has_weight) {
      const auto weight = abi_dtype(in[1].data_type());
      if (!weight || (*weight != *type && *weight != HYLE_B200_F32) || elements(in[1]) != p.cols) return std::nullopt;
      p.dtype = *weight;
    }
    p.entry = Entry::kRmsNorm;
    p.epsilon = norm->epsilon;
    return p;
  }
  if (const auto *norm = op.get_if<LayerNorm>()) {
    // x alone, or x with scale and bias of [hidden], all bf16 (scale without bias is left to others)
    if ((in.size() != 1 && in.size() != 3) || out.size() != 1 || in[0].data_type() != DataType::kBFloat16 ||
        out[0] != in[0] || norm->accumulation_type != DataType::kFloat32 || p.cols > 32768)
      return std::nullopt;
    p.has_weight = in.size() == 3;
    if (p.has_weight && (in[1].data_type() != DataType::kBFloat16 || in[2].data_type() != DataType::kBFloat16 ||
                         elements(in[1]) != p.cols || elements(in[2]) != p.cols))
      return std::nullopt;
    p.entry = Entry::kLayerNorm;
    p.epsilon = norm->epsilon;
    return p;
  }
  if (const auto *gated = op.get_if<GatedActivation>()) {
    // kSilu, kGelu, kGeluTanh on bf16 or f16 (hyle_b200_gate_kind follows GatedActivationKind's order)
    if (static_cast<int>(gated->activation) > HYLE_B200_GATE_GELU_TANH || !type || *type == HYLE_B200_F32 ||
        out.size() != 1 || out[0].data_type() != in[0].data_type())
      return std::nullopt;
    p.entry = Entry::kSwiglu;
    p.kind = static_cast<int>(gated->activation);
    p.dtype = *type;
    if (gated->inputs == GatedInputKind::kPackedHalves) {
      if (in.size() != 1 || p.cols % 2 != 0 || last_extent(out[0]) * 2 != p.cols) return std::nullopt;
      p.cols /= 2;
      p.gate_stride = p.up_stride = 2 * p.cols;
      p.up_offset = p.cols;
    } else {
      if (in.size() != 2 || in[1] != in[0] || out[0] != in[0]) return std::nullopt;
      p.gate_stride = p.up_stride = p.cols;
    }
    return p;
  }
  if (const auto *masked = op.get_if<Softmax>(); masked != nullptr && masked->mask != MaskKind::kNone) {
    // the attention-score form: f16 values, a Bool mask or f16 addends of the same shape or of its
    // trailing axes (last axis included), any scale, f32 accumulation
    const bool additive = masked->mask == MaskKind::kAdditive;
    if (in.size() != 2 || out.size() != 1 || in[0].data_type() != DataType::kFloat16 || out[0] != in[0] ||
        in[1].data_type() != (additive ? DataType::kFloat16 : DataType::kBool) ||
        masked->kind != SoftmaxKind::kSoftmax || in[0].rank() == 0 ||
        in[1].rank() == 0 || !trailing_axes(in[0], in[1]) ||
        (masked->axis != -1 && masked->axis != static_cast<std::int32_t>(in[0].rank()) - 1) ||
        (masked->accumulation_type != DataType::kUnknown && masked->accumulation_type != DataType::kFloat32))
      return std::nullopt;
    p.entry = Entry::kMaskedSoftmax;
    p.kind = additive ? 1 : 0;
    p.epsilon = masked->scale;
    p.rhs_period = elements(in[1]);
    return p;
  }
  if (const auto *softmax = op.get_if<Softmax>()) {
    if (in.size() != 1 || out.size() != 1 || in[0].data_type() != DataType::kFloat32 || out[0] != in[0] ||
        softmax->scale != 1.0F || softmax->mask != MaskKind::kNone || in[0].rank() == 0 ||
        (softmax->axis != -1 && softmax->axis != static_cast<std::int32_t>(in[0].rank()) - 1))
      return std::nullopt;
    p.entry = Entry::kSoftmax;
    p.kind = softmax->kind == SoftmaxKind::kLogSoftmax ? HYLE_B200_LOG_SOFTMAX : HYLE_B200_SOFTMAX;
    p.workspace_bytes = static_cast<std::size_t>(hyle_b200_logits_workspace_bytes(p.rows, p.cols));
    return p;
  }
  if (const auto *cast = op.get_if<Cast>()) {
    const auto from = cast_dtype(in[0].data_type());
    const auto to = cast_dtype(cast->output_type);
    if (in.size() != 1 || out.size() != 1 || !from || !to || out[0].data_type() != cast->output_type ||
        elements(out[0]) != p.count || !cast_pair(*from, *to))
      return std::nullopt;
    p.entry = Entry::kCast;
    p.dtype = *from;
    p.to_dtype = *to;
    return p;
  }
  if (const auto *top = op.get_if<TopK>()) {
    // greedy token: values f32[..., 1] and indices i32[..., 1] over the last axis
    if (in.size() != 1 || out.size() != 2 || top->count != 1 || !top->largest || in[0].rank() == 0 ||
        in[0].data_type() != DataType::kFloat32 || out[0].data_type() != DataType::kFloat32 ||
        out[1].data_type() != DataType::kInt32 ||
        (top->axis != -1 && top->axis != static_cast<std::int32_t>(in[0].rank()) - 1))
      return std::nullopt;
    p.entry = Entry::kArgmax;
    return p;
  }
  if (const auto encode = op.custom_as<model_ops::CacheEncode>()) {
    if (in.size() != 1 || out.size() != 1 || !type) return std::nullopt;
    if (encode->storage.data_type() == DataType::kFloat8E4M3FN) {  // CacheStorage::float8(scale)
      if (out[0].data_type() != DataType::kFloat8E4M3FN || elements(out[0]) != p.count) return std::nullopt;
      p.entry = Entry::kFp8Encode;
      p.dtype = *type;
      p.epsilon = encode->storage.scale();
      return p;
    }
    if (!(encode->storage == CacheStorage::q8_0().value()) || p.cols % 32 != 0 || out[0].data_type() != DataType::kUInt8)
      return std::nullopt;
    p.entry = Entry::kQ8Encode;
    p.dtype = *type;
    return p;
  }
  if (const auto bits = op.custom_as<sampling_ops::RandomBits>()) {
    // identities u32[rows, 4] -> words u32[rows, word_count]
    if (in.size() != 1 || out.size() != 1 || in[0].data_type() != DataType::kUInt32 || in[0].rank() != 2 ||
        in[0].dimensions()[1] != 4 || out[0].data_type() != DataType::kUInt32)
      return std::nullopt;
    p.entry = Entry::kRandomBits;
    p.rows = static_cast<std::uint64_t>(in[0].dimensions()[0]);
    p.cols = bits->word_count;
    return p;
  }
  if (const auto draw = op.custom_as<sampling_ops::Categorical>()) {
    // (log-weights [rows, cols], identities u32[rows, 4]) -> indices i32[rows] (, log p f32[rows])
    if (in.size() != 2 || out.empty() || out.size() > 2 || !type || in[0].rank() != 2 ||
        in[1].data_type() != DataType::kUInt32 || out[0].data_type() != DataType::kInt32 ||
        (out.size() == 2) != draw->return_log_probability)
      return std::nullopt;
    p.entry = Entry::kCategorical;
    p.dtype = *type;
    p.has_weight = draw->return_log_probability;
    return p;
  }
  if (const auto fused = op.custom_as<FusedAddRmsNorm>()) {
    const auto weight = in.size() == 3 ? abi_dtype(in[2].data_type()) : std::nullopt;
    if (in.size() != 3 || out.size() != 2 || in[0].data_type() != DataType::kBFloat16 || in[1] != in[0] ||
        !weight || *weight == HYLE_B200_F16)
      return std::nullopt;
    p.entry = Entry::kAddRmsNorm;
    p.dtype = *weight;
    p.has_weight = true;
    p.epsilon = fused->epsilon;
    return p;
  }
  if (op.custom_as<BiasRowSumMax>()) {
    if (in.size() != 2 || out.size() != 3 || in[0].data_type() != DataType::kFloat32 ||
        in[1].data_type() != DataType::kFloat32)
      return std::nullopt;
    p.entry = Entry::kBiasRowSumMax;
    return p;
  }
  if (op.custom_as<LogitsReduce>()) {
    if (in.size() != 1 || out.size() != 4 || in[0].data_type() != DataType::kFloat32) return std::nullopt;
    p.entry = Entry::kLogitsReduce;
    p.workspace_bytes = static_cast<std::size_t>(hyle_b200_logits_workspace_bytes(p.rows, p.cols));
    return p;
  }
  if (const auto fused = op.custom_as<ActivationMultiply>()) {
    int kind = -1;
    switch (fused->activation) {
      case UnaryKind::kSilu: kind = HYLE_B200_GATE_SILU; break;
      case UnaryKind::kGelu: kind = HYLE_B200_GATE_GELU; break;
      case UnaryKind::kGeluTanh: kind = HYLE_B200_GATE_GELU_TANH; break;
      default: break;
    }
    if (kind < 0 || in.size() != 2 || out.size() != 1 || !type || *type == HYLE_B200_F32 || in[1] != in[0] || out[0] != in[0])
      return std::nullopt;
    p.entry = Entry::kActivationMultiply;
    p.kind = kind;
    p.dtype = *type;
    p.gate_stride = p.up_stride = p.cols;
    return p;
  }
  if (const auto head = op.custom_as<GreedyHead>()) {
    const std::size_t index = head->values ? 2 : 1;
    if (in.size() != 1 || out.size() != index + 1 || in[0].data_type() != DataType::kFloat32 || in[0].rank() == 0 ||
        out[0].data_type() != DataType::kBFloat16 || elements(out[0]) != p.count ||
        (head->values && (out[1].data_type() != DataType::kFloat32 || elements(out[1]) != p.rows)) ||
        out[index].data_type() != DataType::kInt32 || elements(out[index]) != p.rows)
      return std::nullopt;
    p.entry = Entry::kGreedyHead;
    p.has_weight = head->values;
    p.workspace_bytes = static_cast<std::size_t>(hyle_b200_logits_workspace_bytes(p.rows, p.cols));
    return p;
  }
  if (op.custom_as<Q8_0Roundtrip>()) {
    if (in.size() != 1 || out.size() != 3 || in[0].data_type() != DataType::kBFloat16) return std::nullopt;
    p.entry = Entry::kQ8Roundtrip;
    p.workspace_bytes = static_cast<std::size_t>(hyle_b200_sum_squares_workspace_bytes(p.count));
    return p;
  }
  return std::nullopt;
}

inline std::size_t aligned_256(std::size_t bytes) noexcept { return (bytes + 255) & ~static_cast<std::size_t>(255); }
inline std::size_t storage_width(int cast_type) noexcept {
  return cast_type == HYLE_B200_F32 || cast_type == HYLE_B200_I32 ? 4 : (cast_type == HYLE_B200_BF16 || cast_type == HYLE_B200_F16 ? 2 : 1);
}

// The provider's domain including strided INPUTS (plain storage, non-negative strides that are
// multiples of the element size, as the reference reads every operand of its tensor kernels,
// src/compute_provider_cuda/tensor_kernel.cu:70-108): the request is matched with those inputs
// described dense, and the plan gathers each into a dense temporary before the kernel.  Outputs must
// be dense.
// `input` viewed with the dimensions `target` under the NumPy rule (axes aligned at the end; an extent of 1,
// or a missing leading axis, repeats): the strides of the input where the extents agree, zero where it
// repeats -- what the reference's own broadcast view produces (src/compute_ops/operation.cc:440-472).
inline std::optional<TensorDesc> expanded(const TensorDesc &input, std::span<const std::int64_t> target) noexcept {
  if (!input.is_plain() || target.size() < input.rank() || target.size() > kMaxTensorRank) return std::nullopt;
  std::array<std::int64_t, kMaxTensorRank> strides{};
  const std::size_t prefix = target.size() - input.rank();
  for (std::size_t axis = prefix; axis < target.size(); ++axis) {
    const std::int64_t extent = input.dimensions()[axis - prefix];
    if (extent == target[axis]) strides[axis] = input.byte_strides()[axis - prefix];
    else if (extent != 1) return std::nullopt;
  }
  auto made = TensorDesc::strided_bytes(input.data_type(), target, std::span<const std::int64_t>(strides.data(), target.size()));
  if (!made) return std::nullopt;
  return *made;
}

inline std::optional<Plan> match(const Operation &op, std::span<const TensorDesc> in,
                                 std::span<const TensorDesc> out) noexcept {
  if (in.size() > 4) return std::nullopt;
  // What each input is read as.  Binary operands follow the NumPy rule on both sides (infer_binary,
  // src/compute_ops/operation.cc:476-486): an operand that is neither the output's shape nor (on the right)
  // its trailing axes is read through its broadcast view, i.e. as a strided input.
  std::array<TensorDesc, 4> viewed{};
  for (std::size_t i = 0; i < in.size(); ++i) viewed[i] = in[i];
  if (op.get_if<Binary>() != nullptr && in.size() == 2 && out.size() == 1 && out[0].is_dense()) {
    for (std::size_t i = 0; i < 2; ++i) {
      const bool as_is = in[i].rank() == out[0].rank() && elements(in[i]) == elements(out[0]);
      const bool trailing = i == 1 && in[1].is_dense() && trailing_axes(out[0], in[1]);
      if (as_is || trailing) continue;
      const auto view = expanded(in[i], out[0].dimensions());
      if (!view) return std::nullopt;
      viewed[i] = *view;
    }
  }
  bool strided = false;
  for (std::size_t i = 0; i < in.size(); ++i) strided = strided || !viewed[i].is_dense();
  if (!strided) {
    auto plan = match_dense(op, in, out);
    if (plan) plan->total_workspace_bytes = plan->workspace_bytes;
    return plan;
  }
  std::array<TensorDesc, 4> dense_in{};
  for (std::size_t i = 0; i < in.size(); ++i) {
    dense_in[i] = viewed[i];
    if (viewed[i].is_dense()) continue;
    const auto type = cast_dtype(viewed[i].data_type());
    if (!viewed[i].is_plain() || !type || viewed[i].rank() == 0) return std::nullopt;
    for (const auto stride : viewed[i].byte_strides())
      if (stride < 0 || stride % static_cast<std::int64_t>(storage_width(*type)) != 0) return std::nullopt;
    auto made = TensorDesc::dense(viewed[i].data_type(), viewed[i].dimensions());
    if (!made) return std::nullopt;
    dense_in[i] = *made;
  }
  auto plan = match_dense(op, std::span<const TensorDesc>(dense_in.data(), in.size()), out);
  if (!plan) return std::nullopt;
  std::size_t end = aligned_256(plan->workspace_bytes);
  for (std::size_t i = 0; i < in.size(); ++i) {
    if (viewed[i].is_dense()) continue;
    auto &gather = plan->gathers[plan->gather_count++];
    gather.input = static_cast<std::uint8_t>(i);
    gather.rank = static_cast<std::uint8_t>(viewed[i].rank());
    gather.dtype = *cast_dtype(viewed[i].data_type());
    for (std::size_t axis = 0; axis < viewed[i].rank(); ++axis) {
      gather.dimensions[axis] = viewed[i].dimensions()[axis];
      gather.byte_strides[axis] = viewed[i].byte_strides()[axis];
    }
    gather.offset = end;
    end = aligned_256(end + elements(viewed[i]) * storage_width(gather.dtype));
  }
  plan->total_workspace_bytes = end;
  return plan;
}

// Entries whose kernels report through the sequence's device status word.
inline bool uses_status_word(const Plan &p) noexcept {
  switch (p.entry) {
    case Entry::kQ8Encode: case Entry::kFp8Encode: case Entry::kCategorical: case Entry::kQ8Roundtrip: return true;
    case Entry::kScan: return p.dtype == HYLE_B200_I32;
    case Entry::kSoftmax: case Entry::kLogitsReduce: case Entry::kGreedyHead:
      return p.workspace_bytes != 0;  // the streaming kernel
    default: return false;
  }
}

// One call through the C ABI.  Returns its cudaError_t-compatible result.  `status_word` is the
// sequence's device status word, or null for entries that report nothing.
inline int launch(const Plan &p, hyle_b200_stream_t stream, const void *const *in, void *const *out,
                  void *workspace, std::uint32_t *status_word) noexcept {
  switch (p.entry) {
    case Entry::kUnary:
      return hyle_b200_unary(stream, p.kind, p.dtype, in[0], out[0], p.count);
    case Entry::kSelect:
      return hyle_b200_select(stream, p.dtype, in[0], in[1], in[2], out[0], p.count, p.rhs_period, p.gate_stride);
    case Entry::kBinary:
      return hyle_b200_binary(stream, p.kind, p.dtype, in[0], in[1], out[0], p.count, p.rhs_period);
    case Entry::kScan:
      return hyle_b200_scan(stream, p.dtype, in[0], out[0], p.rows, p.cols, p.kind, status_word);
    case Entry::kReduceRows:
      if (p.dtype != HYLE_B200_F32) return hyle_b200_reduce_rows_extremum(stream, p.kind, p.dtype, in[0], out[0], p.rows, p.cols);
      return hyle_b200_reduce_rows_f32(stream, p.kind, static_cast<const float *>(in[0]),
                                       static_cast<float *>(out[0]), p.rows, p.cols);
    case Entry::kRmsNorm:
      return hyle_b200_rms_norm(stream, p.to_dtype, in[0], p.has_weight ? in[1] : nullptr, p.dtype, out[0], p.rows, p.cols,
                                p.epsilon);
    case Entry::kLayerNorm:
      return hyle_b200_layer_norm_bf16(stream, in[0], p.has_weight ? in[1] : nullptr, p.has_weight ? in[2] : nullptr,
                                       out[0], p.rows, p.cols, p.epsilon);
    case Entry::kSwiglu:
    case Entry::kActivationMultiply: {
      const auto *gate = static_cast<const std::uint16_t *>(in[0]);
      const void *up = p.up_offset ? static_cast<const void *>(gate + p.up_offset) : in[1];
      return hyle_b200_gated_activation(stream, p.kind, p.dtype, p.entry == Entry::kActivationMultiply ? 1 : 0, gate, up,
                                        out[0], p.rows, p.cols, p.gate_stride, p.up_stride);
    }
    case Entry::kGreedyHead:
      return hyle_b200_logits_reduce_f32(stream, static_cast<const float *>(in[0]), p.rows, p.cols, nullptr, out[0],
                                         static_cast<std::int32_t *>(out[p.has_weight ? 2 : 1]),
                                         p.has_weight ? static_cast<float *>(out[1]) : nullptr, workspace, p.workspace_bytes,
                                         status_word);
    case Entry::kSoftmax:
      return hyle_b200_softmax_f32(stream, p.kind, static_cast<const float *>(in[0]), static_cast<float *>(out[0]),
                                   p.rows, p.cols, workspace, p.workspace_bytes, status_word);
    case Entry::kMaskedSoftmax:
      if (p.kind == 1)
        return hyle_b200_additive_masked_softmax_f16(stream, in[0], in[1], p.rhs_period, p.epsilon, out[0], p.rows, p.cols);
      return hyle_b200_masked_softmax_f16(stream, in[0], static_cast<const unsigned char *>(in[1]), p.rhs_period, p.epsilon,
                                          out[0], p.rows, p.cols);
    case Entry::kCast:
      return hyle_b200_cast(stream, p.dtype, p.to_dtype, in[0], out[0], p.count);
    case Entry::kArgmax:
      return hyle_b200_logits_reduce_f32(stream, static_cast<const float *>(in[0]), p.rows, p.cols, nullptr, nullptr,
                                         static_cast<std::int32_t *>(out[1]), static_cast<float *>(out[0]), nullptr, 0,
                                         nullptr);
    case Entry::kQ8Encode:
      return hyle_b200_q8_0_encode(stream, p.dtype, in[0], p.count, out[0], status_word);
    case Entry::kFp8Encode:
      return hyle_b200_fp8_e4m3_encode(stream, p.dtype, in[0], p.count, p.epsilon, out[0], status_word);
    case Entry::kRandomBits:
      return hyle_b200_random_bits(stream, static_cast<const std::uint32_t *>(in[0]), p.rows,
                                   static_cast<std::uint32_t>(p.cols), static_cast<std::uint32_t *>(out[0]));
    case Entry::kCategorical:
      return hyle_b200_categorical(stream, p.dtype, in[0], static_cast<const std::uint32_t *>(in[1]), p.rows, p.cols,
                                   static_cast<std::int32_t *>(out[0]),
                                   p.has_weight ? static_cast<float *>(out[1]) : nullptr, status_word);
    case Entry::kAddRmsNorm:
      return hyle_b200_add_rms_norm_bf16(stream, in[0], in[1], in[2], p.dtype, out[0], out[1], p.rows, p.cols,
                                         p.epsilon);
    case Entry::kBiasRowSumMax:
      return hyle_b200_add_bias_row_sum_max_f32(stream, static_cast<const float *>(in[0]),
                                                static_cast<const float *>(in[1]), static_cast<float *>(out[0]),
                                                static_cast<float *>(out[1]), static_cast<float *>(out[2]), p.rows,
                                                p.cols);
    case Entry::kLogitsReduce:
      return hyle_b200_logits_reduce_f32(stream, static_cast<const float *>(in[0]), p.rows, p.cols,
                                         static_cast<float *>(out[0]), out[1], static_cast<std::int32_t *>(out[2]),
                                         static_cast<float *>(out[3]), workspace, p.workspace_bytes, status_word);
    case Entry::kQ8Roundtrip:
      return hyle_b200_q8_0_roundtrip_bf16(stream, in[0], p.count, out[0], out[1], static_cast<double *>(out[2]),
                                           status_word, workspace, p.workspace_bytes);
  }
  return HYLE_B200_INVALID_VALUE;
}

inline AliasSupport alias_support(const Plan &p, std::size_t output, std::size_t input) noexcept {
  const bool in_place = (p.entry == Entry::kUnary || p.entry == Entry::kBinary || p.entry == Entry::kRmsNorm ||
                         p.entry == Entry::kLayerNorm || p.entry == Entry::kSoftmax) &&
                        output == 0 && input == 0;
  return {in_place, 0};
}

// Backend concept:
//   static constexpr BackendId id();                         which backend the provider serves
//   static constexpr mem::MemoryProperty memory();           what the tensors must be
//   static Result<hyle_b200_stream_t> stream(detail::QueueSequence &);
//   static Result<const void *> pointer(mem::ConstBufferView);
//   static Result<void *> mutable_pointer(mem::BufferView);
//   static Status status(int abi_result);                    C ABI result -> Status
//   static detail::EnqueueResult status_word(detail::QueueSequence &, unsigned **word);
//       the sequence's device status word (cleared on first use in the sequence; the sequence's
//       Completion reports what the kernels OR into it)
template <class Backend>
struct Kernel final {
  Plan plan;
  struct Invocation final {
    void *workspace = nullptr;
    // The caller's workspace arrives with arbitrary contents, and the kernels that use one need
    // counters that start at zero (each launch then leaves them zeroed again).  The first enqueue of
    // an invocation therefore records one clear of the workspace on the queue's stream.
    bool workspace_cleared = false;
  };

  Result<Invocation> create_invocation(mem::BufferView workspace, mem::AllocatorRef) const noexcept {
    Invocation invocation{};
    if (plan.total_workspace_bytes != 0) {
      auto pointer = Backend::mutable_pointer(workspace);
      if (!pointer) return std::unexpected(std::move(pointer).error());
      invocation.workspace = *pointer;
    }
    return invocation;
  }
  AliasSupport alias_support(std::size_t output, std::size_t input) const noexcept {
    return b200::alias_support(plan, output, input);
  }
  KernelCommandResult enqueue(Invocation &invocation, detail::QueueSequence &sequence,
                              std::span<const ConstTensorView> inputs,
                              std::span<const TensorView> outputs) const noexcept {
    HYLE_B200_TRACE_ZONE(kEnqueueZone[static_cast<std::size_t>(plan.entry)]);
    auto stream = Backend::stream(sequence);
    if (!stream) return KernelCommandResult::rejected(std::move(stream).error());
    std::array<const void *, 4> in{};
    std::array<void *, 4> out{};
    if (inputs.size() > in.size() || outputs.size() > out.size())
      return KernelCommandResult::rejected(Status::Internal("hyle-b200: binding count changed after prepare"));
    for (std::size_t i = 0; i < inputs.size(); ++i) {
      auto pointer = Backend::pointer(inputs[i].storage());
      if (!pointer) return KernelCommandResult::rejected(std::move(pointer).error());
      in[i] = *pointer;
    }
    for (std::size_t i = 0; i < outputs.size(); ++i) {
      auto pointer = Backend::mutable_pointer(outputs[i].storage());
      if (!pointer) return KernelCommandResult::rejected(std::move(pointer).error());
      out[i] = *pointer;
    }
    if (plan.count == 0 && plan.entry != Entry::kReduceRows) return KernelCommandResult::no_op();
    // Recorded on the Queue's stream: no synchronisation, no allocation, no second Completion
    // (docs/user/compute.md:1560-1565).  Once anything is recorded, a later failure is the
    // Completion's terminal status, never a rejection.
    bool recorded = false;
    unsigned *status_word = nullptr;
    if (uses_status_word(plan)) {
      auto acquired = Backend::status_word(sequence, &status_word);
      recorded = acquired.accepted;
      if (!acquired.status.ok())
        return recorded ? KernelCommandResult::accepted_command(std::move(acquired.status))
                        : KernelCommandResult::rejected(std::move(acquired.status));
    }
    for (std::size_t g = 0; g < plan.gather_count; ++g) {
      const auto &gather = plan.gathers[g];
      void *dense = static_cast<std::byte *>(invocation.workspace) + gather.offset;
      const int gathered = hyle_b200_strided_cast(*stream, gather.dtype, gather.dtype, in[gather.input], dense, gather.rank,
                                                  gather.dimensions.data(), gather.byte_strides.data());
      if (gathered != HYLE_B200_OK)
        return recorded ? KernelCommandResult::accepted_command(Backend::status(gathered))
                        : KernelCommandResult::rejected(Backend::status(gathered));
      in[gather.input] = dense;
      recorded = true;
    }
    if (plan.workspace_bytes != 0 && !invocation.workspace_cleared) {
      const int cleared = hyle_b200_workspace_clear(*stream, invocation.workspace, plan.workspace_bytes);
      if (cleared != HYLE_B200_OK)
        return recorded ? KernelCommandResult::accepted_command(Backend::status(cleared))
                        : KernelCommandResult::rejected(Backend::status(cleared));
      invocation.workspace_cleared = true;
      recorded = true;
    }
    return KernelCommandResult::accepted_command(Backend::status(
        launch(plan, *stream, in.data(), out.data(), plan.workspace_bytes != 0 ? invocation.workspace : nullptr, status_word)));
  }
};

template <class Backend>
struct Factory final {
  Result<KernelProposal> propose(const KernelRequest &request, std::span<ResourceRequirement> inputs,
                                 std::span<ResourceRequirement> outputs) const noexcept {
    HYLE_B200_TRACE_ZONE("hyle_b200.propose");
    const auto plan = match(request.operation, request.inputs, request.outputs);
    if (!plan) return std::unexpected(Status::Unimplemented("hyle-b200: operation outside the provider's domain"));
    const ResourceRequirement storage{.required_properties = Backend::memory(), .minimum_alignment = 16};
    for (auto &requirement : inputs) requirement = storage;
    for (auto &requirement : outputs) requirement = storage;
    const WorkspaceRequirement workspace{.size = plan->total_workspace_bytes, .alignment = 256};
    return KernelProposal{.route = static_cast<std::uint64_t>(plan->entry),
                          .runtime = kRuntime,
                          .workspace_resource = {.required_properties = Backend::memory(), .minimum_alignment = 256},
                          .cost = {.workspace = workspace,
                                   .persistent_bytes = 0,
                                   .copy_bytes = 0,
                                   .repack_bytes = plan->gather_count != 0 ? plan->total_workspace_bytes - aligned_256(plan->workspace_bytes) : 0,
                                   .synchronization_count = 0,
                                   .dispatch_count = 1u + plan->gather_count},
                          .implementation = ProviderImplementationId{static_cast<std::uint64_t>(plan->entry) + 1}};
  }
  KernelPreparation prepare(const KernelPrepareRequest &request, mem::AllocatorRef allocator) const noexcept {
    HYLE_B200_TRACE_ZONE("hyle_b200.prepare");
    const auto plan = match(request.operation, request.inputs, request.outputs);
    if (!plan) return KernelPreparation::unsupported(Status::Unimplemented("hyle-b200: declined at prepare"));
    auto kernel = make_custom_kernel(
        Kernel<Backend>{*plan},
        {.workspace = {.size = plan->total_workspace_bytes, .alignment = 256}, .runtime = kRuntime, .persistent_bytes = 0},
        allocator);
    if (!kernel) return KernelPreparation::error(std::move(kernel).error());
    return KernelPreparation::prepared(std::move(*kernel));
  }
};

// `allocator`: where the Provider's own cold objects live (default: the system allocator), as in
// make_custom_provider (include/hyle/compute/custom_kernel.h:327-360).
template <class Backend>
Result<Provider> make_provider(mem::AllocatorRef allocator = {}) noexcept {
  return make_custom_provider(kIdentity, Backend::id(), Factory<Backend>{}, allocator);
}

}  // namespace hyle::compute::b200

#if defined(HYLE_B200_WITH_REFERENCE_CUDA_BACKEND)
// Production binding: needs the reference's CUDA backend (CUDA Toolkit >= 13.3).
#include <hyle/compute/backends/cuda.h>
namespace hyle::compute::b200 {
struct CudaBackend final {
  static constexpr BackendId id() noexcept { return cuda::kBackendId; }
  static constexpr mem::MemoryProperty memory() noexcept { return mem::MemoryProperty::kDeviceAccessible; }
  static Result<hyle_b200_stream_t> stream(detail::QueueSequence &sequence) noexcept {
    auto s = cuda::stream(sequence);
    if (!s) return std::unexpected(std::move(s).error());
    return reinterpret_cast<hyle_b200_stream_t>(*s);
  }
  static Result<const void *> pointer(mem::ConstBufferView view) noexcept {
    auto p = cuda::pointer<std::byte>(view);
    if (!p) return std::unexpected(std::move(p).error());
    return static_cast<const void *>(*p);
  }
  static Result<void *> mutable_pointer(mem::BufferView view) noexcept {
    auto p = cuda::pointer<std::byte>(view);
    if (!p) return std::unexpected(std::move(p).error());
    return static_cast<void *>(*p);
  }
  static Status status(int result) noexcept { return cuda::status(static_cast<cudaError_t>(result)); }
  // The reference's same-build seam (src/compute_backend_cuda/native_context.h:72-73).  Its Completion
  // decodes DeviceStatusCode values, not this library's bits: a build inside the reference tree maps
  // the bits to codes with a one-thread kernel after the launch, or adopts the codes in the kernels.
  static detail::EnqueueResult status_word(detail::QueueSequence &sequence, unsigned **word) noexcept {
    return cuda::detail::acquire_device_status(sequence, word);
  }
};
inline Result<Provider> provider() noexcept { return make_provider<CudaBackend>(); }
}  // namespace hyle::compute::b200
#endif

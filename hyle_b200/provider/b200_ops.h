// Fused operators of the B200 provider, declared the way HYLE declares its own model operators
// (model_ops::CacheEncode, include/hyle/compute/model_ops.h:215-229): a trivially copyable
// descriptor with an identity, traits and output inference, wrapped by Operation::custom().
// The IDs name the complete schema including the numerical contract; a change gets a new ID.
#pragma once

#include <algorithm>
#include <array>
#include <cstdint>
#include <span>
#include <string_view>

#include <hyle/compute/operation.h>
#include <hyle/compute/tensor_desc.h>

namespace hyle::compute::b200 {

inline constexpr std::uint64_t kNamespace = 0x48594c4542323030ULL;  // "HYLEB200"

// (x, residual, weight) -> (y, h):  h = bf16(f32 x + f32 residual);  y = RmsNorm(h) * weight.
// The norm reads the rounded h, so (y, h) equals Binary{kAdd} followed by RmsNorm bit for bit.
struct FusedAddRmsNorm final {
  static constexpr OperationId operation_id{kNamespace, 1};
  static constexpr std::string_view operation_name = "b200-add-rms-norm";
  float epsilon = 1.0e-6F;

  OperationTraits operation_traits() const noexcept { return {.inputs = {3, 3}, .outputs = 2}; }
  Status infer_output_descriptions(std::span<const TensorDesc> inputs, std::span<TensorDesc> outputs) const noexcept {
    if (inputs.size() != 3 || outputs.size() != 2 || inputs[0] != inputs[1] || inputs[0].rank() == 0 ||
        inputs[2].rank() != 1 || inputs[2].dimensions()[0] != inputs[0].dimensions().back())
      return Status::InvalidArgument("add-rms-norm expects x, residual of one shape and weight[hidden]");
    outputs[0] = outputs[1] = inputs[0];
    return Status::Ok();
  }
};

// (A[rows, cols], bias[cols]) -> (C, rowsum[rows], rowmax[rows]), f32.
struct BiasRowSumMax final {
  static constexpr OperationId operation_id{kNamespace, 2};
  static constexpr std::string_view operation_name = "b200-bias-row-sum-max";

  OperationTraits operation_traits() const noexcept { return {.inputs = {2, 2}, .outputs = 3}; }
  Status infer_output_descriptions(std::span<const TensorDesc> inputs, std::span<TensorDesc> outputs) const noexcept {
    if (inputs.size() != 2 || outputs.size() != 3 || inputs[0].rank() != 2 || inputs[1].rank() != 1 ||
        inputs[1].dimensions()[0] != inputs[0].dimensions()[1])
      return Status::InvalidArgument("bias-row-sum-max expects A[rows, cols] and bias[cols]");
    outputs[0] = inputs[0];
    HYLE_ASSIGN_OR_RETURN(outputs[1], TensorDesc::dense(inputs[0].data_type(), std::array{inputs[0].dimensions()[0]}));
    outputs[2] = outputs[1];
    return Status::Ok();
  }
};

// logits f32[rows, cols] -> (lse f32[rows], probabilities bf16[rows, cols], index i32[rows], value f32[rows]).
struct LogitsReduce final {
  static constexpr OperationId operation_id{kNamespace, 3};
  static constexpr std::string_view operation_name = "b200-logits-reduce";

  OperationTraits operation_traits() const noexcept { return {.inputs = {1, 1}, .outputs = 4}; }
  Status infer_output_descriptions(std::span<const TensorDesc> inputs, std::span<TensorDesc> outputs) const noexcept {
    if (inputs.size() != 1 || outputs.size() != 4 || inputs[0].rank() != 2)
      return Status::InvalidArgument("logits-reduce expects logits[rows, cols]");
    const std::array rows{inputs[0].dimensions()[0]};
    HYLE_ASSIGN_OR_RETURN(outputs[0], TensorDesc::dense(DataType::kFloat32, rows));
    HYLE_ASSIGN_OR_RETURN(outputs[1], TensorDesc::dense(DataType::kBFloat16, inputs[0].dimensions()));
    HYLE_ASSIGN_OR_RETURN(outputs[2], TensorDesc::dense(DataType::kInt32, rows));
    outputs[3] = outputs[0];
    return Status::Ok();
  }
};

// W bf16[rows, cols] -> (Q8_0 carrier u8[rows, cols/32*34], decoded bf16[rows, cols], sum of squares f64[1]).
struct Q8_0Roundtrip final {
  static constexpr OperationId operation_id{kNamespace, 4};
  static constexpr std::string_view operation_name = "b200-q8_0-roundtrip";

  OperationTraits operation_traits() const noexcept { return {.inputs = {1, 1}, .outputs = 3}; }
  Status infer_output_descriptions(std::span<const TensorDesc> inputs, std::span<TensorDesc> outputs) const noexcept {
    if (inputs.size() != 1 || outputs.size() != 3 || inputs[0].rank() != 2 || inputs[0].dimensions()[1] % 32 != 0)
      return Status::InvalidArgument("q8_0-roundtrip expects W[rows, cols] with cols a multiple of 32");
    const std::array carrier{inputs[0].dimensions()[0], inputs[0].dimensions()[1] / 32 * 34};
    HYLE_ASSIGN_OR_RETURN(outputs[0], TensorDesc::dense(DataType::kUInt8, carrier));
    outputs[1] = inputs[0];
    HYLE_ASSIGN_OR_RETURN(outputs[2], TensorDesc::dense(DataType::kFloat64, std::array<std::int64_t, 1>{1}));
    return Status::Ok();
  }
};

// (gate, up) -> out on bf16 / f16 tensors of one shape:  out = storage(storage(activation(gate)) * up), i.e.
// Unary{activation} followed by Binary{kMultiply} with BOTH roundings kept, in one pass.  What a graph
// region presents for that pair of nodes (engine/models/qwen35/block_graph.h:27-40 emits it for 16-bit
// activations).  activation: kSilu, kGelu or kGeluTanh.
struct ActivationMultiply final {
  static constexpr OperationId operation_id{kNamespace, 5};
  static constexpr std::string_view operation_name = "b200-activation-multiply";
  UnaryKind activation = UnaryKind::kSilu;

  OperationTraits operation_traits() const noexcept { return {.inputs = {2, 2}, .outputs = 1}; }
  Status infer_output_descriptions(std::span<const TensorDesc> inputs, std::span<TensorDesc> outputs) const noexcept {
    if (inputs.size() != 2 || outputs.size() != 1 || inputs[0] != inputs[1])
      return Status::InvalidArgument("activation-multiply expects gate and up of one description");
    outputs[0] = inputs[0];
    return Status::Ok();
  }
};

// logits f32[..., V] -> (probabilities bf16[..., V], [values f32[..., 1],] indices i32[..., 1]):
// Softmax{axis=-1} then Cast{bf16}, and TopK{count=1} of the same logits, in one pass over them.
// What a graph region presents for a greedy sampling head that also publishes its distribution
// (engine/inference/sampling_graph.h:339-345 keeps only the index of TopK: `values` = false then).
struct GreedyHead final {
  static constexpr OperationId operation_id{kNamespace, 6};
  static constexpr std::string_view operation_name = "b200-greedy-head";
  bool values = true;

  OperationTraits operation_traits() const noexcept { return {.inputs = {1, 1}, .outputs = values ? 3u : 2u}; }
  Status infer_output_descriptions(std::span<const TensorDesc> inputs, std::span<TensorDesc> outputs) const noexcept {
    if (inputs.size() != 1 || outputs.size() != (values ? 3u : 2u) || inputs[0].rank() == 0 ||
        inputs[0].data_type() != DataType::kFloat32)
      return Status::InvalidArgument("greedy-head expects f32 logits[..., vocabulary]");
    HYLE_ASSIGN_OR_RETURN(outputs[0], TensorDesc::dense(DataType::kBFloat16, inputs[0].dimensions()));
    std::array<std::int64_t, 8> one{};
    const auto dimensions = inputs[0].dimensions();
    if (dimensions.size() > one.size()) return Status::InvalidArgument("greedy-head: rank above 8");
    std::copy(dimensions.begin(), dimensions.end(), one.begin());
    one[dimensions.size() - 1] = 1;
    const std::span<const std::int64_t> selected(one.data(), dimensions.size());
    if (values) {
      HYLE_ASSIGN_OR_RETURN(outputs[1], TensorDesc::dense(DataType::kFloat32, selected));
    }
    HYLE_ASSIGN_OR_RETURN(outputs[values ? 2 : 1], TensorDesc::dense(DataType::kInt32, selected));
    return Status::Ok();
  }
};

}  // namespace hyle::compute::b200

// Graph region provider for the B200 kernel provider (C++23, same-build component of the reference).
//
// The fused kernels behind the C ABI exist as custom operators (b200_ops.h) that a caller would have
// to emit by hand.  Engine graphs emit the unfused recipes instead:
//   Binary{kAdd}(x, residual) -> RmsNorm(h, weight)            engine/models/qwen35/block_graph.h:27-40
//   Unary{kSilu}(gate)        -> Binary{kMultiply}(., up)      engine/models/qwen35/block_graph.h:27-36 (16-bit activations)
//   Softmax{-1}(logits) -> Cast{bf16}   and   TopK{1}(logits)  engine/inference/sampling_graph.h:339-345
// This file makes the provider offer those node sets to graph::compile as REGIONS
// (include/hyle/graph/region_provider.h:153-188,274-311,481-497), each lowered to ONE custom operator
// of the same provider, so that models reach the fused kernels unchanged.
//
// Mechanism, as the reference's own CUDA region providers do it
// (src/graph_route_cuda/dense_bfloat_scores_region.cc:33-60,240-410): the provider's private vtable is
// decorated with a query_extension that answers kRegionProviderExtensionId; discovery matches the
// recipes structurally (operator kinds, arity, exact descriptions, no outside reader of an inner
// value, no control edges); the resource query and compile() re-qualify the chosen node set and hand a
// composite Operation to the provider's ordinary propose/prepare through
// graph::detail::mapped_native_region, which also maps region ports to operator ports.
//
// What a region preserves: every rounding of the unfused recipe.  h = bf16(x + r) is rounded before
// the norm reads it, silu(gate) is rounded to storage before the product, the probabilities are the
// f32 softmax rounded once to bf16: each region's result is the result of its nodes run one by one on
// this provider.
#pragma once

#include <array>
#include <cstdint>
#include <optional>
#include <span>

#include <hyle/container/small_vector.h>
#include <hyle/graph/region_provider.h>

#include "mapped_native_region.h"  // src/graph        (same-build seam)
#include "provider_internal.h"     // src/compute      (same-build seam)

#include "b200_provider.h"

namespace hyle::compute::b200::region {

namespace g = hyle::graph;

inline constexpr RoutePolicyId kPolicy{kNamespace, 0x5245474E /* "REGN" */, 1};
inline constexpr std::uint64_t kRouteAddRmsNorm = 1;
inline constexpr std::uint64_t kRouteActivationMultiply = 2;
inline constexpr std::uint64_t kRouteGreedyHead = 3;
inline constexpr std::size_t kMaxNodes = 3;
inline constexpr std::size_t kMaxPorts = 3;

// One matched recipe: its nodes, the boundary values in the composite operator's port order, and
// the operator itself.
struct Pattern final {
  std::array<g::NodeId, kMaxNodes> nodes{};
  std::size_t size = 0;
  std::array<g::ValueId, kMaxPorts> inputs{};
  std::size_t input_count = 0;
  std::array<g::ValueId, kMaxPorts> outputs{};
  std::size_t output_count = 0;
  std::uint64_t route = 0;
  Operation composite{};

  std::span<const g::NodeId> span() const noexcept { return {nodes.data(), size}; }
  bool contains(g::NodeId node) const noexcept {
    for (std::size_t n = 0; n < size; ++n)
      if (nodes[n] == node) return true;
    return false;
  }
};

namespace detail_region {

template <class T>
std::optional<T> operation(const g::Graph &graph, g::NodeId node) noexcept {
  const auto value = graph.operation(node);
  if (!value) return std::nullopt;
  const auto *typed = value->template get_if<T>();
  return typed ? std::optional<T>{*typed} : std::nullopt;
}
inline g::NodeId producer(const g::Graph &graph, g::ValueId value) noexcept {
  if (value.kind() != g::ValueKind::kNodeOutput) return {};
  const auto result = graph.producer(value);
  return result ? *result : g::NodeId{};
}
// A plain node: the given number of data inputs and outputs, no effect resources, no control
// prerequisites of its own.
inline bool plain_node(const g::Graph &graph, g::NodeId node, std::size_t inputs, std::size_t outputs) noexcept {
  if (!node.valid()) return false;
  const auto in = graph.node_input_count(node), out = graph.node_output_count(node),
             resources = graph.node_resource_count(node), dependencies = graph.node_dependency_count(node);
  return in && out && resources && dependencies && *in == inputs && *out == outputs && *resources == 0 && *dependencies == 0;
}
inline std::optional<TensorDesc> dense_description(const g::Graph &graph, g::ValueId value) noexcept {
  const auto description = graph.value_description(value);
  if (!description || !description->is_plain() || !description->is_dense()) return std::nullopt;
  return *description;
}

// Cold index over the graph: data readers per value (0, 1, "2 or more / published"), the first
// reader, control successors per node, and per value the first TopK{count=1} reader.
struct Uses final {
  container::SmallVector<std::uint8_t, 16, mem::AllocatorRef> data;
  container::SmallVector<g::NodeId, 16, mem::AllocatorRef> reader;
  container::SmallVector<g::NodeId, 16, mem::AllocatorRef> greedy_reader;
  container::SmallVector<std::uint8_t, 16, mem::AllocatorRef> controlled;
  explicit Uses(mem::AllocatorRef allocator) noexcept
      : data(allocator), reader(allocator), greedy_reader(allocator), controlled(allocator) {}

  Status initialize(const g::Graph &graph) noexcept {
    if (!data.try_resize(graph.value_count()) || !reader.try_resize(graph.value_count()) ||
        !greedy_reader.try_resize(graph.value_count()) || !controlled.try_resize(graph.node_count()))
      return Status::ResourceExhausted("b200 region discovery metadata allocation failed");
    for (auto &count : data) count = 0;
    for (auto &node : reader) node = g::NodeId{};
    for (auto &node : greedy_reader) node = g::NodeId{};
    for (auto &flag : controlled) flag = 0;
    for (std::size_t i = 0; i < graph.node_count(); ++i) {
      HYLE_ASSIGN_OR_RETURN(auto node, graph.node_id(i));
      HYLE_ASSIGN_OR_RETURN(auto inputs, graph.node_input_count(node));
      for (std::size_t port = 0; port < inputs; ++port) {
        HYLE_ASSIGN_OR_RETURN(auto value, graph.node_input(node, port));
        auto &count = data[value.ordinal()];
        if (count == 0) reader[value.ordinal()] = node;
        if (count < 2) ++count;
      }
      if (const auto top = operation<TopK>(graph, node); top && top->count == 1 && inputs == 1) {
        HYLE_ASSIGN_OR_RETURN(auto value, graph.node_input(node, 0));
        if (!greedy_reader[value.ordinal()].valid()) greedy_reader[value.ordinal()] = node;
      }
      HYLE_ASSIGN_OR_RETURN(auto dependencies, graph.node_dependency_count(node));
      for (std::size_t n = 0; n < dependencies; ++n) {
        HYLE_ASSIGN_OR_RETURN(auto before, graph.node_dependency(node, n));
        controlled[before.ordinal()] = 1;  // some node waits for `before` through a control edge
      }
    }
    for (std::size_t n = 0; n < graph.output_count(); ++n) {
      HYLE_ASSIGN_OR_RETURN(auto value, graph.output_id(n));
      data[value.ordinal()] = 2;  // a published value has an observer outside every region
    }
    return Status::Ok();
  }
  bool escapes(g::ValueId value, const Pattern &p) const noexcept {
    const auto count = data[value.ordinal()];
    return count >= 2 || (count == 1 && !p.contains(reader[value.ordinal()]));
  }
};

// ---- the three recipes ---------------------------------------------------------------------------------------------
// `norm` is a RmsNorm{f32 accumulation} with a weight whose data input is Binary{kAdd} of two bf16
// tensors of one description.  Outputs in the operator's order (y, h).
inline bool add_rms_norm(const g::Graph &graph, g::NodeId norm, Pattern &p) noexcept {
  const auto rms = operation<RmsNorm>(graph, norm);
  if (!rms || !plain_node(graph, norm, 2, 1) || rms->accumulation_type != DataType::kFloat32) return false;
  const auto h = graph.node_input(norm, 0).value(), weight = graph.node_input(norm, 1).value();
  const auto add_node = producer(graph, h);
  const auto add = operation<Binary>(graph, add_node);
  if (!add || add->kind != BinaryKind::kAdd || !plain_node(graph, add_node, 2, 1)) return false;
  const auto x = graph.node_input(add_node, 0).value(), r = graph.node_input(add_node, 1).value();
  const auto dx = dense_description(graph, x), dr = dense_description(graph, r), dh = dense_description(graph, h),
             dw = dense_description(graph, weight), dy = dense_description(graph, graph.result(norm).value());
  if (!dx || !dr || !dh || !dw || !dy || dx->data_type() != DataType::kBFloat16 || *dr != *dx || *dh != *dx || *dy != *dx ||
      dx->rank() == 0 || dw->rank() != 1 || dw->dimensions()[0] != dx->dimensions().back() ||
      (dw->data_type() != DataType::kBFloat16 && dw->data_type() != DataType::kFloat32))
    return false;
  p = {};
  p.nodes = {add_node, norm, {}};
  p.size = 2;
  p.inputs = {x, r, weight};
  p.input_count = 3;
  p.outputs = {graph.result(norm).value(), h, {}};
  p.output_count = 2;
  p.route = kRouteAddRmsNorm;
  p.composite = Operation::custom(FusedAddRmsNorm{.epsilon = rms->epsilon});
  return true;
}

// `multiply` is Binary{kMultiply} of two 16-bit tensors of one description, one of which is
// Unary{kSilu | kGelu | kGeluTanh} of a tensor of that description.
inline bool activation_multiply(const g::Graph &graph, g::NodeId multiply, Pattern &p) noexcept {
  const auto mul = operation<Binary>(graph, multiply);
  if (!mul || mul->kind != BinaryKind::kMultiply || !plain_node(graph, multiply, 2, 1)) return false;
  for (std::size_t side = 0; side < 2; ++side) {
    const auto activated = graph.node_input(multiply, side).value(), up = graph.node_input(multiply, 1 - side).value();
    const auto unary_node = producer(graph, activated);
    const auto unary = operation<Unary>(graph, unary_node);
    if (!unary || !plain_node(graph, unary_node, 1, 1) ||
        (unary->kind != UnaryKind::kSilu && unary->kind != UnaryKind::kGelu && unary->kind != UnaryKind::kGeluTanh))
      continue;
    const auto gate = graph.node_input(unary_node, 0).value();
    const auto dg = dense_description(graph, gate), da = dense_description(graph, activated), du = dense_description(graph, up),
               dout = dense_description(graph, graph.result(multiply).value());
    if (!dg || !da || !du || !dout || *da != *dg || *du != *dg || *dout != *dg ||
        (dg->data_type() != DataType::kBFloat16 && dg->data_type() != DataType::kFloat16))
      continue;
    p = {};
    p.nodes = {unary_node, multiply, {}};
    p.size = 2;
    p.inputs = {gate, up, {}};
    p.input_count = 2;
    p.outputs = {graph.result(multiply).value(), {}, {}};
    p.output_count = 1;
    p.route = kRouteActivationMultiply;
    p.composite = Operation::custom(ActivationMultiply{.activation = unary->kind});
    return true;
  }
  return false;
}

// `cast` is Cast{bf16} of Softmax{last axis, plain} of f32 logits that a TopK{count=1, largest, last
// axis} node `greedy` also reads.  Outputs in the operator's order (probabilities, [values,] indices).
inline bool greedy_head(const g::Graph &graph, g::NodeId cast, g::NodeId greedy, bool with_values, Pattern &p) noexcept {
  const auto narrow = operation<Cast>(graph, cast);
  if (!narrow || narrow->output_type != DataType::kBFloat16 || !plain_node(graph, cast, 1, 1)) return false;
  const auto soft_node = producer(graph, graph.node_input(cast, 0).value());
  const auto soft = operation<Softmax>(graph, soft_node);
  if (!soft || !plain_node(graph, soft_node, 1, 1) || soft->kind != SoftmaxKind::kSoftmax || soft->scale != 1.0F ||
      soft->mask != MaskKind::kNone)
    return false;
  const auto logits = graph.node_input(soft_node, 0).value();
  const auto dl = dense_description(graph, logits), dp = dense_description(graph, graph.result(cast).value());
  if (!dl || !dp || dl->data_type() != DataType::kFloat32 || dl->rank() == 0) return false;
  const auto last = static_cast<std::int32_t>(dl->rank()) - 1;
  if (soft->axis != -1 && soft->axis != last) return false;
  const auto top = operation<TopK>(graph, greedy);
  if (!top || top->count != 1 || !top->largest || (top->axis != -1 && top->axis != last) || !plain_node(graph, greedy, 1, 2) ||
      graph.node_input(greedy, 0).value() != logits)
    return false;
  p = {};
  p.nodes = {soft_node, cast, greedy};
  p.size = 3;
  p.inputs = {logits, {}, {}};
  p.input_count = 1;
  // the maximum itself is a boundary output only when somebody outside reads it
  if (with_values) p.outputs = {graph.result(cast).value(), graph.result(greedy, 0).value(), graph.result(greedy, 1).value()};
  else p.outputs = {graph.result(cast).value(), graph.result(greedy, 1).value(), {}};
  p.output_count = with_values ? 3 : 2;
  p.route = kRouteGreedyHead;
  p.composite = Operation::custom(GreedyHead{.values = with_values});
  return true;
}

// No value that stays inside the region has a reader outside it, nothing waits for an inner node
// through a control edge, and the caller's node mask admits every node.
inline bool closed(const g::Graph &graph, const Pattern &p, const Uses &uses, std::span<const std::uint8_t> allowed) noexcept {
  for (const auto node : p.span()) {
    if (!allowed.empty() && !allowed[node.ordinal()]) return false;
    if (uses.controlled[node.ordinal()]) return false;
    const auto outputs = graph.node_output_count(node).value();
    for (std::size_t port = 0; port < outputs; ++port) {
      const auto value = graph.result(node, port).value();
      bool boundary = false;
      for (std::size_t n = 0; n < p.output_count; ++n) boundary = boundary || p.outputs[n] == value;
      if (!boundary && uses.escapes(value, p)) return false;
    }
  }
  return true;
}

}  // namespace detail_region

// The region callbacks for one Backend binding of the provider.
template <class Backend>
struct RegionProvider final {
  using ProviderVTable = compute::detail::ProviderVTable;
  using Requirement = compute::detail::ResourceBindingRequirement;
  using Proposal = compute::detail::ProviderOperationProposal;

  // The custom provider's own table (propose / prepare of single operators), captured once.
  static const ProviderVTable *&original_slot() noexcept {
    static const ProviderVTable *table = nullptr;
    return table;
  }
  static const ProviderVTable &original() noexcept { return *original_slot(); }

  struct Described final {
    std::array<TensorDesc, kMaxPorts> inputs;
    std::array<TensorDesc, kMaxPorts> outputs;
    std::array<Requirement, kMaxPorts> input_resources;
    std::array<Requirement, kMaxPorts> output_resources;
    Proposal proposal;
  };

  // The provider's ordinary proposal for the composite operator on the region's descriptions.
  static Status native_proposal(void *context, const g::Graph &graph, const Pattern &p, Described &d,
                                const WorkloadContext &workload = {}) noexcept {
    for (std::size_t n = 0; n < p.input_count; ++n) d.inputs[n] = graph.value_description(p.inputs[n]).value();
    for (std::size_t n = 0; n < p.output_count; ++n) d.outputs[n] = graph.value_description(p.outputs[n]).value();
    std::array<TensorDesc, kMaxPorts> inferred;
    HYLE_RETURN_IF_ERROR(infer_output_descriptions(p.composite, std::span(d.inputs).first(p.input_count),
                                                   std::span(inferred).first(p.output_count)));
    for (std::size_t n = 0; n < p.output_count; ++n)
      if (inferred[n] != d.outputs[n]) return Status::Unimplemented("b200 region: composite output differs from the graph's");
    HYLE_RETURN_IF_ERROR(original().propose(
        context,
        {.operation = p.composite, .inputs = std::span(d.inputs).first(p.input_count),
         .outputs = std::span(d.outputs).first(p.output_count), .workload = workload},
        std::span(d.input_resources).first(p.input_count), std::span(d.output_resources).first(p.output_count), &d.proposal));
    if (d.proposal.cost.persistent_bytes) {
      HYLE_ASSIGN_OR_RETURN(auto bytes, g::detail::mapped_native_region::artifact_bytes(p.input_count, p.output_count));
      if (*d.proposal.cost.persistent_bytes > SIZE_MAX - bytes) return Status::OutOfRange("b200 region metadata bytes overflow");
      *d.proposal.cost.persistent_bytes += bytes;
    }
    return Status::Ok();
  }

  static Status propose(void *context, const g::RegionDiscoveryRequest &request, mem::AllocatorRef allocator,
                        g::RegionProposalWriter &writer) noexcept {
    using namespace detail_region;
    const auto &graph = request.graph;
    if (!request.allowed_nodes.empty() && request.allowed_nodes.size() != graph.node_count())
      return Status::InvalidArgument("b200 region discovery: allowed-node count differs");
    Uses uses(allocator);
    HYLE_RETURN_IF_ERROR(uses.initialize(graph));
    for (std::size_t i = 0; i < graph.node_count(); ++i) {
      HYLE_ASSIGN_OR_RETURN(auto node, graph.node_id(i));
      Pattern p;
      bool found = add_rms_norm(graph, node, p) || activation_multiply(graph, node, p);
      if (!found) {  // a Cast whose logits also feed a greedy TopK
        const auto narrow = operation<Cast>(graph, node);
        if (narrow && plain_node(graph, node, 1, 1)) {
          const auto soft_node = producer(graph, graph.node_input(node, 0).value());
          if (soft_node.valid() && graph.node_input_count(soft_node).value() == 1) {
            const auto logits = graph.node_input(soft_node, 0).value();
            const auto greedy = uses.greedy_reader[logits.ordinal()];
            Pattern none;
            found = greedy.valid() && greedy_head(graph, node, greedy, uses.escapes(graph.result(greedy, 0).value(), none), p);
          }
        }
      }
      if (!found) continue;
      // The residual sum must be wanted outside (the next block reads it): the fused kernel always
      // writes it, and a region cannot have more outputs than its boundary.
      if (p.route == kRouteAddRmsNorm && !uses.escapes(p.outputs[1], p)) continue;
      if (!closed(graph, p, uses, request.allowed_nodes)) continue;
      Described d;
      const auto status = native_proposal(context, graph, p, d);
      if (!status.ok()) {
        if (status.IsUnimplemented() || status.IsInvalidArgument()) continue;  // outside the kernels' domain
        return status;
      }
      HYLE_ASSIGN_OR_RETURN(auto more, writer.try_add({.nodes = p.span(), .cost = d.proposal.cost, .route = p.route,
                                                       .replay_class = d.proposal.runtime.replay_class,
                                                       .implementation = d.proposal.implementation, .policy = kPolicy}));
      if (!more) return Status::Ok();
    }
    return Status::Ok();
  }

  // Re-derive the recipe from the chosen, bounded node set; no graph-wide scan.
  static Status qualify(const g::RegionCompileRequest &request, Pattern &result) noexcept {
    using namespace detail_region;
    if (!request.graph || request.nodes.size() < 2 || request.nodes.size() > kMaxNodes || request.has_unknown_effects ||
        !request.effect_accesses.empty())
      return Status::Unimplemented("b200 region boundary differs");
    const auto &graph = *request.graph;
    for (const auto node : request.nodes) {
      Pattern p;
      bool found = false;
      if (request.route == kRouteAddRmsNorm) found = add_rms_norm(graph, node, p);
      else if (request.route == kRouteActivationMultiply) found = activation_multiply(graph, node, p);
      else if (request.route == kRouteGreedyHead) {
        for (const auto other : request.nodes) {
          if (found || other == node || !operation<TopK>(graph, other)) continue;
          const bool with_values = std::ranges::count(request.outputs, graph.result(other, 0).value()) == 1;
          found = greedy_head(graph, node, other, with_values, p);
        }
      }
      if (!found || p.size != request.nodes.size() || p.input_count != request.inputs.size() ||
          p.output_count != request.outputs.size())
        continue;
      bool exact = true;
      for (const auto inner : p.span()) exact = exact && std::ranges::count(request.nodes, inner) == 1;
      for (std::size_t n = 0; n < p.input_count; ++n) exact = exact && std::ranges::count(request.inputs, p.inputs[n]) == 1;
      for (std::size_t n = 0; n < p.output_count; ++n) exact = exact && std::ranges::count(request.outputs, p.outputs[n]) == 1;
      if (!exact) continue;
      result = p;
      return Status::Ok();
    }
    return Status::Unimplemented("b200 region does not preserve the exact recipe");
  }

  static Status resources(void *context, const g::RegionCompileRequest &request, mem::AllocatorRef,
                          std::span<g::RegionInputRequirement> inputs, std::span<g::RegionOutputRequirement> outputs,
                          g::RegionResourceProposal *result) noexcept {
    *result = {};
    Pattern p;
    HYLE_RETURN_IF_ERROR(qualify(request, p));
    if (inputs.size() != p.input_count || outputs.size() != p.output_count)
      return Status::InvalidArgument("b200 region resource count differs");
    Described d;
    HYLE_RETURN_IF_ERROR(native_proposal(context, *request.graph, p, d, request.workload));
    for (std::size_t n = 0; n < p.input_count; ++n) {
      const auto port = std::ranges::find(request.inputs, p.inputs[n]) - request.inputs.begin();
      inputs[static_cast<std::size_t>(port)] = {.resource = d.input_resources[n]};
    }
    for (std::size_t n = 0; n < p.output_count; ++n) {
      const auto port = std::ranges::find(request.outputs, p.outputs[n]) - request.outputs.begin();
      outputs[static_cast<std::size_t>(port)] = {.resource = d.output_resources[n]};
    }
    *result = {.runtime = d.proposal.runtime, .workspace_resource = d.proposal.workspace_resource,
               .compilation_storage = d.proposal.cost.compilation_storage};
    return Status::Ok();
  }

  static ProviderPrepareOutcome compile(void *context, const g::RegionCompileRequest &request, mem::AllocatorRef allocator,
                                        g::ProviderRegionPrepared *result) noexcept {
    *result = {};
    Pattern p;
    const auto qualification = qualify(request, p);
    if (!qualification.ok()) return ProviderPrepareOutcome::unsupported(qualification);
    if (request.input_resources.size() != p.input_count || request.output_resources.size() != p.output_count)
      return ProviderPrepareOutcome::error(Status::InvalidArgument("b200 region physical resource count differs"));
    Described d;
    const auto status = native_proposal(context, *request.graph, p, d, request.workload);
    if (!status.ok())
      return status.IsUnimplemented() ? ProviderPrepareOutcome::unsupported(status) : ProviderPrepareOutcome::error(status);
    std::array<std::size_t, kMaxPorts> in_ports{}, out_ports{};
    std::array<mem::MemoryResourceRef, kMaxPorts> in_resources{}, out_resources{};
    for (std::size_t n = 0; n < p.input_count; ++n) {
      in_ports[n] = static_cast<std::size_t>(std::ranges::find(request.inputs, p.inputs[n]) - request.inputs.begin());
      in_resources[n] = request.input_resources[in_ports[n]];
    }
    for (std::size_t n = 0; n < p.output_count; ++n) {
      out_ports[n] = static_cast<std::size_t>(std::ranges::find(request.outputs, p.outputs[n]) - request.outputs.begin());
      out_resources[n] = request.output_resources[out_ports[n]];
    }
    return g::detail::mapped_native_region::prepare(
        original(), context,
        {.operation = p.composite, .inputs = std::span(d.inputs).first(p.input_count),
         .outputs = std::span(d.outputs).first(p.output_count), .input_resources = std::span(in_resources).first(p.input_count),
         .output_resources = std::span(out_resources).first(p.output_count), .workspace_resource = request.workspace_resource,
         .route = d.proposal.route, .workload = request.workload},
        d.proposal, std::span(in_ports).first(p.input_count), request.inputs.size(), allocator, result,
        std::span(out_ports).first(p.output_count));
  }

  static const void *query_extension(void *context, ProviderExtensionId id) noexcept {
    static constexpr g::RegionProviderVTable kRegion{.propose = &propose, .propose_resources = &resources, .compile = &compile};
    if (id == g::kRegionProviderExtensionId) return &kRegion;
    return original().query_extension ? original().query_extension(context, id) : nullptr;
  }
};

// The kernel provider with its region extension: what a Context for graph::compile is given.
template <class Backend>
Result<Provider> make_region_provider() noexcept {
  auto provider = make_provider<Backend>();
  if (!provider) return provider;
  using Regions = RegionProvider<Backend>;
  static const compute::detail::ProviderVTable decorated = [&] {
    Regions::original_slot() = compute::detail::ProviderAccess::vtable(*provider);
    auto table = *Regions::original_slot();
    table.query_extension = &Regions::query_extension;
    return table;
  }();
  return compute::detail::ProviderAccess::with_vtable(*provider, &decorated);
}

}  // namespace hyle::compute::b200::region

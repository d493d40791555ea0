// The graph region provider (hyle_b200/provider/b200_region_provider.h) under the REFERENCE's own
// graph::compile.
//
// Part 1 (no GPU): on the reference's CPU backend with a probe Backend that never launches, build the
// recipes engine graphs emit -- Binary{kAdd} -> RmsNorm (engine/models/qwen35/block_graph.h:27-40),
// Unary{kSilu} -> Binary{kMultiply} (the same file's 16-bit feed-forward), Softmax -> Cast{bf16} beside
// TopK{1} on shared logits (engine/inference/sampling_graph.h:339-345) -- compile the graph and read the
// compile report: three regions must be claimed, each by its custom operator, the stray nodes stay
// single operators.  Then near misses: a norm without weight, an f32 residual add, TopK{count=2}, an
// activated gate that is also published, a residual sum nobody else reads: no region may be claimed.
//
// Part 2 (needs a GPU; skipped without one): the same graph on a Context of the thin CUDA-12 backend,
// replayed through graph::Invocation::submit on a Queue, every published value compared byte for byte
// with the direct C-ABI calls of the fused kernels.
//
// Built by tests/provider/Makefile against the reference tree in place.
#include <array>
#include <bit>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include <hyle/compute/backends/cpu.h>
#include <hyle/compute/device.h>
#include <hyle/graph/executable.h>
#include <hyle/graph/execution_source.h>
#include <hyle/graph/graph.h>
#include <hyle/mem/buffer.h>
#include <hyle/simd/dtype.h>

#include "b200_backend.h"
#include "b200_region_provider.h"

using namespace hyle::compute;
namespace graph = hyle::graph;
namespace mem = hyle::mem;
namespace backend = hyle::compute::b200::backend;
using hyle::Result;
using hyle::Status;

static int failures = 0, checks = 0;
static void check(bool ok, const std::string &what) {
  std::printf("%s  %s\n", ok ? "ok  " : "FAIL", what.c_str());
  ++checks;
  if (!ok) ++failures;
}

struct ProbeBackend final {
  static constexpr BackendId id() noexcept { return cpu::kBackendId; }
  static constexpr mem::MemoryProperty memory() noexcept { return mem::MemoryProperty::kHostAccessible; }
  static Result<hyle_b200_stream_t> stream(detail::QueueSequence &) noexcept {
    return std::unexpected(Status::Unimplemented("probe backend: no CUDA stream behind a CPU queue"));
  }
  static Result<const void *> pointer(mem::ConstBufferView) noexcept { return std::unexpected(Status::Unimplemented("probe backend")); }
  static Result<void *> mutable_pointer(mem::BufferView) noexcept { return std::unexpected(Status::Unimplemented("probe backend")); }
  static Status status(int) noexcept { return Status::Internal("probe backend never launches"); }
  static detail::EnqueueResult status_word(detail::QueueSequence &, unsigned **) noexcept {
    return detail::EnqueueResult::rejected(Status::Unimplemented("probe backend"));
  }
};

template <std::size_t N>
static TensorDesc dense(DataType type, const std::int64_t (&dims)[N]) {
  return TensorDesc::dense(type, std::span<const std::int64_t>(dims, N)).value();
}

constexpr std::int64_t kTokens = 64, kHidden = 2048, kFfn = 6144, kBatch = 72, kVocabulary = 19456;

// The values of the model graph a test binds or reads.
struct Model final {
  graph::Graph graph;
  graph::ValueId x, residual, weight, gate, up, logits;          // inputs
  graph::ValueId normed, stream, product, probabilities, token;  // published
};

struct Variation final {
  bool weight = true;            // RmsNorm with a weight
  DataType residual_type = DataType::kBFloat16;
  std::uint32_t top_k = 1;
  bool publish_activated_gate = false;
  bool residual_sum_read_elsewhere = true;
};

static Result<Model> build(const Variation &v) {
  Model m;
  HYLE_ASSIGN_OR_RETURN(auto builder, graph::GraphBuilder::create());
  const auto activations = dense(v.residual_type, {kTokens, kHidden});
  HYLE_ASSIGN_OR_RETURN(m.x, builder.input(activations));
  HYLE_ASSIGN_OR_RETURN(m.residual, builder.input(activations));
  HYLE_ASSIGN_OR_RETURN(m.weight, builder.input(dense(v.residual_type, {kHidden})));
  HYLE_ASSIGN_OR_RETURN(m.gate, builder.input(dense(DataType::kBFloat16, {kTokens, kFfn})));
  HYLE_ASSIGN_OR_RETURN(m.up, builder.input(dense(DataType::kBFloat16, {kTokens, kFfn})));
  HYLE_ASSIGN_OR_RETURN(m.logits, builder.input(dense(DataType::kFloat32, {kBatch, kVocabulary})));
  // residual stream: h = x + residual; y = RmsNorm(h) * w; the stream goes on as h + y
  HYLE_ASSIGN_OR_RETURN(auto h, builder.add(Binary{BinaryKind::kAdd}, m.x, m.residual));
  if (v.weight) {
    HYLE_ASSIGN_OR_RETURN(m.normed, builder.add(RmsNorm{.epsilon = 1e-6F}, h, m.weight));
  } else {
    HYLE_ASSIGN_OR_RETURN(m.normed, builder.add(RmsNorm{.epsilon = 1e-6F}, h));
  }
  if (v.residual_sum_read_elsewhere) {
    HYLE_ASSIGN_OR_RETURN(m.stream, builder.add(Binary{BinaryKind::kAdd}, h, m.normed));
    HYLE_RETURN_IF_ERROR(builder.publish(m.stream));
  }
  HYLE_RETURN_IF_ERROR(builder.publish(m.normed));
  // feed-forward gating on 16-bit activations: silu(gate) * up as two nodes
  HYLE_ASSIGN_OR_RETURN(auto activated, builder.add(Unary{UnaryKind::kSilu}, m.gate));
  HYLE_ASSIGN_OR_RETURN(m.product, builder.add(Binary{BinaryKind::kMultiply}, activated, m.up));
  HYLE_RETURN_IF_ERROR(builder.publish(m.product));
  if (v.publish_activated_gate) HYLE_RETURN_IF_ERROR(builder.publish(activated));
  // greedy head that also publishes its distribution
  HYLE_ASSIGN_OR_RETURN(auto soft, builder.add(Softmax{}, m.logits));
  HYLE_ASSIGN_OR_RETURN(m.probabilities, builder.add(Cast{DataType::kBFloat16}, soft));
  const std::array<graph::ValueId, 1> head_inputs{m.logits};
  HYLE_ASSIGN_OR_RETURN(auto top, builder.add_node(Operation(TopK{.count = v.top_k}), head_inputs));
  HYLE_ASSIGN_OR_RETURN(m.token, builder.result(top, 1));
  HYLE_RETURN_IF_ERROR(builder.publish(m.probabilities));
  HYLE_RETURN_IF_ERROR(builder.publish(m.token));
  HYLE_ASSIGN_OR_RETURN(m.graph, std::move(builder).finish());
  return m;
}

struct Compiled final {
  graph::Executable executable;
  graph::CompileReport report;
};

static Result<Compiled> compile(const Context &context, mem::MemoryResourceRef storage_resource, const graph::Graph &g) {
  const std::array storage{graph::StorageDomain{.resource = storage_resource}};
  HYLE_ASSIGN_OR_RETURN(auto source, graph::ExecutionSource::acquire(context));
  const std::array targets{graph::ExecutionTarget{.source = source, .default_storage = graph::StorageDomainId{0}}};
  HYLE_ASSIGN_OR_RETURN(auto compiled, graph::compile(g, {.storage_domains = storage, .targets = targets}, {}));
  return Compiled{std::move(compiled.executable), std::move(compiled.report)};
}

// How many steps of the report run a custom operator of this provider with the given implementation key.
static std::size_t steps_with_entry(const graph::CompileReport &report, b200::Entry entry) {
  std::size_t count = 0;
  for (std::size_t i = 0; i < report.step_count(); ++i) {
    const auto step = report.step(i);
    if (step && step->implementation == ProviderImplementationId{static_cast<std::uint64_t>(entry) + 1}) ++count;
  }
  return count;
}

static void expect_no_region(const Context &context, const Variation &v, b200::Entry missing, const std::string &what) {
  auto model = build(v);
  if (!model) return check(false, what + ": building the graph: " + std::string(model.error().message()));
  auto compiled = compile(context, mem::system_resource(), model->graph);
  if (!compiled) {
    // declining may leave a node without any provider on this single-provider Context: also a decline
    return check(compiled.error().IsUnimplemented() || compiled.error().IsNotFound() || compiled.error().IsFailedPrecondition(),
                 what + ": not claimed (compile: " + std::string(compiled.error().message()) + ")");
  }
  check(steps_with_entry(compiled->report, missing) == 0, what + ": the near miss is not claimed as a region");
}

static std::uint16_t bf16(float value) { return std::bit_cast<std::uint16_t>(hyle::simd::f32_to_bf16(value)); }

struct Random final {
  std::uint64_t state;
  explicit Random(std::uint64_t seed) : state(seed * 0x9E3779B97F4A7C15ull + 1) {}
  float normal() {
    auto next = [&] {
      state ^= state << 13;
      state ^= state >> 7;
      state ^= state << 17;
      return static_cast<float>(state >> 40) * (1.0f / 16777216.0f);
    };
    const float u = next() + 1e-7f, w = next();
    return std::sqrt(-2.0f * std::log(u)) * std::cos(6.2831853f * w);
  }
};
using Bytes = std::vector<std::byte>;
static Bytes bf16_normal(std::size_t count, std::uint64_t seed, float scale) {
  Random rng(seed);
  std::vector<std::uint16_t> v(count);
  for (auto &x : v) x = bf16(scale * rng.normal());
  Bytes out(count * 2);
  std::memcpy(out.data(), v.data(), out.size());
  return out;
}
static Bytes f32_normal(std::size_t count, std::uint64_t seed, float scale) {
  Random rng(seed);
  std::vector<float> v(count);
  for (auto &x : v) x = scale * rng.normal();
  Bytes out(count * 4);
  std::memcpy(out.data(), v.data(), out.size());
  return out;
}

struct Tensor final {
  mem::Buffer storage;
  TensorView view;
  Tensor(const TensorDesc &desc, mem::MemoryResourceRef resource)
      : storage(mem::Buffer::create(resource, desc.required_bytes().value(), 256).value()),
        view(TensorView::create(desc, storage.view()).value()) {}
  Bytes read() const {
    Bytes out(storage.size());
    storage.view().read(out).IgnoreError();
    return out;
  }
  const void *device() const { return backend::pointer(storage.view()).value(); }
};

static void run_on_gpu() {
  auto provider = b200::region::make_region_provider<backend::Cuda12Backend>();
  auto device = backend::device(0);
  if (!provider || !device) return check(false, "GPU: provider and device");
  auto context = Context::create(*device, std::move(*provider));
  if (!context) return check(false, "GPU: Context::create: " + std::string(context.error().message()));
  auto memory = backend::DeviceMemory::create(*context);
  auto queue = context->create_queue();
  if (!memory || !queue) return check(false, "GPU: memory resource and queue");
  auto model = build({});
  if (!model) return check(false, "GPU: building the graph");
  auto compiled = compile(*context, memory->ref(), model->graph);
  if (!compiled) return check(false, "GPU: graph::compile: " + std::string(compiled.error().message()));
  check(compiled->report.region_count() == 3, "GPU: three regions claimed on the CUDA-12 backend");

  const auto resource = memory->ref();
  const auto &g = model->graph;
  auto tensor_of = [&](graph::ValueId value) { return Tensor(g.value_description(value).value(), resource); };
  Tensor x = tensor_of(model->x), residual = tensor_of(model->residual), weight = tensor_of(model->weight),
         gate = tensor_of(model->gate), up = tensor_of(model->up), logits = tensor_of(model->logits);
  Tensor normed = tensor_of(model->normed), stream = tensor_of(model->stream), product = tensor_of(model->product),
         probabilities = tensor_of(model->probabilities), token = tensor_of(model->token);
  x.storage.view().write(bf16_normal(kTokens * kHidden, 1, 1.0f)).IgnoreError();
  residual.storage.view().write(bf16_normal(kTokens * kHidden, 2, 1.0f)).IgnoreError();
  weight.storage.view().write(bf16_normal(kHidden, 3, 0.5f)).IgnoreError();
  gate.storage.view().write(bf16_normal(kTokens * kFfn, 4, 1.5f)).IgnoreError();
  up.storage.view().write(bf16_normal(kTokens * kFfn, 5, 1.5f)).IgnoreError();
  logits.storage.view().write(f32_normal(kBatch * kVocabulary, 6, 4.0f)).IgnoreError();

  auto invocation = compiled->executable.create_invocation();
  if (!invocation) return check(false, "GPU: create_invocation: " + std::string(invocation.error().message()));
  Status bound = Status::Ok();
  for (auto [value, tensor] : {std::pair{model->x, &x}, {model->residual, &residual}, {model->weight, &weight},
                               {model->gate, &gate}, {model->up, &up}, {model->logits, &logits}})
    bound.Update(invocation->bind(value, tensor->view.as_const()));
  for (auto [value, tensor] : {std::pair{model->normed, &normed}, {model->stream, &stream}, {model->product, &product},
                               {model->probabilities, &probabilities}, {model->token, &token}})
    bound.Update(invocation->bind(value, tensor->view));
  if (!bound.ok()) return check(false, "GPU: binding tensors: " + std::string(bound.message()));
  const std::array queues{graph::QueueBinding{.lane = graph::ExecutionLaneId{0}, .queue = &*queue}};
  const Status prepared = invocation->prepare_replay(queues, {.mode = graph::ReplayMode::kCommands});
  if (!prepared.ok()) return check(false, "GPU: prepare_replay: " + std::string(prepared.message()));
  for (int round = 0; round < 2; ++round) {
    auto done = invocation->submit(queues);
    if (!done) return check(false, "GPU: submit: " + std::string(done.error().message()));
    const Status waited = done->wait();
    if (!waited.ok()) return check(false, "GPU: wait: " + std::string(waited.message()));
  }

  // the fused kernels, called directly on the same inputs
  auto device_buffer = [](std::size_t bytes) {
    void *p = nullptr;
    cudaMalloc(&p, bytes);
    cudaMemset(p, 0xCD, bytes);
    return p;
  };
  auto same = [](const Tensor &tensor, const void *direct) {
    Bytes expected(tensor.storage.size());
    cudaMemcpy(expected.data(), direct, expected.size(), cudaMemcpyDeviceToHost);
    return tensor.read() == expected;
  };
  cudaStream_t s = nullptr;
  cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  auto stream_handle = reinterpret_cast<hyle_b200_stream_t>(s);
  void *y = device_buffer(kTokens * kHidden * 2), *h = device_buffer(kTokens * kHidden * 2), *next = device_buffer(kTokens * kHidden * 2);
  int rc = hyle_b200_add_rms_norm_bf16(stream_handle, x.device(), residual.device(), weight.device(), HYLE_B200_BF16, y, h, kTokens,
                                       kHidden, 1e-6F);
  rc |= hyle_b200_binary(stream_handle, HYLE_B200_BINARY_ADD, HYLE_B200_BF16, h, y, next, kTokens * kHidden, kTokens * kHidden);
  void *m = device_buffer(kTokens * kFfn * 2);
  rc |= hyle_b200_gated_activation(stream_handle, HYLE_B200_GATE_SILU, HYLE_B200_BF16, 1, gate.device(), up.device(), m, kTokens, kFfn,
                                   kFfn, kFfn);
  void *p = device_buffer(kBatch * kVocabulary * 2), *index = device_buffer(kBatch * 4), *value = device_buffer(kBatch * 4);
  const auto workspace_bytes = hyle_b200_logits_workspace_bytes(kBatch, kVocabulary);
  void *workspace = device_buffer(workspace_bytes);
  cudaMemset(workspace, 0, workspace_bytes);
  rc |= hyle_b200_logits_reduce_f32(stream_handle, static_cast<const float *>(logits.device()), kBatch, kVocabulary, nullptr, p,
                                    static_cast<std::int32_t *>(index), static_cast<float *>(value), workspace, workspace_bytes, nullptr);
  const bool ran = rc == HYLE_B200_OK && cudaStreamSynchronize(s) == cudaSuccess;
  check(ran, "GPU: the direct C-ABI calls ran");
  check(same(normed, y) && same(stream, next), "GPU: region {Add, RmsNorm}: y and the continued stream == hyle_b200_add_rms_norm_bf16, byte for byte");
  check(same(product, m), "GPU: region {Unary silu, Multiply} == hyle_b200_gated_activation with the gate rounded, byte for byte");
  check(same(probabilities, p) && same(token, index), "GPU: region {Softmax, Cast, TopK}: probabilities and token == hyle_b200_logits_reduce_f32, byte for byte");
  for (void *pointer : {y, h, next, m, p, index, value, workspace}) cudaFree(pointer);
  cudaStreamDestroy(s);
}

int main() {
  {
    auto provider = b200::region::make_region_provider<ProbeBackend>();
    check(provider.has_value(), "the provider with its region extension");
    if (!provider) return 1;
    auto context = Context::create(cpu::device(), std::move(*provider));
    check(context.has_value(), "Context::create on the reference's CPU backend");
    if (!context) return 1;

    auto model = build({});
    check(model.has_value(), "the model graph: residual add + norm, silu * up, softmax -> bf16 beside a greedy TopK");
    if (!model) {
      std::printf("  %s\n", std::string(model.error().message()).c_str());
      return 1;
    }
    auto compiled = compile(*context, mem::system_resource(), model->graph);
    check(compiled.has_value(), "graph::compile with the region provider");
    if (!compiled) {
      std::printf("  %s\n", std::string(compiled.error().message()).c_str());
      return 1;
    }
    const auto &report = compiled->report;
    std::printf("      nodes %zu, steps %zu, regions %zu\n", report.node_count(), report.step_count(), report.region_count());
    check(report.region_count() == 3, "three regions are claimed");
    check(steps_with_entry(report, b200::Entry::kAddRmsNorm) == 1, "Binary{kAdd} -> RmsNorm runs as b200-add-rms-norm");
    check(steps_with_entry(report, b200::Entry::kActivationMultiply) == 1, "Unary{kSilu} -> Binary{kMultiply} runs as b200-activation-multiply");
    check(steps_with_entry(report, b200::Entry::kGreedyHead) == 1, "Softmax -> Cast{bf16} + TopK{1} runs as b200-greedy-head");
    check(report.step_count() == 4 && steps_with_entry(report, b200::Entry::kBinary) == 1,
          "the eight nodes run as four steps: three regions and the add that continues the residual stream");

    expect_no_region(*context, {.weight = false}, b200::Entry::kAddRmsNorm, "RmsNorm without a weight");
    expect_no_region(*context, {.residual_type = DataType::kFloat32}, b200::Entry::kAddRmsNorm, "f32 residual add");
    expect_no_region(*context, {.top_k = 2}, b200::Entry::kGreedyHead, "TopK{count=2}");
    expect_no_region(*context, {.publish_activated_gate = true}, b200::Entry::kActivationMultiply, "activated gate also published");
    expect_no_region(*context, {.residual_sum_read_elsewhere = false}, b200::Entry::kAddRmsNorm, "residual sum nobody else reads");
  }
  int devices = 0;
  if (cudaGetDeviceCount(&devices) == cudaSuccess && devices > 0) run_on_gpu();
  else std::printf("no CUDA device: the GPU half was skipped\n");
  std::printf("%d check(s), %d failure(s)\n", checks, failures);
  return failures == 0 ? 0 : 1;
}

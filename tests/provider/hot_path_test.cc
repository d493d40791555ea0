// Drives the adapter's HOT path through the REFERENCE's own runtime on a GPU:
//   compute::prepare -> PreparedOperation::create_invocation(workspace) -> OperationInvocation::submit(queue)
//   -> B200Kernel::enqueue -> hyle_b200_* on the Queue's stream -> Completion::wait
// on a Context of the thin CUDA-12 backend (hyle_b200/provider/b200_backend.cc), and compares every
// output byte with the same entry point called directly through the C ABI on the same device inputs.
//
// Every one of the adapter's 22 entries runs twice through one invocation (the second submit reuses
// the workspace the first one left behind), with the caller's workspace POISONED (0xFF) before the
// invocation is created.  Then the error protocol: a NaN in a Q8_0 / FP8 cache-encode input and an
// invalid Categorical row must complete with Status::InvalidArgument, an overflowing i32 Scan with
// Status::OutOfRange (and an untouched output), and the sequence after a failed one must be clean.
// All failures here are host-visible statuses: nothing faults or hangs the GPU.
//
// Built by tests/provider/Makefile against the reference tree in place; prints one line per check
// and exits non-zero when any failed.
#include <array>
#include <bit>
#include <cmath>
#include <cstdint>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <span>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime_api.h>

#include <hyle/compute/device.h>
#include <hyle/compute/model_ops.h>
#include <hyle/compute/prepared_operation.h>
#include <hyle/compute/sampling_ops.h>
#include <hyle/compute/transfer.h>
#include <hyle/mem/buffer.h>
#include <hyle/simd/dtype.h>

#include "b200_backend.h"
#include "b200_provider.h"

using namespace hyle::compute;
namespace mem = hyle::mem;
namespace backend = hyle::compute::b200::backend;
using hyle::Result;
using hyle::Status;

static int failures = 0;
static int checks = 0;
static void check(bool ok, const std::string &what) {
  std::printf("%s  %s\n", ok ? "ok  " : "FAIL", what.c_str());
  ++checks;
  if (!ok) ++failures;
}

// ---- deterministic inputs --------------------------------------------------------------------------------------------
struct Random final {
  std::uint64_t state;
  explicit Random(std::uint64_t seed) : state(seed * 0x9E3779B97F4A7C15ull + 1) {}
  std::uint64_t next() {
    state ^= state << 13;
    state ^= state >> 7;
    state ^= state << 17;
    return state;
  }
  float uniform() { return static_cast<float>(next() >> 40) * (1.0f / 16777216.0f); }  // [0, 1)
  float normal() {
    const float u = uniform() + 1e-7f, v = uniform();
    return std::sqrt(-2.0f * std::log(u)) * std::cos(6.2831853f * v);
  }
};

using Bytes = std::vector<std::byte>;
static std::uint16_t bf16(float value) { return std::bit_cast<std::uint16_t>(hyle::simd::f32_to_bf16(value)); }
static std::uint16_t f16(float value) { return std::bit_cast<std::uint16_t>(hyle::simd::f32_to_f16(value)); }
template <class T>
Bytes bytes_of(const std::vector<T> &values) {
  Bytes out(values.size() * sizeof(T));
  std::memcpy(out.data(), values.data(), out.size());
  return out;
}
static Bytes f32_normal(std::size_t count, std::uint64_t seed, float scale = 1.0f) {
  Random rng(seed);
  std::vector<float> v(count);
  for (auto &x : v) x = scale * rng.normal();
  return bytes_of(v);
}
static Bytes bf16_normal(std::size_t count, std::uint64_t seed, float scale = 1.0f) {
  Random rng(seed);
  std::vector<std::uint16_t> v(count);
  for (auto &x : v) x = bf16(scale * rng.normal());
  return bytes_of(v);
}
static Bytes f16_normal(std::size_t count, std::uint64_t seed, float scale = 1.0f) {
  Random rng(seed);
  std::vector<std::uint16_t> v(count);
  for (auto &x : v) x = f16(scale * rng.normal());
  return bytes_of(v);
}
static Bytes bool_random(std::size_t count, std::uint64_t seed) {
  Random rng(seed);
  Bytes v(count);
  for (auto &x : v) x = static_cast<std::byte>(rng.next() >> 63);
  return v;
}
static Bytes u32_random(std::size_t count, std::uint64_t seed) {
  Random rng(seed);
  std::vector<std::uint32_t> v(count);
  for (auto &x : v) x = static_cast<std::uint32_t>(rng.next() >> 32);
  return bytes_of(v);
}

template <std::size_t N>
static TensorDesc dense(DataType type, const std::int64_t (&dims)[N]) {
  return TensorDesc::dense(type, std::span<const std::int64_t>(dims, N)).value();
}

// ---- a device tensor owned through the reference's Buffer --------------------------------------------------------------
struct Tensor final {
  mem::Buffer storage;
  TensorView view;
  Tensor(const TensorDesc &desc, mem::MemoryResourceRef resource)
      : storage(mem::Buffer::create(resource, desc.required_bytes().value(), 256).value()),
        view(TensorView::create(desc, storage.view()).value()) {}
  Status write(const Bytes &bytes) { return storage.view().write(bytes); }
  Bytes read() const {
    Bytes out(storage.size());
    storage.view().read(out).IgnoreError();
    return out;
  }
  const void *device() const { return backend::pointer(storage.view()).value(); }
};

static void *out_pointer(Tensor &t) { return backend::pointer(t.storage.view()).value(); }

struct Fixture final {
  Context context;
  backend::DeviceMemory memory;
  Queue queue;
};

// The direct C-ABI call of a case: device pointers of the inputs, freshly allocated outputs, a zeroed
// workspace of its own and a zeroed status word, on `stream`.
using Direct = std::function<int(hyle_b200_stream_t stream, const void *const *in, void *const *out, void *workspace,
                                 std::uint64_t workspace_bytes, std::uint32_t *status)>;

struct Case final {
  std::string name;
  Operation operation;
  std::vector<TensorDesc> in;
  std::vector<TensorDesc> out;
  std::vector<Bytes> data;
  std::uint64_t direct_workspace_bytes = 0;
  Direct direct;
  b200::Entry entry;
};

static constexpr std::byte kPoison{0xFF};
static constexpr std::byte kCanary{0xCD};

// Runs one case through the reference's submit() twice and once directly; true when all bytes agree.
static void run_case(Fixture &fixture, const Case &c) {
  const auto resource = fixture.memory.ref();
  std::vector<Tensor> inputs, outputs;
  for (const auto &desc : c.in) inputs.emplace_back(desc, resource);
  for (const auto &desc : c.out) outputs.emplace_back(desc, resource);
  for (std::size_t i = 0; i < inputs.size(); ++i)
    if (!inputs[i].write(c.data[i]).ok()) return check(false, c.name + ": writing an input");
  std::vector<ConstTensorView> in_views;
  std::vector<TensorView> out_views;
  for (auto &t : inputs) in_views.push_back(t.view.as_const());
  for (auto &t : outputs) out_views.push_back(t.view);

  auto prepared = prepare(fixture.context, c.operation, std::span<const ConstTensorView>(in_views),
                          std::span<const TensorView>(out_views), resource);
  if (!prepared) return check(false, c.name + ": prepare: " + std::string(prepared.error().message()));
  if (prepared->provider().id != b200::kIdentity.id) return check(false, c.name + ": selected provider is not hyle-b200");
  if (prepared->implementation().value() != static_cast<std::uint64_t>(c.entry) + 1)
    return check(false, c.name + ": prepared with another entry than the case names");

  // caller-owned workspace with arbitrary (here: all-ones) contents
  const auto requirement = prepared->workspace_requirement();
  mem::Buffer workspace;
  if (requirement.size != 0) {
    workspace = mem::Buffer::create(resource, requirement.size, requirement.alignment).value();
    workspace.view().fill(kPoison).IgnoreError();
  }
  auto invocation = prepared->create_invocation(requirement.size != 0 ? workspace.view() : mem::BufferView{});
  if (!invocation) return check(false, c.name + ": create_invocation: " + std::string(invocation.error().message()));

  std::vector<std::vector<Bytes>> submitted(2);
  for (int round = 0; round < 2; ++round) {
    for (auto &t : outputs) t.storage.view().fill(kCanary).IgnoreError();
    auto done = invocation->submit(fixture.queue, in_views, out_views);
    if (!done) return check(false, c.name + ": submit: " + std::string(done.error().message()));
    const Status waited = done->wait();
    if (!waited.ok()) return check(false, c.name + ": wait: " + std::string(waited.message()));
    for (auto &t : outputs) submitted[round].push_back(t.read());
  }

  // the same entry point, called directly
  std::vector<const void *> in_pointers;
  for (auto &t : inputs) in_pointers.push_back(t.device());
  std::vector<void *> out_pointers(outputs.size(), nullptr);
  for (std::size_t i = 0; i < outputs.size(); ++i) {
    cudaMalloc(&out_pointers[i], outputs[i].storage.size() ? outputs[i].storage.size() : 16);
    cudaMemset(out_pointers[i], static_cast<int>(kCanary), outputs[i].storage.size());
  }
  void *direct_workspace = nullptr;
  if (c.direct_workspace_bytes != 0) {
    cudaMalloc(&direct_workspace, c.direct_workspace_bytes);
    cudaMemset(direct_workspace, 0, c.direct_workspace_bytes);
  }
  std::uint32_t *direct_status = nullptr;
  cudaMalloc(reinterpret_cast<void **>(&direct_status), sizeof(std::uint32_t));
  cudaMemset(direct_status, 0, sizeof(std::uint32_t));
  cudaStream_t stream = nullptr;
  cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  cudaDeviceSynchronize();
  const int rc = c.direct(reinterpret_cast<hyle_b200_stream_t>(stream), in_pointers.data(), out_pointers.data(),
                          direct_workspace, c.direct_workspace_bytes, direct_status);
  const cudaError_t finished = cudaStreamSynchronize(stream);
  bool same = rc == HYLE_B200_OK && finished == cudaSuccess;
  std::string where;
  for (std::size_t i = 0; same && i < outputs.size(); ++i) {
    Bytes direct(outputs[i].storage.size());
    cudaMemcpy(direct.data(), out_pointers[i], direct.size(), cudaMemcpyDeviceToHost);
    for (int round = 0; round < 2; ++round)
      if (direct != submitted[round][i]) {
        same = false;
        where = " (output " + std::to_string(i) + ", submit " + std::to_string(round + 1) + ")";
      }
  }
  std::uint32_t status_bits = 0;
  cudaMemcpy(&status_bits, direct_status, sizeof(status_bits), cudaMemcpyDeviceToHost);
  for (void *pointer : out_pointers) cudaFree(pointer);
  cudaFree(direct_workspace);
  cudaFree(direct_status);
  cudaStreamDestroy(stream);
  if (rc != HYLE_B200_OK) return check(false, c.name + ": the direct call returned " + std::string(hyle_b200_result_string(rc)));
  check(same && status_bits == 0, c.name + ": two submits through the reference's Queue == the direct C-ABI call, byte for byte" + where);
}

// prepare + one submit + wait of a single-input, single-output operator; returns the Completion's status
// and the output bytes.
static Status submit_once(Fixture &fixture, const Operation &operation, std::vector<Tensor> &inputs, std::vector<Tensor> &outputs) {
  std::vector<ConstTensorView> in_views;
  std::vector<TensorView> out_views;
  for (auto &t : inputs) in_views.push_back(t.view.as_const());
  for (auto &t : outputs) out_views.push_back(t.view);
  auto prepared = prepare(fixture.context, operation, std::span<const ConstTensorView>(in_views),
                          std::span<const TensorView>(out_views), fixture.memory.ref());
  if (!prepared) return prepared.error();
  auto invocation = prepared->create_invocation();
  if (!invocation) return invocation.error();
  auto done = invocation->submit(fixture.queue, in_views, out_views);
  if (!done) return done.error();
  return done->wait();
}

int main() {
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
    std::printf("no CUDA device: the hot path needs a GPU\n");
    return 77;
  }
  auto provider = b200::make_provider<backend::Cuda12Backend>();
  check(provider.has_value(), "make_custom_provider(identity, b200 CUDA-12 backend id, Factory)");
  if (!provider) return 1;
  auto device = backend::device(0);
  check(device.has_value(), "backend::device(0)");
  if (!device) return 1;
  auto context = Context::create(*device, std::move(*provider));
  check(context.has_value(), "Context::create on the CUDA-12 backend with hyle-b200 as the only provider");
  if (!context) {
    std::printf("  %s\n", std::string(context.error().message()).c_str());
    return 1;
  }
  auto memory = backend::DeviceMemory::create(*context);
  auto queue = context->create_queue();
  check(memory.has_value() && queue.has_value(), "DeviceMemory resource and a Queue (one non-default stream)");
  if (!memory || !queue) return 1;
  Fixture fixture{std::move(*context), std::move(*memory), std::move(*queue)};

  const std::array<std::int32_t, 1> last_axis{-1};
  std::vector<Case> cases;
  {  // Unary
    const auto x = dense(DataType::kFloat32, {37, 1000});
    cases.push_back({"Unary{kTanh} f32 [37,1000]", Operation(Unary{UnaryKind::kTanh}), {x}, {x}, {f32_normal(37000, 1)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_unary(s, HYLE_B200_UNARY_TANH, HYLE_B200_F32, in[0], out[0], 37000);
                     }, b200::Entry::kUnary});
  }
  {  // strided inputs: gathered into the workspace by hyle_b200_strided_cast, then the dense kernel
    const auto turned = dense(DataType::kFloat32, {37, 1000}).transposed().value();  // [1000,37], strides {4, 4000}
    const auto upright = dense(DataType::kFloat32, {1000, 37});
    cases.push_back({"Unary{kTanh} f32 on a transposed view [1000,37]", Operation(Unary{UnaryKind::kTanh}), {turned}, {upright},
                     {f32_normal(37000, 48)}, 37000 * 4,
                     [](auto s, auto in, auto out, void *ws, std::uint64_t, std::uint32_t *) {
                       const std::int64_t dims[2] = {1000, 37}, strides[2] = {4, 4000};
                       const int rc = hyle_b200_strided_cast(s, HYLE_B200_F32, HYLE_B200_F32, in[0], ws, 2, dims, strides);
                       return rc != HYLE_B200_OK ? rc : hyle_b200_unary(s, HYLE_B200_UNARY_TANH, HYLE_B200_F32, ws, out[0], 37000);
                     }, b200::Entry::kUnary});
    const std::int64_t slice_dims[2] = {64, 2048}, slice_strides[2] = {2 * 3072, 2};
    const auto slice = TensorDesc::strided_bytes(DataType::kBFloat16, slice_dims, slice_strides).value();  // columns 0..2047 of [64,3072]
    const auto rows = dense(DataType::kBFloat16, {64, 2048}), w = dense(DataType::kBFloat16, {2048});
    cases.push_back({"RmsNorm bf16 on a column slice [64,2048] of [64,3072]", Operation(RmsNorm{.epsilon = 1e-6F}), {slice, w}, {rows},
                     {bf16_normal(slice.required_bytes().value() / 2, 49), bf16_normal(2048, 50)}, 64 * 2048 * 2,
                     [](auto s, auto in, auto out, void *ws, std::uint64_t, std::uint32_t *) {
                       const std::int64_t dims[2] = {64, 2048}, strides[2] = {2 * 3072, 2};
                       const int rc = hyle_b200_strided_cast(s, HYLE_B200_BF16, HYLE_B200_BF16, in[0], ws, 2, dims, strides);
                       return rc != HYLE_B200_OK ? rc : hyle_b200_rms_norm_bf16(s, ws, in[1], HYLE_B200_BF16, out[0], 64, 2048, 1e-6F);
                     }, b200::Entry::kRmsNorm});
  }
  {  // Binary under the NumPy rule: a column vector on the right, gathered with a zero stride
    const auto a = dense(DataType::kFloat32, {64, 4096}), column = dense(DataType::kFloat32, {64, 1});
    cases.push_back({"Binary{kMultiply} f32 [64,4096] * [64,1]", Operation(Binary{BinaryKind::kMultiply}), {a, column}, {a},
                     {f32_normal(64 * 4096, 51), f32_normal(64, 52)}, 64 * 4096 * 4,
                     [](auto s, auto in, auto out, void *ws, std::uint64_t, std::uint32_t *) {
                       const std::int64_t dims[2] = {64, 4096}, strides[2] = {4, 0};
                       const int rc = hyle_b200_strided_cast(s, HYLE_B200_F32, HYLE_B200_F32, in[1], ws, 2, dims, strides);
                       return rc != HYLE_B200_OK ? rc
                                                 : hyle_b200_binary(s, HYLE_B200_BINARY_MULTIPLY, HYLE_B200_F32, in[0], ws, out[0], 64 * 4096, 64 * 4096);
                     }, b200::Entry::kBinary});
  }
  {  // Binary with a trailing-axis broadcast
    const auto a = dense(DataType::kFloat32, {64, 4096}), b = dense(DataType::kFloat32, {4096});
    cases.push_back({"Binary{kAdd} f32 [64,4096] + [4096]", Operation(Binary{BinaryKind::kAdd}), {a, b}, {a},
                     {f32_normal(64 * 4096, 2), f32_normal(4096, 3)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_binary(s, HYLE_B200_BINARY_ADD, HYLE_B200_F32, in[0], in[1], out[0], 64 * 4096, 4096);
                     }, b200::Entry::kBinary});
  }
  {  // Select
    const auto m = dense(DataType::kBool, {64, 4096}), a = dense(DataType::kFloat32, {64, 4096}), b = dense(DataType::kFloat32, {4096});
    cases.push_back({"Select f32, when_false broadcast", Operation(Select{}), {m, a, b}, {a},
                     {bool_random(64 * 4096, 4), f32_normal(64 * 4096, 5), f32_normal(4096, 6)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_select(s, HYLE_B200_F32, in[0], in[1], in[2], out[0], 64 * 4096, 64 * 4096, 4096);
                     }, b200::Entry::kSelect});
  }
  {  // Reduce over the last axis
    const auto a = dense(DataType::kFloat32, {64, 4096}), r = dense(DataType::kFloat32, {64});
    cases.push_back({"Reduce{kMaximum, axes={-1}} f32", Operation(Reduce{.kind = ReductionKind::kMaximum, .axes = Axes::from(last_axis).value()}),
                     {a}, {r}, {f32_normal(64 * 4096, 7)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_reduce_rows_f32(s, HYLE_B200_REDUCE_MAXIMUM, static_cast<const float *>(in[0]),
                                                        static_cast<float *>(out[0]), 64, 4096);
                     }, b200::Entry::kReduceRows});
    const auto h = dense(DataType::kFloat16, {64, 4096}), hr = dense(DataType::kFloat16, {64});
    cases.push_back({"Reduce{kMinimum, axes={-1}} f16",
                     Operation(Reduce{.kind = ReductionKind::kMinimum, .axes = Axes::from(last_axis).value(), .accumulation_type = DataType::kFloat32}),
                     {h}, {hr}, {f16_normal(64 * 4096, 47)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_reduce_rows_extremum(s, HYLE_B200_REDUCE_MINIMUM, HYLE_B200_F16, in[0], out[0], 64, 4096);
                     }, b200::Entry::kReduceRows});
  }
  {  // Scan f32
    const auto a = dense(DataType::kFloat32, {16, 5000});
    cases.push_back({"Scan{axis=-1} f32 [16,5000]", Operation(Scan{.axis = -1, .exclusive = false}), {a}, {a}, {f32_normal(80000, 8)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *status) {
                       return hyle_b200_scan(s, HYLE_B200_F32, in[0], out[0], 16, 5000, 0, status);
                     }, b200::Entry::kScan});
  }
  {  // RmsNorm and LayerNorm
    const auto x = dense(DataType::kBFloat16, {64, 2048}), w = dense(DataType::kBFloat16, {2048});
    cases.push_back({"RmsNorm bf16 [64,2048], bf16 weight", Operation(RmsNorm{.epsilon = 1e-6F}), {x, w}, {x},
                     {bf16_normal(64 * 2048, 9), bf16_normal(2048, 10)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_rms_norm_bf16(s, in[0], in[1], HYLE_B200_BF16, out[0], 64, 2048, 1e-6F);
                     }, b200::Entry::kRmsNorm});
    const auto xh = dense(DataType::kFloat16, {64, 2048}), xf = dense(DataType::kFloat32, {24, 5000});
    cases.push_back({"RmsNorm f16 [64,2048], f32 weight", Operation(RmsNorm{.epsilon = 1e-6F}), {xh, dense(DataType::kFloat32, {2048})}, {xh},
                     {f16_normal(64 * 2048, 43), f32_normal(2048, 44)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_rms_norm(s, HYLE_B200_F16, in[0], in[1], HYLE_B200_F32, out[0], 64, 2048, 1e-6F);
                     }, b200::Entry::kRmsNorm});
    cases.push_back({"RmsNorm f32 [24,5000], f32 weight", Operation(RmsNorm{.epsilon = 1e-6F}), {xf, dense(DataType::kFloat32, {5000})}, {xf},
                     {f32_normal(24 * 5000, 45), f32_normal(5000, 46)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_rms_norm(s, HYLE_B200_F32, in[0], in[1], HYLE_B200_F32, out[0], 24, 5000, 1e-6F);
                     }, b200::Entry::kRmsNorm});
    cases.push_back({"LayerNorm bf16 [64,2048], scale and bias", Operation(LayerNorm{.epsilon = 1e-5F}), {x, w, w}, {x},
                     {bf16_normal(64 * 2048, 11), bf16_normal(2048, 12), bf16_normal(2048, 13)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_layer_norm_bf16(s, in[0], in[1], in[2], out[0], 64, 2048, 1e-5F);
                     }, b200::Entry::kLayerNorm});
  }
  {  // GatedActivation, packed halves
    const auto packed = dense(DataType::kBFloat16, {32, 12288}), out = dense(DataType::kBFloat16, {32, 6144});
    cases.push_back({"GatedActivation{kSilu, kPackedHalves} bf16 [32,12288]",
                     Operation(GatedActivation{GatedActivationKind::kSilu, GatedInputKind::kPackedHalves}), {packed}, {out},
                     {bf16_normal(32 * 12288, 14, 1.5f)}, 0,
                     [](auto s, auto in, auto out_, void *, std::uint64_t, std::uint32_t *) {
                       const auto *gate = static_cast<const std::uint16_t *>(in[0]);
                       return hyle_b200_swiglu_bf16(s, gate, gate + 6144, out_[0], 32, 6144, 12288, 12288);
                     }, b200::Entry::kSwiglu});
  }
  {  // Softmax f32: 72 rows with the caller's workspace -> the streaming kernel
    const auto x = dense(DataType::kFloat32, {72, 4096});
    cases.push_back({"Softmax{axis=-1} f32 [72,4096] (streaming kernel, workspace)", Operation(Softmax{}), {x}, {x},
                     {f32_normal(72 * 4096, 15, 4.0f)}, hyle_b200_logits_workspace_bytes(72, 4096),
                     [](auto s, auto in, auto out, void *ws, std::uint64_t ws_bytes, std::uint32_t *status) {
                       return hyle_b200_softmax_f32(s, HYLE_B200_SOFTMAX, static_cast<const float *>(in[0]), static_cast<float *>(out[0]),
                                                    72, 4096, ws, ws_bytes, status);
                     }, b200::Entry::kSoftmax});
  }
  {  // masked, scaled Softmax on f16 scores
    const auto x = dense(DataType::kFloat16, {4, 128, 1024}), m = dense(DataType::kBool, {128, 1024});
    Bytes mask = bool_random(128 * 1024, 16);
    for (std::size_t row = 0; row < 128; ++row) mask[row * 1024] = std::byte{1};  // no fully masked row
    cases.push_back({"Softmax{scale, Boolean mask} f16 [4,128,1024]", Operation(Softmax{.scale = 0.125F, .mask = MaskKind::kBoolean}),
                     {x, m}, {x}, {f16_normal(4 * 128 * 1024, 17, 3.0f), mask}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_masked_softmax_f16(s, in[0], static_cast<const unsigned char *>(in[1]), 128 * 1024, 0.125F,
                                                           out[0], 4 * 128, 1024);
                     }, b200::Entry::kMaskedSoftmax});
    Bytes addends = f16_normal(128 * 1024, 41, 2.0f);
    for (std::size_t i = 0; i < 128 * 1024; i += 3)  // a third of the positions masked outright, never a row's first
      if (i % 1024 != 0) addends[2 * i] = std::byte{0x00}, addends[2 * i + 1] = std::byte{0xfc};
    cases.push_back({"Softmax{scale, additive mask} f16 [4,128,1024]", Operation(Softmax{.scale = 0.125F, .mask = MaskKind::kAdditive}),
                     {x, dense(DataType::kFloat16, {128, 1024})}, {x}, {f16_normal(4 * 128 * 1024, 42, 3.0f), addends}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_additive_masked_softmax_f16(s, in[0], in[1], 128 * 1024, 0.125F, out[0], 4 * 128, 1024);
                     }, b200::Entry::kMaskedSoftmax});
  }
  {  // Cast and TopK{1}
    const auto x = dense(DataType::kFloat32, {16, 40000});
    cases.push_back({"Cast{f32 -> bf16} [16,40000]", Operation(Cast{DataType::kBFloat16}), {x}, {dense(DataType::kBFloat16, {16, 40000})},
                     {f32_normal(640000, 18)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_cast(s, HYLE_B200_F32, HYLE_B200_BF16, in[0], out[0], 640000);
                     }, b200::Entry::kCast});
    cases.push_back({"TopK{count=1} f32 [16,40000]", Operation(TopK{.count = 1}), {x},
                     {dense(DataType::kFloat32, {16, 1}), dense(DataType::kInt32, {16, 1})}, {f32_normal(640000, 19, 4.0f)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_logits_reduce_f32(s, static_cast<const float *>(in[0]), 16, 40000, nullptr, nullptr,
                                                          static_cast<std::int32_t *>(out[1]), static_cast<float *>(out[0]), nullptr, 0, nullptr);
                     }, b200::Entry::kArgmax});
  }
  {  // cache encoders
    const auto w = dense(DataType::kBFloat16, {64, 8192});
    cases.push_back({"CacheEncode{q8_0} bf16 [64,8192]", Operation::custom(model_ops::CacheEncode{CacheStorage::q8_0().value()}), {w},
                     {dense(DataType::kUInt8, {64, 8704})}, {bf16_normal(64 * 8192, 20, 0.02f)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *status) {
                       return hyle_b200_q8_0_encode(s, HYLE_B200_BF16, in[0], 64 * 8192, out[0], status);
                     }, b200::Entry::kQ8Encode});
    cases.push_back({"CacheEncode{float8(0.25)} bf16 [64,8192]", Operation::custom(model_ops::CacheEncode{CacheStorage::float8(0.25F).value()}),
                     {w}, {dense(DataType::kFloat8E4M3FN, {64, 8192})}, {bf16_normal(64 * 8192, 21)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *status) {
                       return hyle_b200_fp8_e4m3_encode(s, HYLE_B200_BF16, in[0], 64 * 8192, 0.25F, out[0], status);
                     }, b200::Entry::kFp8Encode});
  }
  {  // sampling
    const auto ids = dense(DataType::kUInt32, {16, 4}), logits = dense(DataType::kFloat32, {16, 40000});
    cases.push_back({"sampling_ops::RandomBits{8}", Operation::custom(sampling_ops::RandomBits{8}), {ids}, {dense(DataType::kUInt32, {16, 8})},
                     {u32_random(64, 22)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_random_bits(s, static_cast<const std::uint32_t *>(in[0]), 16, 8, static_cast<std::uint32_t *>(out[0]));
                     }, b200::Entry::kRandomBits});
    cases.push_back({"sampling_ops::Categorical{log probability} f32 [16,40000]", Operation::custom(sampling_ops::Categorical{true}),
                     {logits, ids}, {dense(DataType::kInt32, {16}), dense(DataType::kFloat32, {16})},
                     {f32_normal(640000, 23, 2.0f), u32_random(64, 24)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *status) {
                       return hyle_b200_categorical(s, HYLE_B200_F32, in[0], static_cast<const std::uint32_t *>(in[1]), 16, 40000,
                                                    static_cast<std::int32_t *>(out[0]), static_cast<float *>(out[1]), status);
                     }, b200::Entry::kCategorical});
  }
  {  // the fused custom operators
    const auto x = dense(DataType::kBFloat16, {64, 2048}), w = dense(DataType::kBFloat16, {2048});
    cases.push_back({"custom b200-add-rms-norm", Operation::custom(b200::FusedAddRmsNorm{.epsilon = 1e-6F}), {x, x, w}, {x, x},
                     {bf16_normal(64 * 2048, 25), bf16_normal(64 * 2048, 26), bf16_normal(2048, 27)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_add_rms_norm_bf16(s, in[0], in[1], in[2], HYLE_B200_BF16, out[0], out[1], 64, 2048, 1e-6F);
                     }, b200::Entry::kAddRmsNorm});
    const auto a = dense(DataType::kFloat32, {64, 4096}), bias = dense(DataType::kFloat32, {4096}), rows = dense(DataType::kFloat32, {64});
    cases.push_back({"custom b200-bias-row-sum-max", Operation::custom(b200::BiasRowSumMax{}), {a, bias}, {a, rows, rows},
                     {f32_normal(64 * 4096, 28), f32_normal(4096, 29)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_add_bias_row_sum_max_f32(s, static_cast<const float *>(in[0]), static_cast<const float *>(in[1]),
                                                                 static_cast<float *>(out[0]), static_cast<float *>(out[1]),
                                                                 static_cast<float *>(out[2]), 64, 4096);
                     }, b200::Entry::kBiasRowSumMax});
    const auto logits = dense(DataType::kFloat32, {72, 19456});
    cases.push_back({"custom b200-logits-reduce [72,19456] (streaming kernel, workspace)", Operation::custom(b200::LogitsReduce{}), {logits},
                     {dense(DataType::kFloat32, {72}), dense(DataType::kBFloat16, {72, 19456}), dense(DataType::kInt32, {72}),
                      dense(DataType::kFloat32, {72})},
                     {f32_normal(72 * 19456, 30, 4.0f)}, hyle_b200_logits_workspace_bytes(72, 19456),
                     [](auto s, auto in, auto out, void *ws, std::uint64_t ws_bytes, std::uint32_t *status) {
                       return hyle_b200_logits_reduce_f32(s, static_cast<const float *>(in[0]), 72, 19456, static_cast<float *>(out[0]), out[1],
                                                          static_cast<std::int32_t *>(out[2]), static_cast<float *>(out[3]), ws, ws_bytes, status);
                     }, b200::Entry::kLogitsReduce});
    const auto weights = dense(DataType::kBFloat16, {1024, 8192});
    cases.push_back({"custom b200-q8_0-roundtrip [1024,8192] (workspace)", Operation::custom(b200::Q8_0Roundtrip{}), {weights},
                     {dense(DataType::kUInt8, {1024, 8704}), weights, dense(DataType::kFloat64, {1})},
                     {bf16_normal(1024 * 8192, 31, 0.02f)}, hyle_b200_sum_squares_workspace_bytes(1024ull * 8192),
                     [](auto s, auto in, auto out, void *ws, std::uint64_t ws_bytes, std::uint32_t *status) {
                       return hyle_b200_q8_0_roundtrip_bf16(s, in[0], 1024ull * 8192, out[0], out[1], static_cast<double *>(out[2]), status, ws,
                                                            ws_bytes);
                     }, b200::Entry::kQ8Roundtrip});
  }
  {  // what the graph regions lower to, and the wider gating domain
    const auto g = dense(DataType::kBFloat16, {32, 6144});
    cases.push_back({"custom b200-activation-multiply{kSilu} bf16 [32,6144]",
                     Operation::custom(b200::ActivationMultiply{.activation = UnaryKind::kSilu}), {g, g}, {g},
                     {bf16_normal(32 * 6144, 40, 1.5f), bf16_normal(32 * 6144, 41, 1.5f)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_gated_activation(s, HYLE_B200_GATE_SILU, HYLE_B200_BF16, 1, in[0], in[1], out[0], 32, 6144, 6144, 6144);
                     }, b200::Entry::kActivationMultiply});
    const auto h = dense(DataType::kFloat16, {32, 6144});
    cases.push_back({"GatedActivation{kGeluTanh, kSeparate} f16 [32,6144]",
                     Operation(GatedActivation{GatedActivationKind::kGeluTanh, GatedInputKind::kSeparate}), {h, h}, {h},
                     {f16_normal(32 * 6144, 42, 1.5f), f16_normal(32 * 6144, 43, 1.5f)}, 0,
                     [](auto s, auto in, auto out, void *, std::uint64_t, std::uint32_t *) {
                       return hyle_b200_gated_activation(s, HYLE_B200_GATE_GELU_TANH, HYLE_B200_F16, 0, in[0], in[1], out[0], 32, 6144, 6144, 6144);
                     }, b200::Entry::kSwiglu});
    const auto logits = dense(DataType::kFloat32, {72, 19456});
    cases.push_back({"custom b200-greedy-head{values} [72,19456] (streaming kernel, workspace)", Operation::custom(b200::GreedyHead{}), {logits},
                     {dense(DataType::kBFloat16, {72, 19456}), dense(DataType::kFloat32, {72, 1}), dense(DataType::kInt32, {72, 1})},
                     {f32_normal(72 * 19456, 44, 4.0f)}, hyle_b200_logits_workspace_bytes(72, 19456),
                     [](auto s, auto in, auto out, void *ws, std::uint64_t ws_bytes, std::uint32_t *status) {
                       return hyle_b200_logits_reduce_f32(s, static_cast<const float *>(in[0]), 72, 19456, nullptr, out[0],
                                                          static_cast<std::int32_t *>(out[2]), static_cast<float *>(out[1]), ws, ws_bytes, status);
                     }, b200::Entry::kGreedyHead});
  }
  for (const auto &c : cases) run_case(fixture, c);
  std::array<bool, b200::kEntryCount> covered{};
  for (const auto &c : cases) covered[static_cast<std::size_t>(c.entry)] = true;
  bool all = true;
  for (bool one : covered) all = all && one;
  check(all, "every Entry of the adapter (" + std::to_string(b200::kEntryCount) + ") ran through submit()");

  // ---- the error protocol: device status word -> the Completion's terminal status ------------------------------------------
  const auto resource = fixture.memory.ref();
  {  // Q8_0 encode of a NaN: InvalidArgument (src/compute_provider_ggml/ggml_cpu_provider.cc:1720-1721), the block zeroed
    const auto w = dense(DataType::kBFloat16, {8, 256});
    std::vector<std::uint16_t> values(8 * 256, bf16(1.0f));
    values[19] = 0x7FC0;  // NaN
    std::vector<Tensor> in, out;
    in.emplace_back(w, resource);
    out.emplace_back(dense(DataType::kUInt8, {8, 272}), resource);
    in[0].write(bytes_of(values)).IgnoreError();
    const Status status = submit_once(fixture, Operation::custom(model_ops::CacheEncode{CacheStorage::q8_0().value()}), in, out);
    const Bytes carrier = out[0].read();
    bool zeroed = true;
    for (std::size_t i = 0; i < 34; ++i) zeroed = zeroed && carrier[i] == std::byte{0};
    check(status.IsInvalidArgument() && zeroed && carrier[34 + 2] != std::byte{0},
          "CacheEncode{q8_0} with a NaN completes with Status::InvalidArgument; its block is zero bytes, the others are encoded");
    // the next sequence on the same Queue starts from a clean status word
    values[19] = bf16(1.0f);
    in[0].write(bytes_of(values)).IgnoreError();
    check(submit_once(fixture, Operation::custom(model_ops::CacheEncode{CacheStorage::q8_0().value()}), in, out).ok(),
          "the following sequence on the same Queue completes OK (the status word is per sequence)");
  }
  {  // FP8 encode of an infinity
    const auto w = dense(DataType::kFloat32, {4, 64});
    std::vector<float> values(256, 0.5f);
    values[100] = std::numeric_limits<float>::infinity();
    std::vector<Tensor> in, out;
    in.emplace_back(w, resource);
    out.emplace_back(dense(DataType::kFloat8E4M3FN, {4, 64}), resource);
    in[0].write(bytes_of(values)).IgnoreError();
    check(submit_once(fixture, Operation::custom(model_ops::CacheEncode{CacheStorage::float8(1.0F).value()}), in, out).IsInvalidArgument(),
          "CacheEncode{float8} with an infinity completes with Status::InvalidArgument");
  }
  {  // Categorical with a NaN row
    std::vector<float> weights(4 * 1000, 0.0f);
    weights[2 * 1000 + 5] = std::numeric_limits<float>::quiet_NaN();
    std::vector<Tensor> in, out;
    in.emplace_back(dense(DataType::kFloat32, {4, 1000}), resource);
    in.emplace_back(dense(DataType::kUInt32, {4, 4}), resource);
    out.emplace_back(dense(DataType::kInt32, {4}), resource);
    in[0].write(bytes_of(weights)).IgnoreError();
    in[1].write(u32_random(16, 40)).IgnoreError();
    const Status status = submit_once(fixture, Operation::custom(sampling_ops::Categorical{false}), in, out);
    const Bytes drawn = out[0].read();
    std::int32_t index[4];
    std::memcpy(index, drawn.data(), sizeof(index));
    check(status.IsInvalidArgument() && index[2] == -1 && index[0] >= 0 && index[0] < 1000,
          "Categorical with a NaN row completes with Status::InvalidArgument; that row's index is -1");
  }
  {  // checked i32 Scan: overflow -> OutOfRange and nothing written; a fitting scan -> exact prefix sums
    const auto x = dense(DataType::kInt32, {3, 64});
    std::vector<std::int32_t> values(3 * 64, 1);
    values[64 + 10] = std::numeric_limits<std::int32_t>::max();
    std::vector<Tensor> in, out;
    in.emplace_back(x, resource);
    out.emplace_back(x, resource);
    in[0].write(bytes_of(values)).IgnoreError();
    out[0].storage.view().fill(kCanary).IgnoreError();
    const Status overflow = submit_once(fixture, Operation(Scan{}), in, out);
    Bytes after = out[0].read();
    bool untouched = true;
    for (std::byte b : after) untouched = untouched && b == kCanary;
    check(overflow.IsOutOfRange() && untouched, "Scan i32 whose prefix leaves int32 completes with Status::OutOfRange and writes nothing");
    values[64 + 10] = 1;
    in[0].write(bytes_of(values)).IgnoreError();
    const Status fits = submit_once(fixture, Operation(Scan{}), in, out);
    after = out[0].read();
    std::int32_t sums[3 * 64];
    std::memcpy(sums, after.data(), sizeof(sums));
    check(fits.ok() && sums[0] == 1 && sums[63] == 64 && sums[64 + 63] == 64 && sums[128 + 31] == 32, "Scan i32 that fits: exact prefix sums");
  }
  {  // backend facts: event-backed Completions, status copies only for sequences that used the word
    auto counters = backend::counters(fixture.queue);
    check(counters.has_value() && counters->event_completions >= 2 * cases.size() && counters->status_copies >= 6 &&
              counters->status_copies < counters->event_completions && counters->slots_created == 16,
          "Queue: one event-backed Completion per sequence, status words copied back only when acquired, no slot growth");
    // copy_async / fill_async on the Queue's stream
    mem::Buffer a = mem::Buffer::create(resource, 4096, 256).value(), b = mem::Buffer::create(resource, 4096, 256).value();
    auto filled = fill_async(fixture.queue, a.view(), std::byte{0x5A});
    auto copied = copy_async(fixture.queue, b.view(), a.view());
    const bool waited = filled.has_value() && copied.has_value() && copied->wait().ok();
    Bytes back(4096);
    b.view().read(back).IgnoreError();
    bool pattern = waited;
    for (std::byte value : back) pattern = pattern && value == std::byte{0x5A};
    check(pattern, "fill_async then copy_async on the Queue: ordered on its stream, one wait covers the prefix");
    // a provider made for this backend is refused by a Context of another backend id
    check(fixture.queue.drain().ok() && fixture.context.drain().ok(), "Queue::drain and Context::drain");
  }
  {  // Two host threads with a Queue each: prepare on the shared Context and submit concurrently (one producer per
     // Queue at a time, different Queues concurrently: samples/package/graph/custom_kernel/cuda_main.cc:157-166;
     // Factory::propose/prepare are const and may run from several threads).  Each lane repeats its operator and
     // must read back, every time, the bytes a single submit gave before the threads started.
    struct Lane final {
      std::string name;
      Operation operation;
      std::vector<TensorDesc> in, out;
      std::vector<Bytes> data;
      std::string error;
      int rounds = 0;
    };
    const auto weights = dense(DataType::kBFloat16, {256, 8192});
    const auto rows = dense(DataType::kFloat32, {72, 19456});
    std::vector<Lane> lanes;
    lanes.push_back({"b200-q8_0-roundtrip (workspace, status word)", Operation::custom(b200::Q8_0Roundtrip{}), {weights},
                     {dense(DataType::kUInt8, {256, 8704}), weights, dense(DataType::kFloat64, {1})},
                     {bf16_normal(256 * 8192, 70, 0.02f)}});
    lanes.push_back({"b200-logits-reduce (streaming kernel, workspace, status word)", Operation::custom(b200::LogitsReduce{}), {rows},
                     {dense(DataType::kFloat32, {72}), dense(DataType::kBFloat16, {72, 19456}), dense(DataType::kInt32, {72}),
                      dense(DataType::kFloat32, {72})},
                     {f32_normal(72 * 19456, 71, 4.0f)}});
    lanes.push_back({"CacheEncode{q8_0} (status word)", Operation::custom(model_ops::CacheEncode{CacheStorage::q8_0().value()}),
                     {dense(DataType::kBFloat16, {64, 8192})}, {dense(DataType::kUInt8, {64, 8704})}, {bf16_normal(64 * 8192, 72)}});
    constexpr int kRounds = 40;
    auto run_lane = [&](Lane &lane, int rounds, std::vector<Bytes> *expected, bool compare) {
      auto own_queue = fixture.context.create_queue();
      if (!own_queue) return void(lane.error = "create_queue");
      std::vector<Tensor> inputs, outputs;
      for (const auto &desc : lane.in) inputs.emplace_back(desc, resource);
      for (const auto &desc : lane.out) outputs.emplace_back(desc, resource);
      for (std::size_t i = 0; i < inputs.size(); ++i)
        if (!inputs[i].write(lane.data[i]).ok()) return void(lane.error = "writing an input");
      std::vector<ConstTensorView> in_views;
      std::vector<TensorView> out_views;
      for (auto &t : inputs) in_views.push_back(t.view.as_const());
      for (auto &t : outputs) out_views.push_back(t.view);
      auto prepared = prepare(fixture.context, lane.operation, std::span<const ConstTensorView>(in_views),
                              std::span<const TensorView>(out_views), resource);
      if (!prepared) return void(lane.error = "prepare: " + std::string(prepared.error().message()));
      const auto requirement = prepared->workspace_requirement();
      mem::Buffer workspace;
      if (requirement.size != 0) {
        workspace = mem::Buffer::create(resource, requirement.size, requirement.alignment).value();
        workspace.view().fill(kPoison).IgnoreError();
      }
      auto invocation = prepared->create_invocation(requirement.size != 0 ? workspace.view() : mem::BufferView{});
      if (!invocation) return void(lane.error = "create_invocation: " + std::string(invocation.error().message()));
      for (int round = 0; round < rounds; ++round) {
        for (auto &t : outputs) t.storage.view().fill(kCanary).IgnoreError();
        auto done = invocation->submit(*own_queue, in_views, out_views);
        if (!done) return void(lane.error = "submit: " + std::string(done.error().message()));
        const Status waited = done->wait();
        if (!waited.ok()) return void(lane.error = "wait: " + std::string(waited.message()));
        for (std::size_t i = 0; i < outputs.size(); ++i) {
          Bytes now = outputs[i].read();
          if (!compare) expected->push_back(std::move(now));
          else if (now != (*expected)[i]) return void(lane.error = "output " + std::to_string(i) + " differs in round " + std::to_string(round));
        }
        ++lane.rounds;
      }
      if (!own_queue->drain().ok()) lane.error = "drain";
    };
    std::vector<std::vector<Bytes>> expected(lanes.size());
    for (std::size_t k = 0; k < lanes.size(); ++k) run_lane(lanes[k], 1, &expected[k], false);
    bool alone = true;
    for (auto &lane : lanes) {
      alone = alone && lane.error.empty();
      lane.rounds = 0;
    }
    if (alone) {
      std::vector<std::thread> threads;
      for (std::size_t k = 0; k < lanes.size(); ++k)
        threads.emplace_back([&, k] { run_lane(lanes[k], kRounds, &expected[k], true); });
      for (auto &thread : threads) thread.join();
    }
    for (const auto &lane : lanes) {
      check(lane.error.empty() && lane.rounds == kRounds,
            "concurrent Queues: " + lane.name + ", " + std::to_string(kRounds) + " submits beside two other host threads, same bytes every time" +
                (lane.error.empty() ? "" : " [" + lane.error + "]"));
    }
  }
  {  // what the seam costs on the host: submit() of a prepared invocation against the bare C-ABI call
    const auto x = dense(DataType::kFloat32, {1, 1024});
    std::vector<Tensor> in, out;
    in.emplace_back(x, resource);
    out.emplace_back(x, resource);
    in[0].write(f32_normal(1024, 60)).IgnoreError();
    std::vector<ConstTensorView> in_views{in[0].view.as_const()};
    std::vector<TensorView> out_views{out[0].view};
    auto prepared = prepare(fixture.context, Operation(Unary{UnaryKind::kExp}), std::span<const ConstTensorView>(in_views),
                            std::span<const TensorView>(out_views), resource);
    // an invocation carries one flight at a time: eight of them take turns
    std::vector<OperationInvocation> invocations;
    bool timed = prepared.has_value();
    for (int k = 0; k < 8 && timed; ++k) {
      auto made = prepared->create_invocation();
      timed = made.has_value();
      if (timed) invocations.push_back(std::move(*made));
    }
    constexpr int kSubmits = 2000;
    double through_seam = 0.0, direct = 0.0;
    if (timed) {
      // their Completions are kept in a ring: the one replaced finished seven launches ago, so waiting for it
      // returns at once and the loop measures the producer side
      std::vector<Completion> ring(8);
      std::vector<bool> flown(8, false);
      auto submit_one = [&](int i) {
        const std::size_t turn = static_cast<std::size_t>(i) % ring.size();
        if (flown[turn] && !ring[turn].wait().ok()) return false;
        flown[turn] = true;
        auto done = invocations[turn].submit(fixture.queue, in_views, out_views);
        if (!done) {
          std::printf("      submit %d: %s\n", i, std::string(done.error().message()).c_str());
          return false;
        }
        ring[turn] = std::move(*done);
        return true;
      };
      for (int i = 0; i < 100 && timed; ++i) timed = submit_one(i);
      timed = timed && fixture.queue.drain().ok();
      auto t0 = std::chrono::steady_clock::now();
      for (int i = 0; i < kSubmits && timed; ++i) timed = submit_one(i);
      auto t1 = std::chrono::steady_clock::now();
      timed = timed && fixture.queue.drain().ok();
      through_seam = std::chrono::duration<double, std::micro>(t1 - t0).count() / kSubmits;
      auto stream = backend::stream(fixture.queue);
      if (stream) {
        t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < kSubmits; ++i) hyle_b200_unary(*stream, HYLE_B200_UNARY_EXP, HYLE_B200_F32, in[0].device(), out_pointer(out[0]), 1024);
        t1 = std::chrono::steady_clock::now();
        cudaDeviceSynchronize();
        direct = std::chrono::duration<double, std::micro>(t1 - t0).count() / kSubmits;
      }
    }
    check(timed, "2000 submits of a prepared operator (eight invocations in turn) on the Queue, then 2000 direct calls on its stream");
    std::printf("      host cost per operator: %.2f us through OperationInvocation::submit (sequence, Completion, enqueue), "
                "%.2f us for the bare hyle_b200_unary call\n", through_seam, direct);
  }
  std::printf("%d check(s), %d failure(s)\n", checks, failures);
  return failures == 0 ? 0 : 1;
}

// Implementation of the thin CUDA-12 backend (see b200_backend.h).  Same-build component of the
// reference's compute core: it fills detail::BackendVTable (src/compute/backend_internal.h:14-67) and
// reaches the backend queue of an admitted sequence through detail::ContextAccess
// (src/compute/context_state.h), exactly as the reference's CUDA backend does
// (src/compute_backend_cuda/cuda_backend.cc:1849-1858).
#include "b200_backend.h"

#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>
#include <utility>
#include <vector>

#include <cuda_runtime_api.h>

#include "backend_internal.h"
#include "completion_internal.h"
#include "context_state.h"

namespace hyle::compute::b200::backend {
namespace {

using compute::detail::EnqueueResult;

constexpr std::size_t kAllocationAlignment = 256;  // what cudaMalloc guarantees; cuda_internal.h:27
constexpr std::size_t kSlotsPerBlock = 16;

Status runtime_status(cudaError_t error) noexcept {
  if (error == cudaSuccess) return Status::Ok();
  const char *text = cudaGetErrorString(error);
  const NativeError native{.domain = NativeErrorDomain::CudaRuntime, .code = static_cast<std::int64_t>(error)};
  switch (error) {
    case cudaErrorInvalidValue: return Status::FromNative(StatusCode::InvalidArgument, native, text);
    case cudaErrorMemoryAllocation: return Status::FromNative(StatusCode::ResourceExhausted, native, text);
    case cudaErrorNotSupported: return Status::FromNative(StatusCode::Unimplemented, native, text);
    case cudaErrorNotReady: return Status::FromNative(StatusCode::Unavailable, native, text);
    default: return Status::FromNative(StatusCode::Internal, native, text);
  }
}

struct BackendPayload final {};
struct DevicePayload final {
  std::int32_t ordinal = -1;
};

struct ContextState final {
  int ordinal = -1;
};

// Binds the context's device to the calling thread for the scope (the runtime's current device is
// per thread, and a Queue may be used from any thread).
struct DeviceScope final {
  explicit DeviceScope(int ordinal) noexcept {
    if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
    if (previous != ordinal) status = cudaSetDevice(ordinal);
    else previous = -1;
  }
  ~DeviceScope() {
    if (previous >= 0) cudaSetDevice(previous);
  }
  cudaError_t status = cudaSuccess;
  int previous = -1;
};

struct QueueState;

// One sequence's completion state: an event and a status word pair.  Owned by its Queue; handed out
// by begin_sequence and returned when the Completion that wraps it is destroyed.
struct Slot final {
  QueueState *owner = nullptr;
  cudaEvent_t event = nullptr;
  unsigned *device_status = nullptr;
  unsigned *host_status = nullptr;   // pinned
  bool status_used = false;
  bool status_copied = false;
  bool report_status = false;
  bool recorded = false;             // an event covers the sequence (else: the stream is drained to wait)
  bool retired = false;
  Status terminal{};
};

struct StatusBlock final {
  unsigned *device = nullptr;
  unsigned *host = nullptr;
};

struct QueueState final {
  ContextState *context = nullptr;
  cudaStream_t stream = nullptr;
  std::atomic<std::uint32_t> references{1};
  std::mutex mutex;                   // guards the slot lists and counters (Completions retire on any thread)
  std::vector<Slot *> free_slots;
  std::vector<Slot *> all_slots;
  std::vector<StatusBlock> blocks;
  Slot *active_sequence = nullptr;    // producer-side only
  Counters counters{};

  void incref() noexcept { references.fetch_add(1, std::memory_order_relaxed); }
  void decref() noexcept {
    if (references.fetch_sub(1, std::memory_order_acq_rel) == 1) destroy();
  }

  // Creates kSlotsPerBlock more slots (cold: an event each, one device and one pinned word block).
  Status grow() noexcept {
    DeviceScope scope(context->ordinal);
    if (scope.status != cudaSuccess) return runtime_status(scope.status);
    StatusBlock block{};
    cudaError_t error = cudaMalloc(reinterpret_cast<void **>(&block.device), kSlotsPerBlock * sizeof(unsigned));
    if (error != cudaSuccess) return runtime_status(error);
    error = cudaMallocHost(reinterpret_cast<void **>(&block.host), kSlotsPerBlock * sizeof(unsigned));
    if (error != cudaSuccess) {
      cudaFree(block.device);
      return runtime_status(error);
    }
    std::memset(block.host, 0, kSlotsPerBlock * sizeof(unsigned));
    blocks.push_back(block);
    for (std::size_t i = 0; i < kSlotsPerBlock; ++i) {
      auto *slot = new (std::nothrow) Slot{};
      if (slot == nullptr) return Status::ResourceExhausted("b200 backend: completion slot allocation failed");
      error = cudaEventCreateWithFlags(&slot->event, cudaEventDisableTiming);
      if (error != cudaSuccess) {
        delete slot;
        return runtime_status(error);
      }
      slot->owner = this;
      slot->device_status = block.device + i;
      slot->host_status = block.host + i;
      all_slots.push_back(slot);
      free_slots.push_back(slot);
      ++counters.slots_created;
    }
    return Status::Ok();
  }

  Result<Slot *> acquire() noexcept {
    std::lock_guard lock(mutex);
    if (free_slots.empty()) {
      Status grown = grow();
      if (!grown.ok()) return std::unexpected(std::move(grown));
    }
    Slot *slot = free_slots.back();
    free_slots.pop_back();
    slot->status_used = slot->status_copied = slot->report_status = slot->recorded = slot->retired = false;
    slot->terminal = Status::Ok();
    *slot->host_status = 0;
    return slot;
  }

  void release(Slot *slot) noexcept {
    std::lock_guard lock(mutex);
    free_slots.push_back(slot);
  }

  void destroy() noexcept {
    DeviceScope scope(context->ordinal);
    if (stream != nullptr) {
      cudaStreamSynchronize(stream);
      cudaStreamDestroy(stream);
    }
    for (Slot *slot : all_slots) {
      if (slot->event != nullptr) cudaEventDestroy(slot->event);
      delete slot;
    }
    for (const StatusBlock &block : blocks) {
      cudaFree(block.device);
      cudaFreeHost(block.host);
    }
    delete this;
  }
};

// ---- Completion ----------------------------------------------------------------------------------------------------
// Observes the slot once: nullopt while the work is still running.
Result<CompletionPoll> observe(Slot *slot, bool wait) noexcept {
  if (slot == nullptr || slot->owner == nullptr)
    return std::unexpected(Status::Internal("b200 backend: completion slot is invalid"));
  if (!slot->retired) {
    cudaError_t result;
    if (slot->recorded) {
      result = wait ? cudaEventSynchronize(slot->event) : cudaEventQuery(slot->event);
    } else {
      // the event could not be recorded: fall back to the whole stream, as the reference does
      result = wait ? cudaStreamSynchronize(slot->owner->stream) : cudaStreamQuery(slot->owner->stream);
    }
    if (result == cudaErrorNotReady) return CompletionPoll::kPending;
    slot->retired = true;
    if (result != cudaSuccess) {
      slot->terminal = runtime_status(result);  // an asynchronous CUDA failure outranks a software diagnostic
    } else if (slot->status_copied && slot->report_status) {
      slot->terminal.Update(status_from_bits(*slot->host_status));
    }
  }
  if (!slot->terminal.ok()) return std::unexpected(slot->terminal);
  return CompletionPoll::kComplete;
}

Result<CompletionPoll> completion_poll(void *state) noexcept { return observe(static_cast<Slot *>(state), false); }

Status completion_wait(void *state) noexcept {
  auto result = observe(static_cast<Slot *>(state), true);
  if (result) return Status::Ok();
  return std::move(result).error();
}

Status completion_cancel(void *) noexcept {
  return Status::Unimplemented("CUDA work cannot be preemptively cancelled");
}

// The public handle is gone (after wait/poll settled it, or abandoned).  Borrowed execution state may
// be released only after the work has terminated, so an unretired slot is waited for here: this
// backend has no reaper thread, abandoning a pending Completion blocks its destructor instead.
void completion_destroy(void *state, compute::detail::CompletionLifetime lifetime, Status terminal_hint) noexcept {
  auto *slot = static_cast<Slot *>(state);
  auto result = observe(slot, true);
  if (!result) terminal_hint.Update(std::move(result).error());
  QueueState *owner = slot->owner;
  if (lifetime.valid()) {
    lifetime.terminal(lifetime.state, terminal_hint);
    lifetime.release(lifetime.state);
  }
  owner->release(slot);
  owner->decref();
}

const compute::detail::CompletionVTable kCompletionVTable{
    .destroy = &completion_destroy,
    .poll = &completion_poll,
    .wait = &completion_wait,
    .request_cancel = &completion_cancel,
};

// ---- device memory ---------------------------------------------------------------------------------------------------
extern const compute::detail::BackendVTable kBackendVTable;

class CudaMallocResource final : public mem::MemoryResource {
public:
  explicit CudaMallocResource(int ordinal) noexcept : ordinal_(ordinal) {}
  std::string_view name() const noexcept override { return "hyle-b200-cuda12-device"; }
  mem::MemoryProperties properties() const noexcept override {
    return mem::MemoryProperties{
        .flags = mem::MemoryProperty::kDeviceAccessible,
        .minimum_alignment = kAllocationAlignment,
        .maximum_allocation = SIZE_MAX,
        .domain = {&kBackendVTable, static_cast<std::uintptr_t>(ordinal_) + 1},
    };
  }
  Result<mem::ResourceAllocation> allocate(std::size_t size, std::size_t alignment) noexcept override {
    if (alignment > kAllocationAlignment)
      return std::unexpected(Status::InvalidArgument("b200 backend: device allocations are 256-byte aligned"));
    DeviceScope scope(ordinal_);
    if (scope.status != cudaSuccess) return std::unexpected(runtime_status(scope.status));
    void *pointer = nullptr;
    // a zero-size Buffer still needs a non-null handle for views to be valid
    const cudaError_t error = cudaMalloc(&pointer, size == 0 ? kAllocationAlignment : size);
    if (error != cudaSuccess) return std::unexpected(runtime_status(error));
    live_.fetch_add(1, std::memory_order_relaxed);
    return mem::ResourceAllocation{.native_handle = pointer, .size = size, .alignment = alignment};
  }
  void deallocate(mem::ResourceAllocation allocation) noexcept override {
    if (allocation.native_handle == nullptr) return;
    DeviceScope scope(ordinal_);
    cudaFree(allocation.native_handle);
    live_.fetch_sub(1, std::memory_order_relaxed);
  }
  // Synchronous range operations (cold paths of tests and loaders): plain cudaMemcpy / cudaMemset.
  Status read(void *handle, std::size_t offset, std::span<std::byte> destination) noexcept override {
    DeviceScope scope(ordinal_);
    return runtime_status(cudaMemcpy(destination.data(), static_cast<const std::byte *>(handle) + offset,
                                     destination.size(), cudaMemcpyDeviceToHost));
  }
  Status write(void *handle, std::size_t offset, std::span<const std::byte> source) noexcept override {
    DeviceScope scope(ordinal_);
    return runtime_status(cudaMemcpy(static_cast<std::byte *>(handle) + offset, source.data(), source.size(),
                                     cudaMemcpyHostToDevice));
  }
  Status fill(void *handle, std::size_t offset, std::size_t size, std::byte value) noexcept override {
    DeviceScope scope(ordinal_);
    cudaError_t error = cudaMemset(static_cast<std::byte *>(handle) + offset, static_cast<int>(value), size);
    if (error == cudaSuccess) error = cudaDeviceSynchronize();
    return runtime_status(error);
  }
  Status copy(void *destination, std::size_t destination_offset, mem::MemoryResource &source_resource, void *source,
              std::size_t source_offset, std::size_t size) noexcept override {
    if (source_resource.properties().domain != properties().domain)
      return Status::Unimplemented("b200 backend: synchronous copies stay inside one device resource");
    DeviceScope scope(ordinal_);
    return runtime_status(cudaMemcpy(static_cast<std::byte *>(destination) + destination_offset,
                                     static_cast<const std::byte *>(source) + source_offset, size,
                                     cudaMemcpyDeviceToDevice));
  }
  std::size_t live() const noexcept { return live_.load(std::memory_order_relaxed); }
  int ordinal() const noexcept { return ordinal_; }

private:
  int ordinal_;
  std::atomic<std::size_t> live_{0};
};

bool is_device_resource(mem::MemoryResourceRef resource) noexcept {
  return resource.valid() && resource.properties().domain.authority == &kBackendVTable;
}

// ---- backend vtable --------------------------------------------------------------------------------------------------
Result<std::size_t> device_count_impl(const Backend &) noexcept {
  int count = 0;
  const cudaError_t error = cudaGetDeviceCount(&count);
  if (error == cudaErrorNoDevice || error == cudaErrorInsufficientDriver) return std::size_t{0};
  if (error != cudaSuccess) return std::unexpected(runtime_status(error));
  return static_cast<std::size_t>(count);
}

Result<Device> device_impl(const Backend &value, std::size_t index) noexcept {
  auto count = device_count_impl(value);
  if (!count) return std::unexpected(std::move(count).error());
  if (index >= *count) return std::unexpected(Status::OutOfRange("CUDA device index is out of range"));
  return compute::detail::DeviceAccess::make(&kBackendVTable, DevicePayload{static_cast<std::int32_t>(index)});
}

bool same_device_impl(const Device &left, const Device &right) noexcept {
  return compute::detail::DeviceAccess::payload<DevicePayload>(left).ordinal ==
         compute::detail::DeviceAccess::payload<DevicePayload>(right).ordinal;
}

Result<DeviceProperties> properties_impl(const Device &value) noexcept {
  const auto payload = compute::detail::DeviceAccess::payload<DevicePayload>(value);
  if (payload.ordinal < 0) return std::unexpected(Status::NotFound("CUDA device is not available"));
  return DeviceProperties{
      .backend = kBackendId,
      .device_class = DeviceClass::kGpu,
      .backend_name = "b200-cuda12",
      .name = "NVIDIA CUDA device",
      .unified_memory = false,
      .asynchronous_queues = true,
  };
}

Status validate_resource_impl(const Device &value, mem::MemoryResourceRef resource) noexcept {
  if (!resource.valid()) return Status::InvalidArgument("tensor memory resource is invalid");
  const auto payload = compute::detail::DeviceAccess::payload<DevicePayload>(value);
  const auto domain = resource.properties().domain;
  if (domain.authority != &kBackendVTable)
    return Status::FailedPrecondition("b200 backend requires tensor storage from its DeviceMemory resource");
  if (domain.value != static_cast<std::uintptr_t>(payload.ordinal) + 1)
    return Status::FailedPrecondition("tensor storage belongs to another CUDA device");
  return Status::Ok();
}

Status create_context_impl(const Device &value, mem::AllocatorRef, void **output) noexcept {
  if (output == nullptr) return Status::InvalidArgument("CUDA context output is null");
  *output = nullptr;
  const auto payload = compute::detail::DeviceAccess::payload<DevicePayload>(value);
  DeviceScope scope(payload.ordinal);
  if (scope.status != cudaSuccess) return runtime_status(scope.status);
  const cudaError_t error = cudaFree(nullptr);  // creates the primary context now, not in a hot call
  if (error != cudaSuccess) return runtime_status(error);
  auto *state = new (std::nothrow) ContextState{payload.ordinal};
  if (state == nullptr) return Status::ResourceExhausted("b200 backend: context allocation failed");
  *output = state;
  return Status::Ok();
}

void destroy_context_impl(void *context, mem::AllocatorRef) noexcept { delete static_cast<ContextState *>(context); }

Status create_queue_impl(void *context, QueueOptions, mem::AllocatorRef, void **output) noexcept {
  if (output == nullptr) return Status::InvalidArgument("CUDA queue output is null");
  *output = nullptr;
  auto *owner = static_cast<ContextState *>(context);
  DeviceScope scope(owner->ordinal);
  if (scope.status != cudaSuccess) return runtime_status(scope.status);
  auto *queue = new (std::nothrow) QueueState{};
  if (queue == nullptr) return Status::ResourceExhausted("b200 backend: queue allocation failed");
  queue->context = owner;
  cudaError_t error = cudaStreamCreateWithFlags(&queue->stream, cudaStreamNonBlocking);
  if (error != cudaSuccess) {
    delete queue;
    return runtime_status(error);
  }
  Status grown;
  {
    std::lock_guard lock(queue->mutex);
    grown = queue->grow();  // every steady-state sequence then finds a slot without allocating
  }
  if (!grown.ok()) {
    queue->decref();
    return grown;
  }
  *output = queue;
  return Status::Ok();
}

void destroy_queue_impl(void *queue, mem::AllocatorRef) noexcept {
  if (queue != nullptr) static_cast<QueueState *>(queue)->decref();
}

Status begin_sequence_impl(void *queue, void **sequence) noexcept {
  if (sequence == nullptr) return Status::InvalidArgument("CUDA sequence output is null");
  *sequence = nullptr;
  auto *selected = static_cast<QueueState *>(queue);
  if (selected->active_sequence != nullptr) return Status::FailedPrecondition("CUDA sequence is already active");
  auto slot = selected->acquire();
  if (!slot) return std::move(slot).error();
  *sequence = *slot;
  selected->active_sequence = *slot;
  return Status::Ok();
}

Completion finish_sequence_impl(void *queue, void *sequence, bool accepted, Status terminal) noexcept {
  auto *queue_state = static_cast<QueueState *>(queue);
  auto *slot = static_cast<Slot *>(sequence);
  if (slot == nullptr || slot->owner != queue_state)
    return Completion::completed(Status::Internal("CUDA sequence slot does not belong to queue"));
  queue_state->active_sequence = nullptr;
  if (!accepted) {  // nothing was recorded: no event, inline terminal state
    queue_state->release(slot);
    return Completion::completed(std::move(terminal));
  }
  DeviceScope scope(queue_state->context->ordinal);
  if (slot->status_used) {
    const cudaError_t copied = cudaMemcpyAsync(slot->host_status, slot->device_status, sizeof(unsigned),
                                               cudaMemcpyDeviceToHost, queue_state->stream);
    slot->status_copied = copied == cudaSuccess;
    terminal.Update(runtime_status(copied));
  }
  const cudaError_t recorded = cudaEventRecord(slot->event, queue_state->stream);
  slot->recorded = recorded == cudaSuccess;
  // a software diagnostic never replaces an error already seen at enqueue / copy / record time
  slot->report_status = terminal.ok() && recorded == cudaSuccess;
  {
    std::lock_guard lock(queue_state->mutex);
    ++queue_state->counters.event_completions;
    if (slot->status_copied) ++queue_state->counters.status_copies;
  }
  queue_state->incref();  // the Completion keeps the queue's stream and slots alive
  Completion completion = compute::detail::CompletionAccess::make(&kCompletionVTable, slot);
  if (recorded != cudaSuccess) compute::detail::CompletionAccess::append_terminal(completion, runtime_status(recorded));
  compute::detail::CompletionAccess::append_terminal(completion, std::move(terminal));
  return completion;
}

Status reserve_completions_impl(void *queue, std::size_t minimum) noexcept {
  auto *state = static_cast<QueueState *>(queue);
  std::lock_guard lock(state->mutex);
  while (state->all_slots.size() < minimum) {
    Status grown = state->grow();
    if (!grown.ok()) return grown;
  }
  return Status::Ok();
}

// Which cudaMemcpyKind a pair of views needs; nullopt when a side is neither device nor mappable host.
struct CopyRoute final {
  void *destination = nullptr;
  const void *source = nullptr;
  cudaMemcpyKind kind = cudaMemcpyDefault;
  bool queued = false;
};

Result<CopyRoute> copy_route(mem::BufferView destination, mem::ConstBufferView source) noexcept {
  CopyRoute route{};
  const bool device_destination = is_device_resource(destination.resource());
  const bool device_source = is_device_resource(source.resource());
  const auto host_side = [](mem::MemoryResourceRef resource) {
    return resource.valid() && resource.properties().has(mem::MemoryProperty::kHostAccessible) &&
           resource.properties().has(mem::MemoryProperty::kHostAddressIdentity);
  };
  if (device_destination) {
    route.destination = static_cast<std::byte *>(destination.native_handle()) + destination.offset();
  } else if (host_side(destination.resource())) {
    auto mapping = destination.resource().resource().map_host(destination.native_handle(), destination.offset(),
                                                              destination.size(), mem::HostAccess::kWrite);
    if (!mapping) return std::unexpected(std::move(mapping).error());
    route.destination = mapping->data;
  } else {
    return std::unexpected(Status::Unimplemented("b200 backend: copy destination is neither device nor stable host memory"));
  }
  if (device_source) {
    route.source = static_cast<const std::byte *>(source.native_handle()) + source.offset();
  } else if (host_side(source.resource())) {
    auto mapping = source.resource().resource().map_host(source.native_handle(), source.offset(), source.size(),
                                                         mem::HostAccess::kRead);
    if (!mapping) return std::unexpected(std::move(mapping).error());
    route.source = mapping->data;
  } else {
    return std::unexpected(Status::Unimplemented("b200 backend: copy source is neither device nor stable host memory"));
  }
  route.kind = device_destination ? (device_source ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice)
                                  : (device_source ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost);
  const bool pinned = (device_destination || destination.resource().properties().has(mem::MemoryProperty::kHostPinned)) &&
                      (device_source || source.resource().properties().has(mem::MemoryProperty::kHostPinned));
  route.queued = pinned;  // pageable host memory makes cudaMemcpyAsync stage and (partly) block
  return route;
}

Result<TransferProperties> transfer_properties_impl(void *, mem::BufferView destination,
                                                    mem::ConstBufferView source) noexcept {
  auto route = copy_route(destination, source);
  if (!route) return std::unexpected(std::move(route).error());
  return TransferProperties{.mode = route->queued ? TransferMode::kQueuedDirect : TransferMode::kImmediate, .peer = false};
}

EnqueueResult copy_async_impl(void *queue, mem::BufferView destination, mem::ConstBufferView source) noexcept {
  auto *state = static_cast<QueueState *>(queue);
  auto route = copy_route(destination, source);
  if (!route) return EnqueueResult::rejected(std::move(route).error());
  if (destination.size() == 0) return EnqueueResult::no_op();
  DeviceScope scope(state->context->ordinal);
  const cudaError_t error =
      cudaMemcpyAsync(route->destination, route->source, destination.size(), route->kind, state->stream);
  if (error != cudaSuccess) return EnqueueResult::rejected(runtime_status(error));
  return EnqueueResult::accepted_command();
}

EnqueueResult fill_async_impl(void *queue, mem::BufferView destination, std::byte value) noexcept {
  auto *state = static_cast<QueueState *>(queue);
  if (!is_device_resource(destination.resource()))
    return EnqueueResult::rejected(Status::Unimplemented("b200 backend: fill_async takes device storage"));
  if (destination.size() == 0) return EnqueueResult::no_op();
  DeviceScope scope(state->context->ordinal);
  const cudaError_t error =
      cudaMemsetAsync(static_cast<std::byte *>(destination.native_handle()) + destination.offset(),
                      static_cast<int>(value), destination.size(), state->stream);
  if (error != cudaSuccess) return EnqueueResult::rejected(runtime_status(error));
  return EnqueueResult::accepted_command();
}

EnqueueResult wait_completion_impl(void *queue, const compute::detail::CompletionVTable *vtable, void *state) noexcept {
  // A Completion of this backend (any Queue of it): wait for its event on this Queue's stream.
  if (vtable != &kCompletionVTable || state == nullptr)
    return EnqueueResult::rejected(Status::Unimplemented("b200 backend: cannot consume a foreign completion on the device"));
  auto *slot = static_cast<Slot *>(state);
  auto *destination = static_cast<QueueState *>(queue);
  if (!slot->recorded)
    return EnqueueResult::rejected(Status::Unimplemented("b200 backend: source completion has no event"));
  DeviceScope scope(destination->context->ordinal);
  const cudaError_t error = cudaStreamWaitEvent(destination->stream, slot->event, 0);
  if (error != cudaSuccess) return EnqueueResult::rejected(runtime_status(error));
  return EnqueueResult::accepted_command();
}

compute::detail::CompletionEndpoint completion_endpoint_impl(void *queue) noexcept {
  return {&kBackendVTable, queue};
}

bool can_wait_endpoint_impl(void *, compute::detail::CompletionEndpoint source) noexcept {
  return source.authority == &kBackendVTable && source.identity != nullptr;
}

const void *query_extension_impl(void *, BackendExtensionId) noexcept { return nullptr; }

Status drain_context_impl(void *context) noexcept {
  DeviceScope scope(static_cast<ContextState *>(context)->ordinal);
  if (scope.status != cudaSuccess) return runtime_status(scope.status);
  return runtime_status(cudaDeviceSynchronize());
}

Status drain_queue_impl(void *queue) noexcept {
  auto *state = static_cast<QueueState *>(queue);
  DeviceScope scope(state->context->ordinal);
  return runtime_status(cudaStreamSynchronize(state->stream));
}

constinit const compute::detail::BackendVTable kBackendVTable{
    .id = kBackendId,
    .name = "b200-cuda12",
    .device_class = DeviceClass::kGpu,
    .device_count = &device_count_impl,
    .device = &device_impl,
    .same_device = &same_device_impl,
    .properties = &properties_impl,
    .validate_resource = &validate_resource_impl,
    .create_context = &create_context_impl,
    .destroy_context = &destroy_context_impl,
    .create_queue = &create_queue_impl,
    .destroy_queue = &destroy_queue_impl,
    .begin_sequence = &begin_sequence_impl,
    .finish_sequence = &finish_sequence_impl,
    .reserve_completions = &reserve_completions_impl,
    .transfer_properties = &transfer_properties_impl,
    .copy_async = &copy_async_impl,
    .fill_async = &fill_async_impl,
    .wait_completion = &wait_completion_impl,
    .completion_endpoint = &completion_endpoint_impl,
    .can_wait_endpoint = &can_wait_endpoint_impl,
    .query_extension = &query_extension_impl,
    .drain_context = &drain_context_impl,
    .drain_queue = &drain_queue_impl,
};

QueueState *queue_of(const compute::detail::QueueSequence &sequence) noexcept {
  auto *state = compute::detail::ContextAccess::state(sequence);
  if (state == nullptr || state->context == nullptr || state->context->backend_vtable != &kBackendVTable) return nullptr;
  return static_cast<QueueState *>(state->backend_state);
}

}  // namespace

Backend backend() noexcept { return compute::detail::BackendAccess::make(&kBackendVTable, BackendPayload{}); }

Result<Device> device(std::size_t ordinal) noexcept { return device_impl(backend(), ordinal); }

Result<int> device_ordinal(Device value) noexcept {
  if (compute::detail::DeviceAccess::vtable(value) != &kBackendVTable)
    return std::unexpected(Status::InvalidArgument("device does not belong to the b200 CUDA backend"));
  return static_cast<int>(compute::detail::DeviceAccess::payload<DevicePayload>(value).ordinal);
}

// ---- DeviceMemory -------------------------------------------------------------------------------------------------------
Result<DeviceMemory> DeviceMemory::create(const Context &context) noexcept {
  auto *state = compute::detail::ContextAccess::state(context);
  if (state == nullptr || state->backend_vtable != &kBackendVTable)
    return std::unexpected(Status::InvalidArgument("context does not belong to the b200 CUDA backend"));
  auto *resource = new (std::nothrow) CudaMallocResource(static_cast<ContextState *>(state->backend_state)->ordinal);
  if (resource == nullptr) return std::unexpected(Status::ResourceExhausted("b200 backend: resource allocation failed"));
  return DeviceMemory(resource);
}

DeviceMemory &DeviceMemory::operator=(DeviceMemory &&other) noexcept {
  if (this != &other) {
    delete static_cast<CudaMallocResource *>(state_);
    state_ = std::exchange(other.state_, nullptr);
  }
  return *this;
}

DeviceMemory::~DeviceMemory() { delete static_cast<CudaMallocResource *>(state_); }

mem::MemoryResourceRef DeviceMemory::ref() const noexcept {
  return state_ != nullptr ? mem::MemoryResourceRef(*static_cast<CudaMallocResource *>(state_)) : mem::MemoryResourceRef{};
}

std::size_t DeviceMemory::live_allocations() const noexcept {
  return state_ != nullptr ? static_cast<CudaMallocResource *>(state_)->live() : 0;
}

// ---- what the provider adapter uses ---------------------------------------------------------------------------------------
Result<hyle_b200_stream_t> stream(const compute::detail::QueueSequence &sequence) noexcept {
  QueueState *queue = queue_of(sequence);
  if (queue == nullptr)
    return std::unexpected(Status::FailedPrecondition("sequence does not belong to a b200 CUDA queue"));
  return reinterpret_cast<hyle_b200_stream_t>(queue->stream);
}

Result<hyle_b200_stream_t> stream(const Queue &queue) noexcept {
  auto *state = compute::detail::ContextAccess::state(queue);
  if (state == nullptr || state->context == nullptr || state->context->backend_vtable != &kBackendVTable)
    return std::unexpected(Status::FailedPrecondition("queue does not belong to the b200 CUDA backend"));
  return reinterpret_cast<hyle_b200_stream_t>(static_cast<QueueState *>(state->backend_state)->stream);
}

Result<void *> pointer(mem::BufferView view) noexcept {
  if (!is_device_resource(view.resource()))
    return std::unexpected(Status::FailedPrecondition("buffer is not b200 CUDA device storage"));
  return static_cast<void *>(static_cast<std::byte *>(view.native_handle()) + view.offset());
}

Result<const void *> pointer(mem::ConstBufferView view) noexcept {
  if (!is_device_resource(view.resource()))
    return std::unexpected(Status::FailedPrecondition("buffer is not b200 CUDA device storage"));
  return static_cast<const void *>(static_cast<const std::byte *>(view.native_handle()) + view.offset());
}

Status status(int abi_result) noexcept {
  switch (abi_result) {
    case HYLE_B200_OK: return Status::Ok();
    case HYLE_B200_INVALID_VALUE: return Status::InvalidArgument(hyle_b200_result_string(abi_result));
    case HYLE_B200_NOT_SUPPORTED: return Status::Unimplemented(hyle_b200_result_string(abi_result));
    default: break;
  }
  if (abi_result == HYLE_B200_STATIC_SCRATCH_EXCEEDED) return Status::OutOfRange(hyle_b200_result_string(abi_result));
  return runtime_status(static_cast<cudaError_t>(abi_result));
}

EnqueueResult acquire_status_word(compute::detail::QueueSequence &sequence, unsigned **device_word) noexcept {
  if (device_word == nullptr) return EnqueueResult::rejected(Status::InvalidArgument("status output is null"));
  *device_word = nullptr;
  QueueState *queue = queue_of(sequence);
  if (queue == nullptr || queue->active_sequence == nullptr)
    return EnqueueResult::rejected(Status::FailedPrecondition("a device status word requires an admitted sequence"));
  Slot *slot = queue->active_sequence;
  if (slot->status_used) {
    *device_word = slot->device_status;
    return EnqueueResult::no_op();
  }
  DeviceScope scope(queue->context->ordinal);
  const cudaError_t cleared = cudaMemsetAsync(slot->device_status, 0, sizeof(unsigned), queue->stream);
  if (cleared != cudaSuccess) return EnqueueResult::rejected(runtime_status(cleared));
  slot->status_used = true;
  *device_word = slot->device_status;
  return EnqueueResult::accepted_command();
}

Status status_from_bits(unsigned bits) noexcept {
  if (bits == 0) return Status::Ok();
  if (bits & HYLE_B200_STATUS_INVALID_Q8_INPUT)
    return Status::InvalidArgument("cache encoder requires finite inputs and representable Q8_0 scales");
  if (bits & HYLE_B200_STATUS_INVALID_FP8_INPUT)
    return Status::InvalidArgument("cache encoder requires finite numeric inputs");
  if (bits & HYLE_B200_STATUS_INVALID_CATEGORICAL_ROW)
    return Status::InvalidArgument("categorical weights need a finite maximum and no NaN in every row");
  if (bits & HYLE_B200_STATUS_SCAN_OVERFLOW) return Status::OutOfRange("integer prefix sum overflows I32");
  if (bits & HYLE_B200_STATUS_EXCHANGE_TIMEOUT)
    return Status::DeadlineExceeded("a peer's partial sum did not arrive within the exchange's poll limit");
  if (bits & HYLE_B200_STATUS_STREAM_WAIT_TIMEOUT)
    return Status::Unavailable("the streaming logits kernel gave up waiting for a row's partials; rows are NaN");
  return Status::Internal("kernel library returned an unknown device status");
}

Result<Counters> counters(const Queue &queue) noexcept {
  auto *state = compute::detail::ContextAccess::state(queue);
  if (state == nullptr || state->context == nullptr || state->context->backend_vtable != &kBackendVTable)
    return std::unexpected(Status::FailedPrecondition("queue does not belong to the b200 CUDA backend"));
  auto *backend_queue = static_cast<QueueState *>(state->backend_state);
  std::lock_guard lock(backend_queue->mutex);
  return backend_queue->counters;
}

}  // namespace hyle::compute::b200::backend

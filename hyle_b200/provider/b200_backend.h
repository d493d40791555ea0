// A thin CUDA backend for HYLE Contexts, built with the CUDA 12.x runtime.
//
// The reference's own CUDA backend (src/compute_backend_cuda) needs CUDA Toolkit >= 13.3 and its
// public header uses CUDA-13-only types (include/hyle/compute/backends/cuda.h:101), so it cannot be
// compiled beside a 12.x toolkit.  This file is the part of it the kernel provider needs, as a
// SAME-BUILD component of the reference's compute core (it fills the private
// detail::BackendVTable, src/compute/backend_internal.h:14-67):
//
//   * a Queue owns one non-default cudaStream_t; one producer records into it at a time
//     (begin_sequence rejects a second one, as src/compute_backend_cuda/cuda_backend.cc:1029-1042);
//   * finish_sequence with nothing accepted completes inline; otherwise it records an event and
//     returns an event-backed Completion (poll = cudaEventQuery, wait = cudaEventSynchronize;
//     cuda_backend.cc:1044-1089);
//   * a per-sequence DEVICE STATUS WORD: the first acquire_status_word() of a sequence clears a device
//     word on the stream and hands it to the kernels; finish_sequence copies it to pinned host memory
//     in stream order and the Completion's terminal status reports it (the protocol of
//     src/compute_backend_cuda/device_status_kernel.h:7-13 and cuda_device_status.cc:88-104, with this
//     kernel library's status BITS, include/hyle_b200.h, instead of the reference's codes);
//   * device memory is a mem::MemoryResource over cudaMalloc: 256-byte aligned, flagged
//     kDeviceAccessible only, read/write/fill through cudaMemcpy / cudaMemset
//     (src/compute_backend_cuda/cuda_memory.cc:26-49, cuda_internal.h:27);
//   * copy_async / fill_async record cudaMemcpyAsync / cudaMemsetAsync on the Queue's stream.
//
// Not here (the provider does not need them): stream import, command capture, peer transfers,
// managed and pinned resources, cross-queue device waits (wait_completion is Unimplemented, so a
// caller falls back to an explicit host wait), NVML facts.
#pragma once

#include <cstddef>

#include <hyle/compute/completion.h>
#include <hyle/compute/detail/queue_sequence.h>
#include <hyle/compute/device.h>
#include <hyle/error/result.h>
#include <hyle/mem/buffer.h>
#include <hyle/mem/resource.h>

#include "hyle_b200.h"

namespace hyle::compute::b200::backend {

// "HYLE" / "B200" + "CUDA12": distinct from cuda::kBackendId, so a provider made for one backend is
// refused by a Context of the other (src/compute/custom_kernel.cc:64-67).
inline constexpr BackendId kBackendId{0x48594c4542323030ULL, 0x4355444131320001ULL};

Backend backend() noexcept;
Result<Device> device(std::size_t ordinal) noexcept;
Result<int> device_ordinal(Device device) noexcept;

// Owner of one cudaMalloc allocation domain on the Context's device.  ref() is non-owning, like
// every MemoryResourceRef: this object must outlive the Buffers made from it.
class DeviceMemory final {
public:
  DeviceMemory() noexcept = default;
  DeviceMemory(const DeviceMemory &) = delete;
  DeviceMemory &operator=(const DeviceMemory &) = delete;
  DeviceMemory(DeviceMemory &&other) noexcept : state_(other.state_) { other.state_ = nullptr; }
  DeviceMemory &operator=(DeviceMemory &&other) noexcept;
  ~DeviceMemory();

  static Result<DeviceMemory> create(const Context &context) noexcept;
  bool valid() const noexcept { return state_ != nullptr; }
  mem::MemoryResourceRef ref() const noexcept;
  // Live allocations and bytes, for leak checks.
  std::size_t live_allocations() const noexcept;

private:
  explicit DeviceMemory(void *state) noexcept : state_(state) {}
  void *state_ = nullptr;
};

// The Queue's stream, through the admitted sequence (no new producer is acquired).
Result<hyle_b200_stream_t> stream(const detail::QueueSequence &sequence) noexcept;
Result<hyle_b200_stream_t> stream(const Queue &queue) noexcept;

// Device address of a view of DeviceMemory storage; other resources are refused.
Result<void *> pointer(mem::BufferView view) noexcept;
Result<const void *> pointer(mem::ConstBufferView view) noexcept;

// cudaError_t-compatible result of a hyle_b200_* call -> Status.
Status status(int abi_result) noexcept;

// Inside one admitted sequence only.  The first use in a sequence records a clear of the word on the
// stream; propagate the EnqueueResult even if a later command fails.  Kernels OR their status bits
// into the word; the sequence's Completion reports them (status_from_bits).
detail::EnqueueResult acquire_status_word(detail::QueueSequence &sequence, unsigned **device_word) noexcept;

// What a Completion reports for a status word: the reference's wording where it has one
// (src/compute_provider_ggml/ggml_cpu_provider.cc:1720-1721; cuda_device_status.cc:96-99).
Status status_from_bits(unsigned bits) noexcept;

// Counters for tests: how many sequences ended with an event-backed Completion, and how many
// status words were copied back.
struct Counters final {
  std::size_t event_completions = 0;
  std::size_t status_copies = 0;
  std::size_t slots_created = 0;
};
Result<Counters> counters(const Queue &queue) noexcept;

// The adapter's Backend concept (hyle_b200/provider/b200_provider.h) bound to this backend.
struct Cuda12Backend final {
  static constexpr BackendId id() noexcept { return kBackendId; }
  static constexpr mem::MemoryProperty memory() noexcept { return mem::MemoryProperty::kDeviceAccessible; }
  static Result<hyle_b200_stream_t> stream(detail::QueueSequence &sequence) noexcept {
    return backend::stream(sequence);
  }
  static Result<const void *> pointer(mem::ConstBufferView view) noexcept { return backend::pointer(view); }
  static Result<void *> mutable_pointer(mem::BufferView view) noexcept { return backend::pointer(view); }
  static Status status(int result) noexcept { return backend::status(result); }
  static detail::EnqueueResult status_word(detail::QueueSequence &sequence, unsigned **word) noexcept {
    return acquire_status_word(sequence, word);
  }
};

}  // namespace hyle::compute::b200::backend

// Paged append through libhyle_b200.so, shaped like the reference CUDA backend's launcher
// (src/compute_backend_cuda/cuda_paged_append.h: launch_paged_append(kernel, arena, rows, metadata,
// spec, stream), defined at cuda_paged_append.cu:70-81).
//
// The reference reaches that launcher from its backend extension table
// (include/hyle/compute/detail/paged_append_backend.h:24-31; enqueue_append at
// src/compute_backend_cuda/cuda_paged_append.cc:81-109), which belongs to the backend itself and
// cannot be supplied by an out-of-tree provider.  The drop-in is therefore this one function:
// enqueue_append keeps its carrier validation and calls b200::launch_paged_append where it called
// the CUDA launcher.  Same wire structs, same device-side guards, same "one fixed-topology launch
// whose shape depends on the spec only" property (so `supports_command_capture` stays true).
#pragma once

#include <cstdint>

#include <hyle/compute/detail/device_lengths_paged_append_wire.h>
#include <hyle/compute/detail/paged_append_wire.h>

#include "hyle_b200.h"

namespace hyle::compute::b200 {

// Returns the cudaError_t value of the launch (0 = success), like the function it replaces.
// HYLE_B200_INVALID_VALUE (= cudaErrorInvalidValue) for a geometry prepare_append would have
// refused (src/compute_backend_cuda/cuda_paged_append.cc:28-33).
inline int launch_paged_append(void *arena, const void *rows, const void *metadata,
                               compute::detail::PagedAppendNativeSpec spec, hyle_b200_stream_t stream) noexcept {
  return hyle_b200_paged_append(stream, arena, rows, metadata, spec.page_rows, spec.physical_pages, spec.input_rows,
                                spec.instruction_capacity, static_cast<std::uint64_t>(spec.row_bytes));
}

// The device-lengths variant (launch_device_lengths_paged_append, cuda_paged_append.cu:148-154;
// called from enqueue_lengths, src/compute_backend_cuda/cuda_paged_append.cc:125-147).  `status` is the
// queue's device status word with the reference's codes.  HYLE_B200_NOT_SUPPORTED for a domain
// prepare_lengths declines (cuda_paged_append.cc:112-115).
inline int launch_device_lengths_paged_append(void *arena, const void *rows, const void *metadata, const void *query_lengths,
                                              const void *kv_lengths, compute::detail::DeviceLengthsPagedAppendSpec spec,
                                              unsigned *status, hyle_b200_stream_t stream) noexcept {
  return hyle_b200_paged_append_device_lengths(
      stream, arena, rows, metadata, static_cast<const std::int32_t *>(query_lengths),
      static_cast<const std::int32_t *>(kv_lengths), spec.storage.page_rows, spec.storage.physical_pages,
      spec.storage.input_rows, spec.storage.instruction_capacity, static_cast<std::uint64_t>(spec.storage.row_bytes),
      spec.requests, status);
}

}  // namespace hyle::compute::b200

// TEST INFRASTRUCTURE.  C entry point over the reference's own paged-append CUDA kernel, which the
// Makefile compiles in place from the reference tree (src/compute_backend_cuda/cuda_paged_append.cu,
// launcher at :70-81).  GPU parity tests run it beside the product kernel on the same episodes; the
// product never links it.
#include <cstddef>
#include <cstdint>

#include "cuda_paged_append.h"

extern "C" __attribute__((visibility("default"))) int hyle_ref_paged_append(
    void *stream, void *arena, const void *rows, const void *metadata, uint32_t page_rows, uint32_t physical_pages,
    uint32_t input_rows, uint32_t instruction_capacity, uint64_t row_bytes) {
  hyle::compute::detail::PagedAppendNativeSpec spec{};
  spec.page_rows = page_rows;
  spec.physical_pages = physical_pages;
  spec.input_rows = input_rows;
  spec.instruction_capacity = instruction_capacity;
  spec.row_bytes = static_cast<std::size_t>(row_bytes);
  namespace ref = hyle::compute::cuda::detail;
  return static_cast<int>(ref::launch_paged_append(ref::paged_append_kernel(), arena, rows, metadata, spec,
                                                   static_cast<cudaStream_t>(stream)));
}

// The device-lengths variant of the same file (launcher at cuda_paged_append.cu:148-154).
extern "C" __attribute__((visibility("default"))) int hyle_ref_paged_append_device_lengths(
    void *stream, void *arena, const void *rows, const void *metadata, const void *query_lengths, const void *kv_lengths,
    uint32_t page_rows, uint32_t physical_pages, uint32_t input_rows, uint32_t instruction_capacity, uint64_t row_bytes,
    uint32_t requests, unsigned *status) {
  hyle::compute::detail::DeviceLengthsPagedAppendSpec spec{};
  spec.storage.page_rows = page_rows;
  spec.storage.physical_pages = physical_pages;
  spec.storage.input_rows = input_rows;
  spec.storage.instruction_capacity = instruction_capacity;
  spec.storage.row_bytes = static_cast<std::size_t>(row_bytes);
  spec.requests = requests;
  namespace ref = hyle::compute::cuda::detail;
  return static_cast<int>(ref::launch_device_lengths_paged_append(ref::device_lengths_paged_append_kernel(), arena, rows,
                                                                  metadata, query_lengths, kv_lengths, spec, status,
                                                                  static_cast<cudaStream_t>(stream)));
}

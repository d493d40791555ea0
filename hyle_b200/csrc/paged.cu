// Paged append: copy rows into the pages of a cache arena as a list of device-resident
// instructions says (the step after CacheEncode: encoded rows -> KV pages).
//
// Wire format and rules follow include/hyle/compute/detail/paged_append_wire.h:11-25 and the
// reference kernel's guards (src/compute_backend_cuda/cuda_paged_append.cu:11-62):
//   metadata     = {active_count, 0, 0, 0} followed by `instruction_capacity` instructions of
//                  {source_kind, source_page, source_row, destination_page, destination_row, rows, 0, 0}
//   source_kind 0  reads `rows` packed new rows starting at source_row of the input
//   source_kind 1  reads them from (source_page, source_row) of the same arena
//   destination    (destination_page * page_rows + destination_row) rows into the arena
// An episode whose active_count exceeds the capacity or whose reserved words are not zero does
// nothing; an instruction with non-zero reserved words, zero rows, an unknown source kind or any
// coordinate outside the arena / the input is skipped.  Rows are moved as bytes.
//
// Byte work bound by HBM: an instruction's byte range is cut into slices of 16 KB and the
// (instruction, slice) pairs are spread over the grid, so a few long instructions and many short
// ones both fill the machine; 16-byte accesses when the row size and the bases allow, 2-byte
// elements otherwise (the reference moves 16-bit elements).
#include "common.cuh"

namespace hb {
namespace {

constexpr int kThreads = 256;
constexpr uint64_t kSliceBytes = 16384;

struct Instruction {
  uint32_t source_kind, source_page, source_row, destination_page;
  uint32_t destination_row, rows, reserved0, reserved1;
};
struct Metadata {
  uint32_t active_count, reserved0, reserved1, reserved2;
};
static_assert(sizeof(Instruction) == 32 && sizeof(Metadata) == 16, "wire format");

struct Spec {
  uint32_t page_rows, physical_pages, input_rows, instruction_capacity;
  uint64_t row_bytes;
  uint32_t slices;  // slices per instruction the grid provides for: ceil(page_rows * row_bytes / kSliceBytes)
};

template <bool kVector>
__global__ void __launch_bounds__(kThreads)
paged_append_kernel(unsigned char *arena, const unsigned char *__restrict__ input, const Metadata *__restrict__ metadata,
                    const Spec spec) {
  grid_dependency_sync();
  const uint32_t active = metadata->active_count;
  if (active > spec.instruction_capacity || metadata->reserved0 != 0 || metadata->reserved1 != 0 || metadata->reserved2 != 0)
    return;
  const Instruction *instructions = reinterpret_cast<const Instruction *>(metadata + 1);
  const uint64_t units = static_cast<uint64_t>(active) * spec.slices;
  for (uint64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    const uint64_t index = unit / spec.slices;
    const uint32_t slice = static_cast<uint32_t>(unit - index * spec.slices);
    const Instruction in = instructions[index];
    if (in.reserved0 != 0 || in.reserved1 != 0 || in.rows == 0 || in.source_kind > 1 ||
        in.destination_page >= spec.physical_pages || in.destination_row > spec.page_rows ||
        in.rows > spec.page_rows - in.destination_row)
      continue;
    const unsigned char *source;
    if (in.source_kind == 0) {
      if (in.source_row > spec.input_rows || in.rows > spec.input_rows - in.source_row) continue;
      source = input + static_cast<uint64_t>(in.source_row) * spec.row_bytes;
    } else {
      if (in.source_page >= spec.physical_pages || in.source_row > spec.page_rows || in.rows > spec.page_rows - in.source_row)
        continue;
      source = arena + (static_cast<uint64_t>(in.source_page) * spec.page_rows + in.source_row) * spec.row_bytes;
    }
    unsigned char *destination = arena + (static_cast<uint64_t>(in.destination_page) * spec.page_rows + in.destination_row) * spec.row_bytes;
    const uint64_t bytes = static_cast<uint64_t>(in.rows) * spec.row_bytes;
    const uint64_t begin = static_cast<uint64_t>(slice) * kSliceBytes;
    if (begin >= bytes) continue;
    const uint64_t end = min(begin + kSliceBytes, bytes);
    if constexpr (kVector) {
      const uint4 *from = reinterpret_cast<const uint4 *>(source + begin);
      uint4 *to = reinterpret_cast<uint4 *>(destination + begin);
      const uint32_t vectors = static_cast<uint32_t>((end - begin) / 16);
      for (uint32_t v = threadIdx.x; v < vectors; v += kThreads * 4) {  // up to four loads in flight
        uint4 held[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (v + k * kThreads < vectors) held[k] = ld_stream(from + v + k * kThreads);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (v + k * kThreads < vectors) st_stream(to + v + k * kThreads, held[k]);
      }
    } else {
      const unsigned short *from = reinterpret_cast<const unsigned short *>(source + begin);
      unsigned short *to = reinterpret_cast<unsigned short *>(destination + begin);
      const uint32_t elements = static_cast<uint32_t>((end - begin) / 2);
      for (uint32_t e = threadIdx.x; e < elements; e += kThreads) to[e] = from[e];
    }
  }
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" int hyle_b200_paged_append(hyle_b200_stream_t stream, void *arena, const void *input_rows_data,
                                      const void *metadata, uint32_t page_rows, uint32_t physical_pages,
                                      uint32_t input_rows, uint32_t instruction_capacity, uint64_t row_bytes) {
  if (instruction_capacity == 0) return HYLE_B200_OK;
  if (arena == nullptr || metadata == nullptr || (input_rows_data == nullptr && input_rows != 0) || page_rows == 0 ||
      row_bytes == 0 || row_bytes % 2 != 0 || !aligned_to(metadata, 4) || !aligned_to(arena, 2) ||
      !aligned_to(input_rows_data, 2))
    return HYLE_B200_INVALID_VALUE;
  Spec spec{page_rows, physical_pages, input_rows, instruction_capacity, row_bytes, 0};
  const uint64_t longest = static_cast<uint64_t>(page_rows) * row_bytes;
  const uint64_t slices = (longest + kSliceBytes - 1) / kSliceBytes;
  if (slices > 0xffffffffull) return HYLE_B200_NOT_SUPPORTED;
  spec.slices = static_cast<uint32_t>(slices);
  // The grid depends only on capacities known to the host, never on the device-side active count.
  const uint64_t units = static_cast<uint64_t>(instruction_capacity) * spec.slices;
  const unsigned grid = clamp_grid(units, static_cast<uint64_t>(sm_count()) * 8);
  const bool vector = row_bytes % 16 == 0 && aligned_to(arena, 16) && (input_rows_data == nullptr || aligned_to(input_rows_data, 16));
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (vector)
    return launch(paged_append_kernel<true>, dim3(grid), dim3(kThreads), 0, s, static_cast<unsigned char *>(arena),
                  static_cast<const unsigned char *>(input_rows_data), static_cast<const Metadata *>(metadata), spec);
  return launch(paged_append_kernel<false>, dim3(grid), dim3(kThreads), 0, s, static_cast<unsigned char *>(arena),
                static_cast<const unsigned char *>(input_rows_data), static_cast<const Metadata *>(metadata), spec);
}

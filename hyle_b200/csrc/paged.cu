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

// ---- device-lengths variant ----------------------------------------------------------------------
// The episode holds no finished instructions: after the header come a directory {requests, pages},
// `requests` request bounds and `pages` dirty-page records
// (include/hyle/compute/detail/device_lengths_paged_append_wire.h:8-24), and the kernel derives
// each page's three ranges from the query / KV lengths that live on the device
// (src/compute_backend_cuda/cuda_paged_append.cu:82-146):
//   rows [0, inherited)          from the beginning of source_page of the arena (copy on write),
//   rows [inherited, live)       from the packed new rows of the page's request,
//   rows [live, initialized)     zero.
struct Directory {
  uint32_t requests, pages, reserved[6];
};
struct Request {
  uint32_t query_rows, minimum_previous_rows, maximum_previous_rows, maximum_kv_rows, reserved[4];
};
struct Page {
  uint32_t request, logical_page, destination_page, initialized_rows, source_page, source_rows, reserved[2];
};
static_assert(sizeof(Directory) == 32 && sizeof(Request) == 32 && sizeof(Page) == 32, "wire format");

constexpr uint32_t kMaxRequests = 32;
constexpr unsigned kStatusIndexOutOfRange = 1, kStatusInvalidSequenceOffsets = 4;  // device_status_kernel.h:7-13

template <bool kVector>
__global__ void __launch_bounds__(kThreads)
paged_append_lengths_kernel(unsigned char *arena, const unsigned char *__restrict__ input, const Metadata *__restrict__ metadata,
                            const int32_t *__restrict__ query_lengths, const int32_t *__restrict__ kv_lengths, const Spec spec,
                            const uint32_t requests, unsigned *status) {
  grid_dependency_sync();
  __shared__ int32_t s_offset[kMaxRequests], s_previous[kMaxRequests], s_last[kMaxRequests];
  __shared__ uint32_t s_pages;
  __shared__ bool s_valid;
  const Instruction *words = reinterpret_cast<const Instruction *>(metadata + 1);
  const Directory *directory = reinterpret_cast<const Directory *>(words);
  // Warp 0 checks the episode: lane r owns request r, the row offsets are a prefix sum over lanes.
  if (threadIdx.x < kWarpSize) {
    const uint32_t lane = threadIdx.x;
    const uint32_t active = metadata->active_count;
    bool valid = *reinterpret_cast<volatile unsigned *>(status) == 0;
    const uint32_t listed = directory->requests, pages = directory->pages;
    if (active == 0 || active > spec.instruction_capacity || metadata->reserved0 != 0 || metadata->reserved1 != 0 ||
        metadata->reserved2 != 0 || listed != requests || listed > kMaxRequests || pages > active - 1 ||
        listed > active - 1 - pages)
      valid = false;
    if (lane < 6 && directory->reserved[lane] != 0) valid = false;
    valid = __all_sync(kFullMask, valid);
    int64_t rows = 0;
    int32_t previous = 0, last = 0;
    bool mine = true;
    if (valid && lane < requests) {
      const Request bounds = reinterpret_cast<const Request *>(words + 1)[lane];
      const int32_t q = query_lengths[lane], kv = kv_lengths[lane];
      const int64_t old = static_cast<int64_t>(kv) - q;
      mine = (bounds.reserved[0] | bounds.reserved[1] | bounds.reserved[2] | bounds.reserved[3]) == 0 && q >= 0 &&
             static_cast<uint32_t>(q) <= bounds.query_rows && kv >= 0 && static_cast<uint32_t>(kv) <= bounds.maximum_kv_rows &&
             old >= static_cast<int64_t>(bounds.minimum_previous_rows) && old <= static_cast<int64_t>(bounds.maximum_previous_rows);
      rows = mine ? q : 0;
      previous = static_cast<int32_t>(old);
      last = kv;
    }
    int64_t inclusive = rows;
#pragma unroll
    for (int step = 1; step < kWarpSize; step <<= 1) {
      const int64_t below = __shfl_up_sync(kFullMask, inclusive, step);
      if (lane >= static_cast<uint32_t>(step)) inclusive += below;
    }
    if (lane < requests && inclusive > static_cast<int64_t>(spec.input_rows)) mine = false;
    valid = __all_sync(kFullMask, valid && mine);
    if (lane < kMaxRequests) {
      s_offset[lane] = static_cast<int32_t>(inclusive - rows);
      s_previous[lane] = previous;
      s_last[lane] = last;
    }
    if (lane == 0) {
      s_valid = valid;
      s_pages = pages;
      if (!valid) atomicCAS(status, 0u, kStatusInvalidSequenceOffsets);
    }
  }
  __syncthreads();
  if (!s_valid) return;
  const Page *pages = reinterpret_cast<const Page *>(words + 1 + requests);
  const uint64_t units = static_cast<uint64_t>(s_pages) * spec.slices;
  for (uint64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    const uint64_t index = unit / spec.slices;
    const uint32_t slice = static_cast<uint32_t>(unit - index * spec.slices);
    const Page p = pages[index];
    bool good = p.request < requests && p.destination_page < spec.physical_pages && p.initialized_rows != 0 &&
                p.initialized_rows <= spec.page_rows && p.source_rows <= spec.page_rows && p.reserved[0] == 0 && p.reserved[1] == 0;
    uint32_t inherited = 0, live = 0;
    uint64_t source_row = 0;
    if (good) {
      const uint64_t begin = static_cast<uint64_t>(p.logical_page) * spec.page_rows;
      const uint64_t prior = static_cast<uint64_t>(s_previous[p.request]), next = static_cast<uint64_t>(s_last[p.request]);
      inherited = begin < prior ? static_cast<uint32_t>(min(static_cast<uint64_t>(p.initialized_rows), prior - begin)) : 0u;
      live = begin < next ? static_cast<uint32_t>(min(static_cast<uint64_t>(p.initialized_rows), next - begin)) : 0u;
      const uint32_t added = live - inherited;
      source_row = added ? static_cast<uint64_t>(s_offset[p.request]) + (begin > prior ? begin : prior) - prior : 0;
      good = !(inherited > live || (inherited && (p.source_page >= spec.physical_pages || inherited > p.source_rows)) ||
               (added && (source_row > spec.input_rows || added > spec.input_rows - source_row)));
    }
    if (!good) {  // the record is skipped and reported; the reference's block stops here as well
      if (threadIdx.x == 0) atomicCAS(status, 0u, kStatusIndexOutOfRange);
      continue;
    }
    const uint64_t bytes = static_cast<uint64_t>(p.initialized_rows) * spec.row_bytes;
    const uint64_t begin_byte = static_cast<uint64_t>(slice) * kSliceBytes;
    if (begin_byte >= bytes) continue;
    const uint64_t end_byte = min(begin_byte + kSliceBytes, bytes);
    const uint64_t inherited_bytes = static_cast<uint64_t>(inherited) * spec.row_bytes;
    const uint64_t live_bytes = static_cast<uint64_t>(live) * spec.row_bytes;
    // Byte b of the destination range comes from old_page[b], new_rows[b - inherited_bytes] or is zero.
    const unsigned char *old_page = arena + static_cast<uint64_t>(inherited ? p.source_page : 0) * spec.page_rows * spec.row_bytes;
    const unsigned char *new_rows = input + source_row * spec.row_bytes - inherited_bytes;
    unsigned char *destination = arena + static_cast<uint64_t>(p.destination_page) * spec.page_rows * spec.row_bytes;
    if constexpr (kVector) {
      for (uint64_t b = begin_byte + threadIdx.x * 16ull; b < end_byte; b += kThreads * 16ull * 4) {
        uint4 held[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t at = b + static_cast<uint64_t>(k) * kThreads * 16;
          held[k] = make_uint4(0, 0, 0, 0);
          if (at < end_byte && at < live_bytes)
            held[k] = ld_stream(reinterpret_cast<const uint4 *>((at < inherited_bytes ? old_page : new_rows) + at));
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t at = b + static_cast<uint64_t>(k) * kThreads * 16;
          if (at < end_byte) st_stream(reinterpret_cast<uint4 *>(destination + at), held[k]);
        }
      }
    } else {
      for (uint64_t b = begin_byte + threadIdx.x * 2ull; b < end_byte; b += kThreads * 2ull) {
        unsigned short value = 0;
        if (b < live_bytes) value = *reinterpret_cast<const unsigned short *>((b < inherited_bytes ? old_page : new_rows) + b);
        *reinterpret_cast<unsigned short *>(destination + b) = value;
      }
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

extern "C" int hyle_b200_paged_append_device_lengths(hyle_b200_stream_t stream, void *arena, const void *input_rows_data,
                                                     const void *metadata, const int32_t *query_lengths,
                                                     const int32_t *kv_lengths, uint32_t page_rows, uint32_t physical_pages,
                                                     uint32_t input_rows, uint32_t instruction_capacity, uint64_t row_bytes,
                                                     uint32_t requests, uint32_t *status_word) {
  // The domain prepare_lengths qualifies (src/compute_backend_cuda/cuda_paged_append.cc:110-115).
  if (requests == 0 || requests > kMaxRequests || input_rows > 0x7fffffffu || instruction_capacity < requests + 2)
    return HYLE_B200_NOT_SUPPORTED;
  if (arena == nullptr || metadata == nullptr || input_rows_data == nullptr || query_lengths == nullptr || kv_lengths == nullptr ||
      status_word == nullptr || page_rows == 0 || physical_pages == 0 || input_rows == 0 || row_bytes == 0 || row_bytes % 2 != 0 ||
      !aligned_to(metadata, 4) || !aligned_to(arena, 2) || !aligned_to(input_rows_data, 2) || !aligned_to(query_lengths, 4) ||
      !aligned_to(kv_lengths, 4) || !aligned_to(status_word, 4))
    return HYLE_B200_INVALID_VALUE;
  Spec spec{page_rows, physical_pages, input_rows, instruction_capacity, row_bytes, 0};
  const uint64_t slices = (static_cast<uint64_t>(page_rows) * row_bytes + kSliceBytes - 1) / kSliceBytes;
  if (slices > 0xffffffffull) return HYLE_B200_NOT_SUPPORTED;
  spec.slices = static_cast<uint32_t>(slices);
  const uint64_t units = static_cast<uint64_t>(instruction_capacity - 1 - requests) * spec.slices;
  const unsigned grid = clamp_grid(units, static_cast<uint64_t>(sm_count()) * 8);
  const bool vector = row_bytes % 16 == 0 && aligned_to(arena, 16) && aligned_to(input_rows_data, 16);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  auto kernel = vector ? paged_append_lengths_kernel<true> : paged_append_lengths_kernel<false>;
  return launch(kernel, dim3(grid), dim3(kThreads), 0, s, static_cast<unsigned char *>(arena),
                static_cast<const unsigned char *>(input_rows_data), static_cast<const Metadata *>(metadata), query_lengths,
                kv_lengths, spec, requests, status_word);
}

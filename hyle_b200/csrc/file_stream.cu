// File -> pinned host memory -> device, as a stream of chunks in file order.
//
// The reference feeds on-disk weight banks to the GPU through a pipeline of in-flight staging slots
// (include/hyle/compute/file_stream.h:23-31: `in_flight_slots`, `staging_bytes_per_slot`;
// include/hyle/compute/cuda_file_stream.h:10-14 binds it to a CUDA Queue with pinned staging;
// scheduling in src/compute_stream/file_stream.cc).  This is that pipeline for the one consumer this
// library has, a kernel that decodes Q8_0 blocks (the GGUF Q8_0 weight layout is this library's
// carrier: rows of k/32 blocks of 34 bytes, src/compute_ops/low_precision.cc:269-297):
//
//   reader thread:   pread(chunk) into pinned slot s  ->  cudaMemcpyAsync(device slot s) on the copy
//                    stream  ->  event copied[s]
//   next(consumer):  the consumer's stream waits for copied[s] (device-side), gets the device pointer;
//                    the call also records done[previous slot] on the consumer's stream, which the copy
//                    stream waits for before it overwrites that slot
//
// so disk reads, host->device copies and the consumer's kernels overlap, the host never waits for the
// GPU except to reuse a pinned slot whose copy is still in flight, and NOTHING allocates after open():
// `slots` pinned buffers, `slots` device buffers, 2 x `slots` events, one stream, one thread.
#include <atomic>
#include <cerrno>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include "common.cuh"

namespace {

constexpr uint32_t kMaxSlots = 16;
constexpr uint64_t kDefaultChunkBytes = 8ull << 20;
constexpr uint32_t kMaxReaders = 16;
// default: half of the host's hardware threads, at most 8 (one thread moves about 10 GB/s out of the page cache)
uint32_t default_readers() {
  const unsigned threads = std::thread::hardware_concurrency();
  const unsigned half = threads / 2;
  return half < 1 ? 1u : (half > 8 ? 8u : half);
}
constexpr uint64_t kPieceBytes = 1ull << 20;  // what one pread call of one reader covers

}  // namespace

struct hyle_b200_file_stream {
  int fd = -1;
  int device = 0;
  uint64_t file_offset = 0, bytes = 0, chunk_bytes = 0, chunks = 0;
  uint32_t slots = 0;
  unsigned char *pinned[kMaxSlots] = {};
  unsigned char *resident[kMaxSlots] = {};
  cudaEvent_t copied[kMaxSlots] = {};  // the H2D copy into slot s has completed
  cudaEvent_t done[kMaxSlots] = {};    // the consumer has finished with slot s
  cudaStream_t copy_stream = nullptr;
  std::thread reader;
  std::mutex mutex;
  std::condition_variable changed;
  uint64_t issued = 0;      // chunks whose copy has been issued (reader -> consumer)
  uint64_t handed = 0;      // chunks handed to the consumer by next()
  uint64_t released = 0;    // chunks whose done[] event has been recorded (consumer -> reader)
  int error = HYLE_B200_OK; // first reader failure
  bool closing = false;
  uint64_t file_bytes = 0;  // size of the file at open
  uint64_t group_chunks = 0;  // chunks copied by read_group so far (slot rotation across groups)
  hyle_b200_file_stream_report report{};

  // A chunk is read by `readers` threads at once, a piece of kPieceBytes each (one thread copies from the page
  // cache at about 10 GB/s; the host-to-device link takes five times that).  The coordinator (the reader
  // thread, or the caller of read_group) posts a job and takes pieces itself; helpers take the rest.
  uint32_t readers = 1;
  std::thread helpers[kMaxReaders];
  std::mutex job_mutex;
  std::condition_variable job_posted, job_finished;
  uint64_t job_generation = 0;
  unsigned char *job_target = nullptr;
  uint64_t job_offset = 0, job_bytes = 0, job_pieces = 0;
  std::atomic<uint64_t> job_ticket{0};  // generation << 32 | next piece
  uint64_t job_done = 0, job_calls = 0;
  bool job_failed = false, helpers_stop = false;

  // Pieces of job `generation` until none is left.  The ticket holds the job's generation beside the next
  // piece, and a piece is claimed by compare-and-swap on the pair: a helper that wakes up late can never
  // claim (or skip) a piece of a job it was not woken for.  The job's fields are written before the
  // ticket is published (release) and read after it is seen (acquire).
  void take_pieces(uint64_t generation) {
    uint64_t calls = 0, finished = 0;
    bool failed = false;
    for (;;) {
      uint64_t ticket = job_ticket.load(std::memory_order_acquire);
      uint64_t piece = 0;
      bool claimed = false;
      while ((ticket >> 32) == (generation & 0xffffffffull) && (ticket & 0xffffffffull) < job_pieces) {
        if (job_ticket.compare_exchange_weak(ticket, ticket + 1, std::memory_order_acq_rel, std::memory_order_acquire)) {
          piece = ticket & 0xffffffffull;
          claimed = true;
          break;
        }
      }
      if (!claimed) break;
      const uint64_t begin = piece * kPieceBytes, size = job_bytes - begin < kPieceBytes ? job_bytes - begin : kPieceBytes;
      uint64_t have = 0;
      while (have < size && !failed) {
        const ssize_t got = pread(fd, job_target + begin + have, size - have, static_cast<off_t>(job_offset + begin + have));
        ++calls;
        if (got < 0 && errno == EINTR) continue;
        if (got <= 0) failed = true;  // error, or the file ends inside the range
        else have += static_cast<uint64_t>(got);
      }
      ++finished;
    }
    if (finished == 0) return;
    std::lock_guard lock(job_mutex);
    job_done += finished;
    job_calls += calls;
    job_failed = job_failed || failed;
    if (job_done == job_pieces) job_finished.notify_all();
  }

  void helper_loop() {
    uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock lock(job_mutex);
        job_posted.wait(lock, [&] { return helpers_stop || job_generation != seen; });
        if (helpers_stop) return;
        seen = job_generation;
      }
      take_pieces(seen);
    }
  }

  // bytes of the file at `offset` -> target, by all readers; the number of pread calls comes back in *calls.
  // One coordinator at a time (the reader thread, or the caller of read_group).
  bool read_parallel(unsigned char *target, uint64_t offset, uint64_t size, uint64_t *calls) {
    uint64_t generation = 0;
    {
      std::lock_guard lock(job_mutex);
      job_target = target;
      job_offset = offset;
      job_bytes = size;
      job_pieces = (size + kPieceBytes - 1) / kPieceBytes;
      job_done = 0;
      job_calls = 0;
      job_failed = false;
      generation = ++job_generation;
      job_ticket.store((generation & 0xffffffffull) << 32, std::memory_order_release);
    }
    if (job_pieces == 0) {
      *calls = 0;
      return true;
    }
    if (readers > 1 && job_pieces > 1) job_posted.notify_all();
    take_pieces(generation);
    std::unique_lock lock(job_mutex);
    job_finished.wait(lock, [&] { return job_done == job_pieces; });
    *calls = job_calls;
    return !job_failed;
  }

  uint64_t chunk_size(uint64_t index) const {
    const uint64_t start = index * chunk_bytes;
    return bytes - start < chunk_bytes ? bytes - start : chunk_bytes;
  }

  void fail(int code) {
    std::lock_guard lock(mutex);
    if (error == HYLE_B200_OK) error = code;
    changed.notify_all();
  }

  void read_loop() {
    if (cudaSetDevice(device) != cudaSuccess) return fail(HYLE_B200_INVALID_VALUE);
    for (uint64_t index = 0; index < chunks; ++index) {
      const uint32_t slot = static_cast<uint32_t>(index % slots);
      if (index >= slots) {
        // slot reuse: its previous chunk must have been released by the consumer (the event exists
        // then), and its previous copy must have left the pinned buffer
        std::unique_lock lock(mutex);
        changed.wait(lock, [&] { return closing || released > index - slots; });
        if (closing) return;
        lock.unlock();
        if (cudaEventSynchronize(copied[slot]) != cudaSuccess) return fail(HYLE_B200_IO_ERROR);
        if (cudaStreamWaitEvent(copy_stream, done[slot], 0) != cudaSuccess) return fail(HYLE_B200_IO_ERROR);
      }
      const uint64_t size = chunk_size(index);
      uint64_t calls = 0;
      if (!read_parallel(pinned[slot], file_offset + index * chunk_bytes, size, &calls)) return fail(HYLE_B200_IO_ERROR);
      if (cudaMemcpyAsync(resident[slot], pinned[slot], size, cudaMemcpyHostToDevice, copy_stream) != cudaSuccess ||
          cudaEventRecord(copied[slot], copy_stream) != cudaSuccess)
        return fail(HYLE_B200_IO_ERROR);
      {
        std::lock_guard lock(mutex);  // the report is read under the same lock
        report.io_calls += calls;
        report.bytes_read += size;
        ++report.copies;
        report.bytes_copied += size;
        issued = index + 1;
        if (closing) return;
      }
      changed.notify_all();
    }
  }
};

extern "C" int hyle_b200_file_stream_open(const char *path, uint64_t file_offset, uint64_t bytes,
                                          const hyle_b200_file_stream_options *options, hyle_b200_file_stream **out) {
  if (out == nullptr) return HYLE_B200_INVALID_VALUE;
  *out = nullptr;
  if (path == nullptr) return HYLE_B200_INVALID_VALUE;
  uint64_t chunk = options != nullptr && options->chunk_bytes != 0 ? options->chunk_bytes : kDefaultChunkBytes;
  uint32_t slots = options != nullptr && options->slots != 0 ? options->slots : 4;
  const uint64_t granule = options != nullptr && options->chunk_granule != 0 ? options->chunk_granule : 1;
  if (slots < 2 || slots > kMaxSlots || chunk < granule) return HYLE_B200_INVALID_VALUE;
  chunk -= chunk % granule;  // whole records per chunk (34-byte Q8_0 blocks, rows ...)
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return HYLE_B200_IO_ERROR;
  struct stat info {};
  if (fstat(fd, &info) != 0 || static_cast<uint64_t>(info.st_size) < file_offset ||
      static_cast<uint64_t>(info.st_size) - file_offset < bytes) {
    ::close(fd);
    return HYLE_B200_IO_ERROR;  // the range is not inside the file
  }
  auto *stream = new (std::nothrow) hyle_b200_file_stream();
  if (stream == nullptr) {
    ::close(fd);
    return static_cast<int>(cudaErrorMemoryAllocation);
  }
  stream->fd = fd;
  stream->file_bytes = static_cast<uint64_t>(info.st_size);
  stream->file_offset = file_offset;
  stream->bytes = bytes;
  stream->chunk_bytes = chunk;
  stream->chunks = (bytes + chunk - 1) / chunk;
  stream->slots = slots;
  stream->readers = options != nullptr && options->readers != 0 ? options->readers : default_readers();
  if (stream->readers > kMaxReaders) stream->readers = kMaxReaders;
  cudaError_t error = cudaGetDevice(&stream->device);
  if (error == cudaSuccess) error = cudaStreamCreateWithFlags(&stream->copy_stream, cudaStreamNonBlocking);
  for (uint32_t s = 0; s < slots && error == cudaSuccess; ++s) {
    error = cudaHostAlloc(reinterpret_cast<void **>(&stream->pinned[s]), chunk, cudaHostAllocDefault);
    if (error == cudaSuccess && bytes != 0) error = cudaMalloc(reinterpret_cast<void **>(&stream->resident[s]), chunk);
    if (error == cudaSuccess) error = cudaEventCreateWithFlags(&stream->copied[s], cudaEventDisableTiming);
    if (error == cudaSuccess) error = cudaEventCreateWithFlags(&stream->done[s], cudaEventDisableTiming);
  }
  if (error != cudaSuccess) {
    hyle_b200_file_stream_close(stream);
    return static_cast<int>(error);
  }
  stream->report.staging_bytes = chunk * slots;
  stream->report.device_bytes = bytes != 0 ? chunk * slots : 0;
  stream->report.chunk_bytes = chunk;
  stream->report.chunks = stream->chunks;
  for (uint32_t h = 1; h < stream->readers; ++h) stream->helpers[h] = std::thread([stream] { stream->helper_loop(); });
  if (stream->chunks != 0) stream->reader = std::thread([stream] { stream->read_loop(); });
  *out = stream;
  return HYLE_B200_OK;
}

extern "C" int hyle_b200_file_stream_next(hyle_b200_file_stream *stream, hyle_b200_stream_t consumer, const void **device_chunk,
                                          uint64_t *chunk_bytes, uint64_t *chunk_offset) {
  if (stream == nullptr || device_chunk == nullptr || chunk_bytes == nullptr) return HYLE_B200_INVALID_VALUE;
  *device_chunk = nullptr;
  *chunk_bytes = 0;
  auto consumer_stream = reinterpret_cast<cudaStream_t>(consumer);
  // whatever the consumer enqueued on the previous chunk is what must finish before its slot is reused
  if (stream->handed != 0 && stream->released < stream->handed) {
    const uint32_t previous = static_cast<uint32_t>((stream->handed - 1) % stream->slots);
    const cudaError_t recorded = cudaEventRecord(stream->done[previous], consumer_stream);
    if (recorded != cudaSuccess) return static_cast<int>(recorded);
    {
      std::lock_guard lock(stream->mutex);
      stream->released = stream->handed;
    }
    stream->changed.notify_all();
  }
  if (stream->handed == stream->chunks) return HYLE_B200_OK;  // end of the range: *chunk_bytes == 0
  const uint64_t index = stream->handed;
  {
    std::unique_lock lock(stream->mutex);
    stream->changed.wait(lock, [&] { return stream->issued > index || stream->error != HYLE_B200_OK; });
    if (stream->issued <= index) return stream->error;
  }
  const uint32_t slot = static_cast<uint32_t>(index % stream->slots);
  const cudaError_t waited = cudaStreamWaitEvent(consumer_stream, stream->copied[slot], 0);
  if (waited != cudaSuccess) return static_cast<int>(waited);
  *device_chunk = stream->resident[slot];
  *chunk_bytes = stream->chunk_size(index);
  if (chunk_offset != nullptr) *chunk_offset = index * stream->chunk_bytes;
  stream->handed = index + 1;
  return HYLE_B200_OK;
}

// A group of byte ranges -> device destinations of the caller's own, through the pinned slots: the calling
// thread reads chunk k + 1 while the copy of chunk k is in flight.
extern "C" int hyle_b200_file_stream_read_group(hyle_b200_file_stream *stream, hyle_b200_stream_t consumer,
                                                const hyle_b200_file_range *ranges, uint32_t count) {
  if (stream == nullptr || (ranges == nullptr && count != 0) || stream->chunks != 0) return HYLE_B200_INVALID_VALUE;
  for (uint32_t r = 0; r < count; ++r) {
    if (ranges[r].bytes != 0 && ranges[r].destination == nullptr) return HYLE_B200_INVALID_VALUE;
    if (ranges[r].file_offset > stream->file_bytes || stream->file_bytes - ranges[r].file_offset < ranges[r].bytes)
      return HYLE_B200_IO_ERROR;  // nothing has been copied
  }
  bool copied_any = false;
  for (uint32_t r = 0; r < count; ++r) {
    for (uint64_t done_bytes = 0; done_bytes < ranges[r].bytes;) {
      const uint32_t slot = static_cast<uint32_t>(stream->group_chunks % stream->slots);
      // the slot's previous copy must have left the pinned buffer (an event never recorded is complete)
      if (cudaEventSynchronize(stream->copied[slot]) != cudaSuccess) return HYLE_B200_IO_ERROR;
      const uint64_t size = ranges[r].bytes - done_bytes < stream->chunk_bytes ? ranges[r].bytes - done_bytes : stream->chunk_bytes;
      uint64_t calls = 0;
      if (!stream->read_parallel(stream->pinned[slot], ranges[r].file_offset + done_bytes, size, &calls))
        return HYLE_B200_IO_ERROR;  // the file shrank after open, or a read error
      cudaError_t error = cudaMemcpyAsync(static_cast<unsigned char *>(ranges[r].destination) + done_bytes, stream->pinned[slot],
                                          size, cudaMemcpyHostToDevice, stream->copy_stream);
      if (error == cudaSuccess) error = cudaEventRecord(stream->copied[slot], stream->copy_stream);
      if (error != cudaSuccess) return static_cast<int>(error);
      {
        std::lock_guard lock(stream->mutex);
        stream->report.io_calls += calls;
        stream->report.bytes_read += size;
        stream->report.bytes_copied += size;
        ++stream->report.copies;
      }
      ++stream->group_chunks;
      done_bytes += size;
      copied_any = true;
    }
  }
  if (!copied_any) return HYLE_B200_OK;
  // the consumer's stream continues after the group's last copy
  const uint32_t last = static_cast<uint32_t>((stream->group_chunks - 1) % stream->slots);
  const cudaError_t chained = cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(consumer), stream->copied[last], 0);
  return chained == cudaSuccess ? HYLE_B200_OK : static_cast<int>(chained);
}

extern "C" int hyle_b200_file_stream_get_report(hyle_b200_file_stream *stream, hyle_b200_file_stream_report *report) {
  if (stream == nullptr || report == nullptr) return HYLE_B200_INVALID_VALUE;
  std::lock_guard lock(stream->mutex);
  *report = stream->report;
  return HYLE_B200_OK;
}

extern "C" int hyle_b200_file_stream_close(hyle_b200_file_stream *stream) {
  if (stream == nullptr) return HYLE_B200_OK;
  {
    std::lock_guard lock(stream->mutex);
    stream->closing = true;
  }
  stream->changed.notify_all();
  if (stream->reader.joinable()) stream->reader.join();
  {
    std::lock_guard lock(stream->job_mutex);
    stream->helpers_stop = true;
  }
  stream->job_posted.notify_all();
  for (auto &helper : stream->helpers)
    if (helper.joinable()) helper.join();
  int device = 0;
  const bool switched = cudaGetDevice(&device) == cudaSuccess && device != stream->device && cudaSetDevice(stream->device) == cudaSuccess;
  if (stream->copy_stream != nullptr) cudaStreamSynchronize(stream->copy_stream);
  for (uint32_t s = 0; s < kMaxSlots; ++s) {
    // a consumer kernel may still be reading a device slot: the slot is freed after its last event
    if (stream->done[s] != nullptr) {
      cudaEventSynchronize(stream->done[s]);
      cudaEventDestroy(stream->done[s]);
    }
    if (stream->copied[s] != nullptr) cudaEventDestroy(stream->copied[s]);
    if (stream->resident[s] != nullptr) cudaFree(stream->resident[s]);
    if (stream->pinned[s] != nullptr) cudaFreeHost(stream->pinned[s]);
  }
  if (stream->copy_stream != nullptr) cudaStreamDestroy(stream->copy_stream);
  if (switched) cudaSetDevice(device);
  if (stream->fd >= 0) ::close(stream->fd);
  delete stream;
  return HYLE_B200_OK;
}

// The Q8_0 bank of `count` values at `file_offset` of `path`, decoded to bf16 at `out` (device), chunk by
// chunk on `consumer`: disk, PCIe and the decode kernel overlap.  Returns after the last launch is
// enqueued and the pipeline is torn down (which waits for the last decode).
extern "C" int hyle_b200_q8_0_decode_file_bf16(hyle_b200_stream_t consumer, const char *path, uint64_t file_offset, uint64_t count,
                                               void *out_bf16, const hyle_b200_file_stream_options *options,
                                               hyle_b200_file_stream_report *report) {
  if (count % 32 != 0 || (count != 0 && out_bf16 == nullptr)) return HYLE_B200_INVALID_VALUE;
  hyle_b200_file_stream_options chosen{};
  if (options != nullptr) chosen = *options;
  chosen.chunk_granule = 34 * 8;  // whole blocks, and chunk offsets that keep the decoded output 16-byte aligned (8 blocks = 512 B of bf16)
  hyle_b200_file_stream *stream = nullptr;
  int code = hyle_b200_file_stream_open(path, file_offset, count / 32 * 34, &chosen, &stream);
  if (code != HYLE_B200_OK) return code;
  auto *out = static_cast<unsigned char *>(out_bf16);
  for (;;) {
    const void *chunk = nullptr;
    uint64_t bytes = 0, offset = 0;
    code = hyle_b200_file_stream_next(stream, consumer, &chunk, &bytes, &offset);
    if (code != HYLE_B200_OK || bytes == 0) break;
    const uint64_t values = bytes / 34 * 32;
    code = hyle_b200_q8_0_decode_bf16(consumer, chunk, values, out + offset / 34 * 32 * 2);
    if (code != HYLE_B200_OK) break;
  }
  if (report != nullptr) hyle_b200_file_stream_get_report(stream, report);
  hyle_b200_file_stream_close(stream);
  return code;
}

// Scan{axis = -1, exclusive}: prefix sums along the rows of a dense [rows, cols] tensor
// (include/hyle/compute/operation.h:314-321; CPU route src/compute_provider_ggml/standard_index.cc:113-157).
//   f32: float accumulation; the operator permits reassociation, so the blocked order below is allowed.
//   i32: when any inclusive prefix (the final total included, also for an exclusive scan) leaves the
//        int32 range the call reports it and writes NO output, as the reference does.  That takes a
//        decision about the whole tensor before the first store, i.e. two kernels.  The first one only
//        decides: per row the sum of magnitudes (a plain reduction, loads marked evict-last so that the
//        row stays in L2); a row whose magnitudes sum to at most INT32_MAX cannot overflow, any other
//        row (rare) is checked exactly by its CTA.  The second one is the f32 scan's walk on 32-bit
//        integers with wrap-around arithmetic: every prefix is known to fit, so sums modulo 2^32 are
//        the true values, and its loads hit L2.
//
// HBM-bound: 8 bytes per value.  One CTA walks a row in chunks of 4 values per thread with the row's
// running total carried in a register; the (row, chunk) steps of a CTA form one sequence and the loads
// of the next step are issued before the current one is combined, so a chunk's shuffles and its single
// barrier hide behind the next chunk's memory latency.  Many short rows take 256-thread CTAs (eight
// per SM), few long rows 1024-thread CTAs (two per SM).
#include <type_traits>

#include "common.cuh"

namespace hb {
namespace {

constexpr unsigned kScanOverflow = HYLE_B200_STATUS_SCAN_OVERFLOW;

template <class T> struct Quad { T v[4]; };

// kStream: the values are not needed again (evict-first); the checking pass of the integer scan
// loads normally so that the writing pass finds rows of moderate size in L2.
template <class T, bool kVector, bool kStream>
__device__ __forceinline__ Quad<T> load_quad(const T *row, uint64_t first, uint64_t cols) {
  Quad<T> q;
  if constexpr (kVector) {
    if (first < cols) {
      const uint4 *address = reinterpret_cast<const uint4 *>(row + first);
      const uint4 w = kStream ? ld_stream(address) : __ldg(address);
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) memcpy(&q.v[k], &words[k], 4);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) q.v[k] = T(0);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) q.v[k] = first + k < cols ? row[first + k] : T(0);
  }
  return q;
}

template <class T, bool kVector>
__device__ __forceinline__ void store_quad(T *row, uint64_t first, uint64_t cols, const T (&v)[4]) {
  if constexpr (kVector) {
    if (first < cols) {
      uint32_t words[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) memcpy(&words[k], &v[k], 4);
      st_stream(reinterpret_cast<uint4 *>(row + first), make_uint4(words[0], words[1], words[2], words[3]));
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (first + k < cols) row[first + k] = v[k];
  }
}

template <class Acc>
__device__ __forceinline__ Acc warp_inclusive(Acc value, unsigned lane) {
#pragma unroll
  for (int step = 1; step < kWarpSize; step <<= 1) {
    const Acc below = __shfl_up_sync(kFullMask, value, step);
    if (lane >= static_cast<unsigned>(step)) value += below;
  }
  return value;
}

__device__ __forceinline__ uint64_t scan_policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ int4 load_keep(const int4 *p, uint64_t policy) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.s32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ unsigned long long magnitude(int32_t v) {
  return static_cast<unsigned long long>(v < 0 ? 0u - static_cast<uint32_t>(v) : static_cast<uint32_t>(v));
}

// The deciding pass of the checked i32 scan.  CTA per row (grid-stride): sum of magnitudes; above
// INT32_MAX the CTA checks the row's prefixes exactly (each thread a contiguous segment: its sum and
// the extremes of its running sum, then the segments in order).
constexpr int kCheckThreads = 256;
template <bool kVector>
__global__ void __launch_bounds__(kCheckThreads)
scan_i32_check_kernel(const int32_t *__restrict__ in, uint64_t rows, uint64_t cols, unsigned *status) {
  grid_dependency_sync();
  constexpr int kWarps = kCheckThreads / kWarpSize;
  __shared__ unsigned long long s_warp[kWarps];
  __shared__ long long s_sum[kCheckThreads], s_low[kCheckThreads], s_high[kCheckThreads];
  __shared__ int s_exact;
  const unsigned lane = threadIdx.x % kWarpSize, warp = threadIdx.x / kWarpSize;
  const uint64_t policy = scan_policy_evict_last();
  bool bad = false;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int32_t *values = in + row * cols;
    unsigned long long total = 0;
    if constexpr (kVector) {
      const int4 *vectors = reinterpret_cast<const int4 *>(values);
      const uint64_t count = cols / 4;
      uint64_t v = threadIdx.x;
      for (; v + 3 * kCheckThreads < count; v += 4 * kCheckThreads) {
        int4 q[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) q[k] = load_keep(vectors + v + k * kCheckThreads, policy);
#pragma unroll
        for (int k = 0; k < 4; ++k) total += magnitude(q[k].x) + magnitude(q[k].y) + magnitude(q[k].z) + magnitude(q[k].w);
      }
      for (; v < count; v += kCheckThreads) {
        const int4 q = load_keep(vectors + v, policy);
        total += magnitude(q.x) + magnitude(q.y) + magnitude(q.z) + magnitude(q.w);
      }
    } else {
      for (uint64_t i = threadIdx.x; i < cols; i += kCheckThreads) total += magnitude(values[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(kFullMask, total, o);
    if (lane == 0) s_warp[warp] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long all = 0;
      for (int w = 0; w < kWarps; ++w) all += s_warp[w];
      s_exact = all > static_cast<unsigned long long>(INT32_MAX);
    }
    __syncthreads();
    if (s_exact) {  // rare: the magnitudes alone do not rule an overflow out
      const uint64_t segment = (cols + kCheckThreads - 1) / kCheckThreads;
      const uint64_t begin = min(threadIdx.x * segment, cols), end = min(begin + segment, cols);
      long long sum = 0, low = 0, high = 0;  // extremes of the running sum inside the segment (0 = before it)
      for (uint64_t i = begin; i < end; ++i) {
        sum += values[i];
        low = sum < low ? sum : low;
        high = sum > high ? sum : high;
      }
      s_sum[threadIdx.x] = sum, s_low[threadIdx.x] = low, s_high[threadIdx.x] = high;
      __syncthreads();
      if (threadIdx.x == 0) {
        long long base = 0;
        for (int t = 0; t < kCheckThreads; ++t) {
          if (base + s_low[t] < static_cast<long long>(INT32_MIN) || base + s_high[t] > static_cast<long long>(INT32_MAX)) bad = true;
          base += s_sum[t];
        }
      }
    }
    __syncthreads();  // the shared arrays are reused by the next row
  }
  if (bad) atomicOr(status, kScanOverflow);
}

// The same decision with a WARP per row, for rows of at most 16384 values: no barrier at all, eight
// 16-byte loads in flight per lane.  The exact check of a suspicious row is done by its warp: each lane
// a contiguous segment, the segments chained by shuffles.
template <bool kVector>
__global__ void __launch_bounds__(kCheckThreads)
scan_i32_check_warp_kernel(const int32_t *__restrict__ in, uint64_t rows, uint32_t cols, unsigned *status) {
  grid_dependency_sync();
  const unsigned lane = threadIdx.x % kWarpSize;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (kCheckThreads / kWarpSize);
  const uint64_t policy = scan_policy_evict_last();
  bool bad = false;
  for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (kCheckThreads / kWarpSize) + threadIdx.x / kWarpSize; row < rows;
       row += warps) {
    const int32_t *values = in + row * cols;
    unsigned long long total = 0;
    if constexpr (kVector) {
      const int4 *vectors = reinterpret_cast<const int4 *>(values);
      const uint32_t count = cols / 4;
      uint32_t v = lane;
      for (; v + 7 * kWarpSize < count; v += 8 * kWarpSize) {
        int4 q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) q[k] = load_keep(vectors + v + k * kWarpSize, policy);
#pragma unroll
        for (int k = 0; k < 8; ++k) total += magnitude(q[k].x) + magnitude(q[k].y) + magnitude(q[k].z) + magnitude(q[k].w);
      }
      for (; v < count; v += kWarpSize) {
        const int4 q = load_keep(vectors + v, policy);
        total += magnitude(q.x) + magnitude(q.y) + magnitude(q.z) + magnitude(q.w);
      }
    } else {
      for (uint32_t i = lane; i < cols; i += kWarpSize) total += magnitude(values[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(kFullMask, total, o);
    if (total > static_cast<unsigned long long>(INT32_MAX)) {  // warp-uniform, rare
      const uint32_t segment = (cols + kWarpSize - 1) / kWarpSize;
      const uint32_t begin = min(lane * segment, cols), end = min(begin + segment, cols);
      long long sum = 0, low = 0, high = 0;
      for (uint32_t i = begin; i < end; ++i) {
        sum += values[i];
        low = sum < low ? sum : low;
        high = sum > high ? sum : high;
      }
      long long base = sum;  // exclusive prefix of the segment sums, lane by lane
#pragma unroll
      for (int step = 1; step < kWarpSize; step <<= 1) {
        const long long below = __shfl_up_sync(kFullMask, base, step);
        if (lane >= static_cast<unsigned>(step)) base += below;
      }
      base -= sum;
      bad |= base + low < static_cast<long long>(INT32_MIN) || base + high > static_cast<long long>(INT32_MAX);
    }
  }
  if (__any_sync(kFullMask, bad) && lane == 0) atomicOr(status, kScanOverflow);
}

// kWrite = false walks without storing (kept for the checking instantiation of wide accumulators).
template <class T, class Acc, int kThreads, bool kVector, bool kWrite>
__global__ void __launch_bounds__(kThreads)
scan_rows_kernel(const T *__restrict__ in, T *__restrict__ out, uint64_t rows, uint64_t cols, int exclusive, unsigned *status) {
  grid_dependency_sync();
  constexpr int kWarps = kThreads / kWarpSize;
  constexpr uint64_t kChunk = static_cast<uint64_t>(kThreads) * 4;
  constexpr bool kChecked = !std::is_same<T, float>::value;  // the integer scan: decided by the pass before
  __shared__ Acc s_total[2][kWarps];
  if constexpr (kChecked && kWrite) {
    if ((*reinterpret_cast<volatile unsigned *>(status) & kScanOverflow) != 0) return;  // the check failed: no output
  }
  const unsigned lane = threadIdx.x % kWarpSize, warp = threadIdx.x / kWarpSize;
  const uint64_t chunks = (cols + kChunk - 1) / kChunk;
  const uint64_t mine = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint64_t steps = mine * chunks;
  bool bad = false;
  Acc carry = 0;
  uint64_t row = blockIdx.x, chunk = 0;
  Quad<T> next = steps ? load_quad<T, kVector, kWrite>(in + row * cols, threadIdx.x * 4ull, cols) : Quad<T>{};
  for (uint64_t step = 0; step < steps; ++step) {
    const Quad<T> q = next;
    const uint64_t at_row = row, at = chunk * kChunk + threadIdx.x * 4ull;
    if (++chunk == chunks) chunk = 0, row += gridDim.x;
    if (step + 1 < steps) next = load_quad<T, kVector, kWrite>(in + row * cols, chunk * kChunk + threadIdx.x * 4ull, cols);
    if (at < kChunk) carry = 0;  // first chunk of a row
    Acc p[4];
    p[0] = static_cast<Acc>(q.v[0]);
#pragma unroll
    for (int k = 1; k < 4; ++k) p[k] = p[k - 1] + static_cast<Acc>(q.v[k]);
    const Acc through = warp_inclusive(p[3], lane);  // this warp's total up to and including this lane
    Acc (&totals)[kWarps] = s_total[step & 1];
    if (lane == kWarpSize - 1) totals[warp] = through;
    __syncthreads();
    // every warp scans the warp totals for itself: no second barrier, and the buffers alternate
    const Acc listed = lane < kWarps ? totals[lane] : Acc(0);
    const Acc upto = warp_inclusive(listed, lane);
    // exclusive prefixes are fetched from the neighbour, never formed as "inclusive - own": with an
    // infinity in the chunk that difference would be NaN for values in front of it
    const Acc upto_previous_warp = __shfl_sync(kFullMask, upto, (warp + kWarpSize - 1) % kWarpSize);
    const Acc before_warp = warp == 0 ? Acc(0) : upto_previous_warp;
    const Acc chunk_total = __shfl_sync(kFullMask, upto, kWarps - 1);
    const Acc through_previous_lane = __shfl_up_sync(kFullMask, through, 1);
    const Acc before_lane = lane == 0 ? Acc(0) : through_previous_lane;
    const Acc base = carry + (before_warp + before_lane);
    carry += chunk_total;
    if constexpr (kChecked && !kWrite) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const long long value = static_cast<long long>(base + p[k]);
        bad |= value < static_cast<long long>(INT32_MIN) || value > static_cast<long long>(INT32_MAX);
      }
    }
    if constexpr (kWrite) {
      T result[4];
      if (exclusive) {
        result[0] = static_cast<T>(base);
#pragma unroll
        for (int k = 1; k < 4; ++k) result[k] = static_cast<T>(base + p[k - 1]);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) result[k] = static_cast<T>(base + p[k]);
      }
      store_quad<T, kVector>(out + at_row * cols, at, cols, result);
    }
  }
  if constexpr (kChecked && !kWrite) {
    if (__any_sync(kFullMask, bad) && lane == 0) atomicOr(status, kScanOverflow);
  }
}

// Many short rows: a WARP per row.  A lane takes four consecutive values of each 128-value piece, kPieces
// pieces (16: 8 KB of a row per warp) are loaded before the first is scanned (independent 16-byte loads in
// flight: with one warp per row there are few warps, so each must keep many loads going), and a piece costs one
// warp scan of the lanes' totals -- no shared memory and no barrier, which is what the CTA form above spends
// most of its stalls on when a row is only a few of its chunks long.
template <class T, class Acc, bool kVector, bool kExclusive>
__global__ void __launch_bounds__(256)
scan_rows_warp_kernel(const T *__restrict__ in, T *__restrict__ out, uint64_t rows, uint32_t cols, unsigned *status) {
  grid_dependency_sync();
  constexpr int kPieces = 16;
  constexpr bool kChecked = !std::is_same<T, float>::value;  // the integer scan: decided by the pass before
  if constexpr (kChecked) {
    if ((*reinterpret_cast<volatile unsigned *>(status) & kScanOverflow) != 0) return;  // the check failed: no output
  }
  const unsigned lane = threadIdx.x % kWarpSize;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x / kWarpSize);
  for (uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x / kWarpSize) + threadIdx.x / kWarpSize; row < rows; row += warps) {
    const T *row_in = in + row * cols;
    T *row_out = out + row * cols;
    Acc carry = 0;
    for (uint32_t first = 0; first < cols; first += kPieces * 128) {
      Quad<T> q[kPieces];
#pragma unroll
      for (int j = 0; j < kPieces; ++j) q[j] = load_quad<T, kVector, true>(row_in, first + j * 128 + lane * 4, cols);
#pragma unroll
      for (int j = 0; j < kPieces; ++j) {
        const uint32_t at = first + j * 128 + lane * 4;
        if (first + j * 128 >= cols) break;  // warp-uniform
        Acc p[4];
        p[0] = static_cast<Acc>(q[j].v[0]);
#pragma unroll
        for (int k = 1; k < 4; ++k) p[k] = p[k - 1] + static_cast<Acc>(q[j].v[k]);
        const Acc through = warp_inclusive(p[3], lane);
        // exclusive prefixes are fetched from the neighbour, never formed as "inclusive - own"
        const Acc through_previous_lane = __shfl_up_sync(kFullMask, through, 1);
        const Acc base = carry + (lane == 0 ? Acc(0) : through_previous_lane);
        carry += __shfl_sync(kFullMask, through, kWarpSize - 1);
        T result[4];
        if constexpr (kExclusive) {
          result[0] = static_cast<T>(base);
#pragma unroll
          for (int k = 1; k < 4; ++k) result[k] = static_cast<T>(base + p[k - 1]);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) result[k] = static_cast<T>(base + p[k]);
        }
        store_quad<T, kVector>(row_out, at, cols, result);
      }
    }
  }
}

template <class T, class Acc, bool kVector>
int launch_scan_warp(cudaStream_t stream, const T *in, T *out, uint64_t rows, uint64_t cols, int exclusive, unsigned *status) {
  const unsigned grid = clamp_grid((rows + 7) / 8, static_cast<uint64_t>(sm_count()) * 8);
  return launch(exclusive ? scan_rows_warp_kernel<T, Acc, kVector, true> : scan_rows_warp_kernel<T, Acc, kVector, false>, dim3(grid),
                dim3(256), 0, stream, in, out, rows, static_cast<uint32_t>(cols), status);
}

template <class T, class Acc, int kThreads, bool kVector, bool kWrite>
int launch_scan(cudaStream_t stream, const T *in, T *out, uint64_t rows, uint64_t cols, int exclusive, unsigned *status,
                unsigned ctas_per_sm) {
  const unsigned grid = clamp_grid(rows, static_cast<uint64_t>(sm_count()) * ctas_per_sm);
  return launch(scan_rows_kernel<T, Acc, kThreads, kVector, kWrite>, dim3(grid), dim3(kThreads), 0, stream, in, out, rows, cols,
                exclusive, status);
}

template <class T, class Acc, bool kWrite>
int dispatch_scan(cudaStream_t stream, const T *in, T *out, uint64_t rows, uint64_t cols, int exclusive, unsigned *status) {
  const bool vector = cols % 4 == 0 && aligned_to(in, 16) && aligned_to(out, 16);
  if (cols <= 16384 && rows >= static_cast<uint64_t>(sm_count()) * 8)  // many short rows: a warp each
    return vector ? launch_scan_warp<T, Acc, true>(stream, in, out, rows, cols, exclusive, status)
                  : launch_scan_warp<T, Acc, false>(stream, in, out, rows, cols, exclusive, status);
  // Wide CTAs when there are too few rows to fill the machine with narrow ones, or rows long
  // enough that a narrow CTA would spend its time on barriers.
  const bool wide = rows < static_cast<uint64_t>(sm_count()) * 8 || cols >= 32768;
  if (wide)
    return vector ? launch_scan<T, Acc, 1024, true, kWrite>(stream, in, out, rows, cols, exclusive, status, 2)
                  : launch_scan<T, Acc, 1024, false, kWrite>(stream, in, out, rows, cols, exclusive, status, 2);
  return vector ? launch_scan<T, Acc, 256, true, kWrite>(stream, in, out, rows, cols, exclusive, status, 8)
                : launch_scan<T, Acc, 256, false, kWrite>(stream, in, out, rows, cols, exclusive, status, 8);
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" int hyle_b200_scan(hyle_b200_stream_t stream, int dtype, const void *in, void *out, uint64_t rows, uint64_t cols,
                              int exclusive, uint32_t *status_word) {
  if (dtype != HYLE_B200_F32 && dtype != HYLE_B200_I32) return HYLE_B200_NOT_SUPPORTED;
  if (rows == 0 || cols == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr || !aligned_to(in, 4) || !aligned_to(out, 4) || in == out ||
      (dtype == HYLE_B200_I32 && (status_word == nullptr || !aligned_to(status_word, 4))))
    return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == HYLE_B200_F32)
    return dispatch_scan<float, float, true>(s, static_cast<const float *>(in), static_cast<float *>(out), rows, cols, exclusive,
                                             status_word);
  // pass 1 decides (and leaves the rows in L2), pass 2 scans modulo 2^32 and writes unless pass 1 objected
  const bool vector = cols % 4 == 0 && aligned_to(in, 16);
  const unsigned grid = clamp_grid(rows, static_cast<uint64_t>(sm_count()) * 8);
  int checked;
  if (cols <= 16384 && rows >= static_cast<uint64_t>(sm_count()) * 8) {  // many short rows: a warp each
    const unsigned warp_grid = clamp_grid((rows + kCheckThreads / kWarpSize - 1) / (kCheckThreads / kWarpSize),
                                          static_cast<uint64_t>(sm_count()) * 8);
    checked = vector ? launch(scan_i32_check_warp_kernel<true>, dim3(warp_grid), dim3(kCheckThreads), 0, s,
                              static_cast<const int32_t *>(in), rows, static_cast<uint32_t>(cols), status_word)
                     : launch(scan_i32_check_warp_kernel<false>, dim3(warp_grid), dim3(kCheckThreads), 0, s,
                              static_cast<const int32_t *>(in), rows, static_cast<uint32_t>(cols), status_word);
  } else {
    checked = vector ? launch(scan_i32_check_kernel<true>, dim3(grid), dim3(kCheckThreads), 0, s,
                              static_cast<const int32_t *>(in), rows, cols, status_word)
                     : launch(scan_i32_check_kernel<false>, dim3(grid), dim3(kCheckThreads), 0, s,
                              static_cast<const int32_t *>(in), rows, cols, status_word);
  }
  if (checked != HYLE_B200_OK) return checked;
  return dispatch_scan<uint32_t, uint32_t, true>(s, static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), rows, cols,
                                                 exclusive, status_word);
}

// sampling_ops::RandomBits and sampling_ops::Categorical (include/hyle/compute/sampling_ops.h:21-68).
//
// RandomBits is a counter-based generator with bit equality across backends: word w of row r is lane
// w % 4 of Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011) with
// key = identity[r][0..1] and counter = (w / 4 as 64 bits, identity[r][2], identity[r][3])
// (src/compute_provider_native/sampling.cc:76-88).  Pure 32-bit integer work, one block of four
// words per thread.
//
// Categorical draws one index per row of log-weights by inverting the cumulative distribution at
//   u = ((x0 * 2^20 + (x1 >> 12)) + 0.5) * 2^-52,   (x0, x1, ..) = block 0 of the row's identity
// (sampling.cc:157-161): the first index whose cumulative weight exp(x - max) exceeds total * u.
// The operator's contract leaves the draw algorithm and the floating math to each backend ("selected
// IDs need not match across backends"); what is fixed is the uniform above, that -inf has zero mass,
// that a row with NaN, +inf or no finite value is rejected, and the optional output
// log p = x[selected] - max - log(total).  Here: one CTA per row, the row read from HBM once (maximum,
// validity and weight sums together), then 1/16 of it again from L2 to locate the draw; f32 weights
// 2^(x log2e - shift) added in f64, fixed reduction orders: a row's result does not depend on the other
// rows, the grid or the run.
#include "common.cuh"

#include <math_constants.h>

namespace hb {
namespace {

// ---- Philox-4x32-10 ------------------------------------------------------------------------------
// The counter-based generator of Salmon, Moraes, Dror and Shaw, "Parallel random numbers: as easy as
// 1, 2, 3" (SC'11).  The round function, its multipliers (0xD2511F53, 0xCD9E8D57) and its key increments
// (0x9E3779B9, 0xBB67AE85) are those of the Random123 library, v1.14.0, Copyright 2010-2012
// D. E. Shaw Research, distributed under the BSD 3-Clause license (redistributions must retain that
// copyright notice, the list of conditions and the disclaimer of the Random123 LICENSE file).  The
// operator demands bit equality with the reference's generator
// (third_party/random123_counter/philox.h), so the arithmetic below is necessarily the published one;
// ten rounds, the counter in words 0-1, the identity's words 2-3 beside it and words 0-1 as the key.
struct Words {
  uint32_t x0, x1, x2, x3;
};

// One widening multiply instruction gives both halves of a product.
__device__ __forceinline__ uint64_t multiply_wide(uint32_t a, uint32_t b) {
  uint64_t product;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(product) : "r"(a), "r"(b));
  return product;
}

// The ten round keys of one identity: the same for every block of its row.
struct RoundKeys {
  uint32_t k0[10], k1[10];
};
__device__ __forceinline__ RoundKeys round_keys(uint32_t key0, uint32_t key1) {
  RoundKeys keys;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    keys.k0[round] = key0 + static_cast<uint32_t>(round) * 0x9e3779b9u;
    keys.k1[round] = key1 + static_cast<uint32_t>(round) * 0xbb67ae85u;
  }
  return keys;
}
__device__ __forceinline__ Words philox_rounds(Words v, const RoundKeys &keys) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = multiply_wide(0xd2511f53u, v.x0), p1 = multiply_wide(0xcd9e8d57u, v.x2);
    v = Words{static_cast<uint32_t>(p1 >> 32) ^ v.x1 ^ keys.k0[round], static_cast<uint32_t>(p1),
              static_cast<uint32_t>(p0 >> 32) ^ v.x3 ^ keys.k1[round], static_cast<uint32_t>(p0)};
  }
  return v;
}

__device__ __forceinline__ Words philox_block(const uint32_t *identity, uint64_t index) {
  const Words v{static_cast<uint32_t>(index), static_cast<uint32_t>(index >> 32), identity[2], identity[3]};
  return philox_rounds(v, round_keys(identity[0], identity[1]));
}

constexpr int kBitsThreads = 256;
constexpr int kBitsSpan = 16;  // blocks per lane and span

// Rows of few words (RandomBits{8}: two blocks per row): one block per thread, rows and blocks flattened.
__global__ void __launch_bounds__(kBitsThreads)
random_bits_block_kernel(const uint32_t *__restrict__ identities, uint32_t *out, uint64_t rows, uint32_t words) {
  grid_dependency_sync();
  const uint64_t blocks_per_row = (static_cast<uint64_t>(words) + 3) / 4;
  const uint64_t total = rows * blocks_per_row;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kBitsThreads;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBitsThreads + threadIdx.x; i < total; i += stride) {
    const uint64_t row = i / blocks_per_row, block = i - row * blocks_per_row;
    const Words w = philox_block(identities + row * 4, block);
    uint32_t *dst = out + row * words + block * 4;
    const uint32_t left = words - static_cast<uint32_t>(block * 4);
    if (left >= 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      *reinterpret_cast<uint4 *>(dst) = make_uint4(w.x0, w.x1, w.x2, w.x3);
    } else {
      dst[0] = w.x0;
      if (left > 1) dst[1] = w.x1;
      if (left > 2) dst[2] = w.x2;
      if (left > 3) dst[3] = w.x3;
    }
  }
}

// Long rows: a warp takes kBitsSpan x 32 consecutive blocks of one row.  Lane l computes blocks l, l + 32, ...
// of the span, so every store instruction of the warp writes 512 contiguous bytes, and the row's identity is
// loaded and its ten round keys are formed once per span instead of once per block.
__global__ void __launch_bounds__(kBitsThreads)
random_bits_span_kernel(const uint32_t *__restrict__ identities, uint32_t *out, uint64_t rows, uint32_t words) {
  grid_dependency_sync();
  const uint32_t blocks_per_row = (words + 3) / 4;
  const uint32_t spans_per_row = (blocks_per_row + kBitsSpan * 32 - 1) / (kBitsSpan * 32);
  const uint64_t total = rows * spans_per_row;
  const int lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (kBitsThreads / 32);
  for (uint64_t span = static_cast<uint64_t>(blockIdx.x) * (kBitsThreads / 32) + threadIdx.x / 32; span < total; span += warps) {
    const uint64_t row = span / spans_per_row;
    const uint32_t first = static_cast<uint32_t>(span - row * spans_per_row) * (kBitsSpan * 32);
    const uint32_t *identity = identities + row * 4;
    const uint32_t id0 = identity[0], id1 = identity[1], id2 = identity[2], id3 = identity[3];
    const RoundKeys keys = round_keys(id0, id1);
    uint32_t *row_out = out + row * words;
    const bool aligned = (reinterpret_cast<uintptr_t>(row_out) & 15) == 0;
#pragma unroll
    for (int k = 0; k < kBitsSpan; ++k) {
      const uint32_t block = first + k * 32 + lane;
      if (block < blocks_per_row) {
        const Words w = philox_rounds(Words{block, 0u, id2, id3}, keys);
        uint32_t *dst = row_out + static_cast<uint64_t>(block) * 4;
        const uint32_t left = words - block * 4;
        if (left >= 4 && aligned) {
          *reinterpret_cast<uint4 *>(dst) = make_uint4(w.x0, w.x1, w.x2, w.x3);
        } else {
          dst[0] = w.x0;
          if (left > 1) dst[1] = w.x1;
          if (left > 2) dst[2] = w.x2;
          if (left > 3) dst[3] = w.x3;
        }
      }
    }
  }
}

// ---- Categorical ---------------------------------------------------------------------------------
// Two CTAs of 512 threads per SM, a row each: while one CTA waits for its loads the other computes, and
// 296 rows are in flight at once (a batch of 256 rows is one wave).  The row is read from HBM once; the
// second pass re-reads 1/16 of it (one warp's run), which is in L2.
constexpr int kDrawThreads = 512;
constexpr int kDrawCtasPerSm = 2;
constexpr int kDrawWarps = kDrawThreads / 32;
constexpr int kDrawBatch = 8;  // chunk loads in flight per warp in the second pass
constexpr uint32_t kDrawMaxChunks = 1024;  // chunk totals of one run kept in shared memory (rows up to 524 288 wide)
static_assert(kDrawThreads / 32 * kDrawMaxChunks * 32 == 524288, "the shared table covers the documented row width");

template <int kDtype>
__device__ __forceinline__ float load_logit(const void *row, uint32_t i) {
  if constexpr (kDtype == HYLE_B200_F32) return static_cast<const float *>(row)[i];
  if constexpr (kDtype == HYLE_B200_BF16) return bf16_to_f32(static_cast<const unsigned short *>(row)[i]);
  return f16_to_f32(static_cast<const unsigned short *>(row)[i]);
}

__device__ __forceinline__ double warp_inclusive_scan(double v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double up = __shfl_up_sync(kFullMask, v, o);
    if (lane >= o) v += up;
  }
  return v;
}

__device__ __forceinline__ float weight_of(float x, float neg_scaled_max) {
  // exp(x - max) as 2^(x log2e - max log2e): one fused multiply-add and one ex2; -inf gives 0
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(x, 1.4426950408889634f, neg_scaled_max)));
  return r;
}

// One CTA per row, a warp owns a contiguous run of the row (coalesced loads).
//   pass 1  maximum, validity and the weight sums in ONE read of the row ("online": running maximum
//           per lane, sums rescaled when it grows; lanes -> warp -> row in f64 with fixed trees);
//           thread 0 chains the 32 warp totals -> the threshold total * u falls into one warp's span
//   pass 2  (1/32 of the row, from L2) all warps form the chunk totals of that run (32 elements each,
//           fixed tree); warp 0 chains them in f64 to the chunk where the cumulative weight first
//           exceeds the threshold and scans the 32 elements of that chunk.
// Pass 1 and pass 2 add the same weights in different orders, so when the threshold lies within
// rounding of a boundary the walk can end without a crossing; the draw then is the next element
// of positive mass (what exact arithmetic would give), or, at the very end of the row, the last
// index holding the maximum (src/compute_provider_native/sampling.cc:171-176).
template <int kDtype>
__global__ void __launch_bounds__(kDrawThreads, kDrawCtasPerSm)
categorical_kernel(const void *logits, const uint32_t *__restrict__ identities, int32_t *index_out, float *log_probability,
                   uint64_t rows, uint32_t cols, uint32_t *status_word) {
  grid_dependency_sync();
  __shared__ float s_max[kDrawWarps], s_shift[kDrawWarps];
  __shared__ uint32_t s_bad[kDrawWarps];
  __shared__ double s_sum[kDrawWarps];
  __shared__ double s_before[kDrawWarps + 1];
  __shared__ double s_chunk[kDrawMaxChunks];
  __shared__ int32_t s_selected;   // >= 0: the draw;  -1: not found yet
  __shared__ uint32_t s_resume;    // where to look for the next element of positive mass
  __shared__ uint32_t s_next;
  __shared__ int32_t s_last;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint32_t run = ((cols + kDrawWarps - 1) / kDrawWarps + 31) / 32 * 32;  // elements per warp, whole chunks
  const uint32_t begin = min(warp * run, cols), end = min(begin + run, cols);
  constexpr size_t kWidth = kDtype == HYLE_B200_F32 ? 4 : 2;

  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const void *x = static_cast<const unsigned char *>(logits) + row * cols * kWidth;
    // pass 1 (the only read of the row from HBM): maximum, validity AND the weight sums, "online".  A lane
    // sums 2^(x log2 e - s) against its own shift s and raises s when an element would exceed it.  The
    // shifts are INTEGERS, so every rescaling (lane, lane -> warp, warp -> row) is an exact power of two: no
    // lane's weights carry a rounding of their own shift, which would move the threshold by parts in 10^7
    // and the draw with it.  A raised shift gets kDrawHeadroom binades of room, so a slowly growing maximum
    // does not rescale at every record (the path diverges the warp): weights then sit at most 2^-headroom
    // below 1, which only narrows the range above the flush-to-zero floor from 126 to 118 binades.
    // Four 16-byte loads are in flight per lane.
    // the row's uniform does not depend on the data: its ten Philox rounds run under the first loads
    const Words random = philox_block(identities + row * 4, 0);
    const double uniform =
        (static_cast<double>(random.x0) * 1048576.0 + static_cast<double>(random.x1 >> 12) + 0.5) * 2.220446049250313e-16;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kDrawHeadroom = 8.0f;
    constexpr float kNoShift = -3.0e38f;  // below every finite x log2 e: the first finite element raises it
    float lane_max = -CUDART_INF_F, lane_shift = kNoShift;
    double lane_sum = 0.0;
    uint32_t bad = 0;
    auto rescale = [](double value, float from_shift, float to_shift) {  // value * 2^(from - to), to >= from: exact
      const int exponent = static_cast<int>(fmaxf(from_shift - to_shift, -1022.0f));  // 2^-1022 of a sum <= 2^20 is nothing
      return value * __hiloint2double((1023 + exponent) << 20, 0);
    };
    auto absorb = [&](const float (&v)[4]) {
      const float high = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));  // drops NaN: those show in the weights
      const float scaled = __fmul_rn(high, kLog2e);
      if (scaled > lane_shift && high < CUDART_INF_F) {  // rare after the first elements
        const float shift = ceilf(scaled) + kDrawHeadroom;
        lane_sum = rescale(lane_sum, lane_shift, shift);
        lane_shift = shift;
      }
      lane_max = fmaxf(lane_max, high);
      const float minus = -lane_shift;
      // four weights are added in f32 (a rounding of 6e-8 of their sum, unbiased), the running sum is f64;
      // a NaN element makes its weight NaN, -inf gives 0, +inf is rejected through the maximum
      const float weights = (weight_of(v[0], minus) + weight_of(v[1], minus)) + (weight_of(v[2], minus) + weight_of(v[3], minus));
      bad |= (weights != weights || high == CUDART_INF_F) ? 1u : 0u;
      lane_sum += static_cast<double>(weights);
    };
    // f32 rows whose start is 16-byte aligned are read as float4 (the sums do not depend on the order of
    // the elements inside a warp's run); runs start at multiples of 32 elements
    const bool vectors = kDtype == HYLE_B200_F32 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const uint32_t vector_end = vectors ? begin + (end - begin) / 4 * 4 : begin;
    {
      const float *row_values = static_cast<const float *>(x);
      uint32_t i = begin + 4 * lane;
      for (; i + 3 * 128 < vector_end; i += 4 * 128) {
        float4 q[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) q[k] = *reinterpret_cast<const float4 *>(row_values + i + k * 128);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float v[4] = {q[k].x, q[k].y, q[k].z, q[k].w};
          absorb(v);
        }
      }
      for (; i < vector_end; i += 128) {
        const float4 q = *reinterpret_cast<const float4 *>(row_values + i);
        const float v[4] = {q.x, q.y, q.z, q.w};
        absorb(v);
      }
    }
    for (uint32_t i = vector_end + lane; i < end; i += 32) {
      const float one = load_logit<kDtype>(x, i);
      const float v[4] = {one, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};  // -inf: weight 0, no effect on max or probe
      absorb(v);
    }
    float maximum = lane_max;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(kFullMask, maximum, o));
    bad = __any_sync(kFullMask, bad != 0) ? 1u : 0u;
    // lanes -> warp: against the largest shift of the warp, one fixed tree per warp
    float warp_shift = lane_shift;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) warp_shift = fmaxf(warp_shift, __shfl_xor_sync(kFullMask, warp_shift, o));
    const double sum = warp_sum(bad ? 0.0 : rescale(lane_sum, lane_shift, warp_shift));
    if (lane == 0) {
      s_max[warp] = maximum;
      s_shift[warp] = warp_shift;
      s_bad[warp] = bad;
      s_sum[warp] = sum;
    }
    __syncthreads();
    maximum = s_max[0];
    bad = s_bad[0];
    float row_shift = s_shift[0];
#pragma unroll
    for (int w = 1; w < kDrawWarps; ++w) {
      maximum = fmaxf(maximum, s_max[w]);
      row_shift = fmaxf(row_shift, s_shift[w]);
      bad |= s_bad[w];
    }
    if (bad != 0 || !(maximum > -CUDART_INF_F)) {  // CTA-uniform: reject the row
      if (t == 0) {
        index_out[row] = -1;
        if (log_probability != nullptr) log_probability[row] = CUDART_NAN_F;
        if (status_word != nullptr) atomicOr(status_word, HYLE_B200_STATUS_INVALID_CATEGORICAL_ROW);
      }
      __syncthreads();
      continue;
    }
    // every weight from here on is 2^(x log2 e - row_shift); the common factor cancels in the draw and
    // is put back into the log-probability below
    const float neg_scaled_max = -row_shift;
    if (t == 0) {
      // thread 0 chains the warp totals, each brought (exactly) to the row's shift
      double running = 0.0;
      for (int w = 0; w < kDrawWarps; ++w) {
        s_before[w] = running;
        running += rescale(s_sum[w], s_shift[w], row_shift);
      }
      s_before[kDrawWarps] = running;
      s_selected = -1;
      s_resume = cols;
      s_next = cols;
      s_last = -1;
    }
    __syncthreads();
    const double total = s_before[kDrawWarps];
    const double threshold = total * uniform;
    // pass 2: the run whose span of the cumulative sum holds the threshold.  Every thread finds the
    // owner from the same shared values, so the choice is CTA-uniform.
    int owner = kDrawWarps - 1;
#pragma unroll
    for (int w = kDrawWarps - 2; w >= 0; --w)
      if (threshold < s_before[w + 1]) owner = w;
    const uint32_t owner_begin = min(owner * run, cols), owner_end = min(owner_begin + run, cols);
    const uint32_t chunks = (owner_end - owner_begin + 31) / 32;
    if (chunks <= kDrawMaxChunks) {
      // all warps share the owner's run: chunk totals (fixed tree) into shared memory ...
      // (the loads of kDrawBatch chunks are issued before the first is summed: the run comes from L2 and a
      // load per chunk in sequence would cost an L2 round trip each)
      for (uint32_t first = warp; first < chunks; first += kDrawWarps * kDrawBatch) {
        float value[kDrawBatch];
#pragma unroll
        for (int k = 0; k < kDrawBatch; ++k) {
          const uint32_t c = first + k * kDrawWarps, i = owner_begin + 32 * c + lane;
          value[k] = c < chunks && i < owner_end ? load_logit<kDtype>(x, i) : -CUDART_INF_F;  // -inf: weight 0
        }
#pragma unroll
        for (int k = 0; k < kDrawBatch; ++k) {
          const uint32_t c = first + k * kDrawWarps;
          const double chunk_total = warp_sum(static_cast<double>(weight_of(value[k], neg_scaled_max)));
          if (lane == 0 && c < chunks) s_chunk[c] = chunk_total;
        }
      }
      __syncthreads();
      // ... then warp 0 chains them, 32 at a time, to the chunk where the cumulative weight first
      // exceeds the threshold, and scans the 32 elements of that chunk
      // (two levels: each lane adds a strip of consecutive chunk totals, one scan finds the strip, a second
      // one the chunk inside it: two warp scans instead of one per 32 chunks)
      if (warp == 0) {
        const uint32_t strip = (chunks + 31) / 32;  // <= 32 because chunks <= kDrawMaxChunks
        double strip_total = 0.0;
        for (uint32_t k = 0; k < strip; ++k) {
          const uint32_t c = lane * strip + k;
          if (c < chunks) strip_total += s_chunk[c];
        }
        const double start = s_before[owner];
        const double inclusive = start + warp_inclusive_scan(strip_total, lane);
        const unsigned crossed = __ballot_sync(kFullMask, strip_total > 0.0 && inclusive > threshold);
        int32_t found = -1;
        if (crossed != 0) {
          const int first = __ffs(crossed) - 1;
          const double previous = __shfl_sync(kFullMask, inclusive, first > 0 ? first - 1 : 0);
          const double strip_before = first > 0 ? previous : start;
          const uint32_t c = first * strip + lane;
          const bool mine = lane < strip && c < chunks;
          const double chunk_total = mine ? s_chunk[c] : 0.0;
          const double through = strip_before + warp_inclusive_scan(chunk_total, lane);
          const unsigned reached = __ballot_sync(kFullMask, mine && chunk_total > 0.0 && through > threshold);
          const unsigned filled = __ballot_sync(kFullMask, mine && chunk_total > 0.0);  // not empty: the strip's total is positive
          // the strip sums and the scan may disagree in the last bit: then the strip's last chunk of mass
          const int chosen = reached != 0 ? __ffs(reached) - 1 : 31 - __clz(filled);
          const double chunk_previous = __shfl_sync(kFullMask, through, chosen > 0 ? chosen - 1 : 0);
          const double before = chosen > 0 ? chunk_previous : strip_before;
          const uint32_t base = owner_begin + 32 * (first * strip + chosen);
          const uint32_t i = base + lane;
          const double weight = i < owner_end ? static_cast<double>(weight_of(load_logit<kDtype>(x, i), neg_scaled_max)) : 0.0;
          const double within = before + warp_inclusive_scan(weight, lane);
          const unsigned hit = __ballot_sync(kFullMask, weight > 0.0 && within > threshold);
          const unsigned massive = __ballot_sync(kFullMask, weight > 0.0);  // not empty: the chunk's total is positive
          // the same for the elements: the chunk's last element of mass
          found = static_cast<int32_t>(base + (hit != 0 ? __ffs(hit) - 1 : 31 - __clz(massive)));
        }
        if (lane == 0) {
          s_selected = found;
          s_resume = owner_end;  // only read when found < 0
        }
      }
    } else if (warp == owner) {
      // a run too long for the shared table: the owning warp walks it alone
      double cumulative = s_before[warp];
      int32_t found = -1;
      constexpr int kStep = 4;  // chunks whose totals are formed together: their tree sums overlap
      for (uint32_t base = begin; base < end && found < 0; base += 32 * kStep) {
        double weight[kStep], chunk_total[kStep];
#pragma unroll
        for (int k = 0; k < kStep; ++k) {
          const uint32_t i = base + 32 * k + lane;
          weight[k] = i < end ? static_cast<double>(weight_of(load_logit<kDtype>(x, i), neg_scaled_max)) : 0.0;
        }
#pragma unroll
        for (int k = 0; k < kStep; ++k) chunk_total[k] = warp_sum(weight[k]);
#pragma unroll
        for (int k = 0; k < kStep; ++k) {
          const double after = cumulative + chunk_total[k];
          if (found < 0 && after > threshold) {  // the crossing is inside this chunk (warp-uniform)
            const double inclusive = cumulative + warp_inclusive_scan(weight[k], lane);
            const unsigned crossed = __ballot_sync(kFullMask, weight[k] > 0.0 && inclusive > threshold);
            const unsigned massive = __ballot_sync(kFullMask, weight[k] > 0.0);
            found = static_cast<int32_t>(base + 32 * k + (crossed != 0 ? __ffs(crossed) - 1 : 31 - __clz(massive)));
          }
          cumulative = after;
        }
      }
      if (lane == 0) {
        s_selected = found;
        s_resume = end;
      }
    }
    __syncthreads();
    if (s_selected < 0) {  // CTA-uniform; rare
      const uint32_t resume = s_resume;
      uint32_t next = cols;
      int32_t last = -1;
      for (uint32_t i = t; i < cols; i += kDrawThreads) {
        const float v = load_logit<kDtype>(x, i);
        if (i >= resume && v > -CUDART_INF_F && weight_of(v, neg_scaled_max) > 0.0f) next = min(next, i);
        if (v == maximum) last = static_cast<int32_t>(i);
      }
      if (next < cols) atomicMin(&s_next, next);
      if (last >= 0) atomicMax(&s_last, last);
      __syncthreads();
      if (t == 0) s_selected = s_next < cols ? static_cast<int32_t>(s_next) : s_last;
      __syncthreads();
    }
    if (t == 0) {
      const int32_t selected = s_selected;
      index_out[row] = selected;
      if (log_probability != nullptr)
        // log p = x - log(sum e^x), and sum e^x = total * 2^row_shift
        log_probability[row] = static_cast<float>(static_cast<double>(load_logit<kDtype>(x, static_cast<uint32_t>(selected))) -
                                                  (log(total) + static_cast<double>(row_shift) * 0.6931471805599453));
    }
    __syncthreads();  // shared scratch is reused by the next row
  }
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" int hyle_b200_random_bits(hyle_b200_stream_t stream, const uint32_t *identities, uint64_t rows,
                                     uint32_t word_count, uint32_t *out) {
  if (rows == 0 || word_count == 0) return HYLE_B200_OK;
  if (identities == nullptr || out == nullptr || word_count > 0x7fffffffu || !aligned_to(identities, 4) ||
      !aligned_to(out, 4))
    return HYLE_B200_INVALID_VALUE;
  const uint64_t blocks_per_row = (static_cast<uint64_t>(word_count) + 3) / 4;
  if (blocks_per_row >= 128) {  // rows of 512 words and more: warp spans
    const uint64_t spans = rows * ((blocks_per_row + kBitsSpan * 32 - 1) / (kBitsSpan * 32));
    const unsigned span_grid = clamp_grid((spans + kBitsThreads / 32 - 1) / (kBitsThreads / 32), static_cast<uint64_t>(sm_count()) * 8);
    return launch(random_bits_span_kernel, dim3(span_grid), dim3(kBitsThreads), 0, reinterpret_cast<cudaStream_t>(stream),
                  identities, out, rows, word_count);
  }
  const uint64_t blocks = rows * blocks_per_row;
  const unsigned grid = clamp_grid((blocks + kBitsThreads - 1) / kBitsThreads, static_cast<uint64_t>(sm_count()) * 8);
  return launch(random_bits_block_kernel, dim3(grid), dim3(kBitsThreads), 0, reinterpret_cast<cudaStream_t>(stream), identities,
                out, rows, word_count);
}

extern "C" int hyle_b200_categorical(hyle_b200_stream_t stream, int dtype, const void *log_weights,
                                     const uint32_t *identities, uint64_t rows, uint64_t cols, int32_t *index_out,
                                     float *log_probability_out, uint32_t *status_word) {
  if (rows == 0) return HYLE_B200_OK;
  if (log_weights == nullptr || identities == nullptr || index_out == nullptr || cols == 0 || cols > 0x7fffffffull)
    return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = clamp_grid(rows, static_cast<uint64_t>(sm_count()) * kDrawCtasPerSm);
  const uint32_t width = static_cast<uint32_t>(cols);
  if (dtype == HYLE_B200_F32)
    return launch(categorical_kernel<HYLE_B200_F32>, dim3(grid), dim3(kDrawThreads), 0, s, log_weights, identities, index_out,
                  log_probability_out, rows, width, status_word);
  if (dtype == HYLE_B200_BF16)
    return launch(categorical_kernel<HYLE_B200_BF16>, dim3(grid), dim3(kDrawThreads), 0, s, log_weights, identities, index_out,
                  log_probability_out, rows, width, status_word);
  if (dtype == HYLE_B200_F16)
    return launch(categorical_kernel<HYLE_B200_F16>, dim3(grid), dim3(kDrawThreads), 0, s, log_weights, identities, index_out,
                  log_probability_out, rows, width, status_word);
  return HYLE_B200_INVALID_VALUE;
}

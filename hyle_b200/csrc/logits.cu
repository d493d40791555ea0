// Row softmax family over f32 rows: log-sum-exp, softmax (bf16 or f32 out), log-softmax and
// argmax, in ONE pass over HBM.
//
// A vocabulary row (151 936 f32 = 608 KB) does not fit one SM, so a thread-block cluster shares it:
// CTA k of the cluster keeps slice k of the row in its own shared memory, and only three scalars
// per CTA cross the cluster (distributed shared memory reads of the peers' slots):
//   phase A  global -> registers -> shared; NaN-propagating running maximum (one instruction/element)
//   exchange (max)                                                           cluster barrier 1
//   phase B  e = expf(x - max) written back to shared; f32 thread sums, f64 from the warp up;
//            lowest index whose value equals the maximum
//   exchange (sum, index)                                                    cluster barrier 2
//   phase C  shared -> bf16/f32 probabilities (or x - shift) -> 16-byte global stores
// HBM traffic is the algorithmic minimum (4 B read + 2 B written per element for bf16 output); the
// second and third touches of every element hit shared memory.
//
// Semantics follow src/simd/math/activations.cc:301-334 (softmax: f32 exp, f64 sum, multiply by
// float(1/sum); log-softmax shift = max + float(log(sum)); rows with NaN/+inf or only -inf are all
// NaN) and src/simd/sort/top_k.cc:17-27 (argmax: larger value first, NaN last, lower index on ties).
#include "common.cuh"

#include <cooperative_groups.h>
#include <math_constants.h>

namespace cg = cooperative_groups;

namespace hb {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kLoadBatch = 4;  // 16-byte loads in flight per thread in phase A
constexpr uint32_t kNoIndex = 0xffffffffu;
constexpr int kMaxCluster = 8;
constexpr size_t kTwoCtaSliceBytes = 76 * 1024;   // two CTAs of this size share an SM
constexpr size_t kMaxSliceBytes = 200 * 1024;     // one CTA per SM

enum Mode { kProbsBf16 = 0, kProbsF32 = 1, kLogF32 = 2, kArgmaxOnly = 3 };

struct LogitsParams {
  const float *in;
  uint64_t rows;
  uint32_t cols;
  uint32_t slice;  // elements per CTA, a multiple of 8
  float *lse;
  void *out;       // probabilities / log-probabilities, or nullptr
  int32_t *index;
  float *value;
  uint32_t *status;  // device status word (may be null): HYLE_B200_STATUS_STREAM_WAIT_TIMEOUT
};

// TopK's value output is the ELEMENT at the winning index (src/simd/sort/top_k.cc returns
// scores[index]).  The folded maximum equals it except in sign: the fold orders -0 below +0, so a row
// whose first maximal element is -0 with a +0 later folds to +0 while the winner is the -0 element.
// One load that hits L2 (the row was just read).
__device__ __forceinline__ float element_at(const LogitsParams &p, uint64_t row, uint32_t index, float folded) {
  return index < p.cols ? p.in[row * p.cols + index] : folded;
}

struct Best {
  float value;
  uint32_t index;
};

// TopK order restricted to non-NaN candidates; "no candidate" is (-inf, kNoIndex) and loses ties.
__device__ __forceinline__ Best better_of(Best a, Best b) {
  const bool take_b = b.value > a.value || (b.value == a.value && b.index < a.index);
  return take_b ? b : a;
}

__device__ __forceinline__ void consider(float x, uint32_t index, Best &best) {
  if (x > best.value) {  // strict: the first of equal values stays; NaN never enters
    best.value = x;
    best.index = index;
  }
}

__device__ __forceinline__ Best warp_best(Best best) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(kFullMask, best.value, o);
    other.index = __shfl_xor_sync(kFullMask, best.index, o);
    best = better_of(best, other);
  }
  return best;
}

// Full TopK{1} order for one row, by one CTA, from global memory: larger value first, NaN last,
// lower index on ties.  Used for rows the fast paths cannot decide (NaN present, or nothing above
// -inf).  All threads of the CTA must call it.
__device__ __noinline__ void rescan_argmax(const float *whole, uint32_t cols, int32_t *index_out, float *value_out) {
  __shared__ Best s_best[kWarps];
  __shared__ uint32_t s_first[kWarps];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  Best best{-CUDART_INF_F, kNoIndex};
  uint32_t first_floor = kNoIndex;  // first -inf
  for (uint32_t i = t; i < cols; i += blockDim.x) {
    const float x = whole[i];
    consider(x, i, best);
    if (x == -CUDART_INF_F && first_floor == kNoIndex) first_floor = i;
  }
  best = warp_best(best);
  first_floor = __reduce_min_sync(kFullMask, first_floor);
  if (lane == 0) {
    s_best[warp] = best;
    s_first[warp] = first_floor;
  }
  __syncthreads();
  if (t == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x / 32); ++w) {
      best = better_of(best, s_best[w]);
      first_floor = min(first_floor, s_first[w]);
    }
    // nothing above -inf: the first -inf, else the row is all NaN and element 0 stays
    const uint32_t chosen = best.index != kNoIndex ? best.index : (first_floor != kNoIndex ? first_floor : 0u);
    if (index_out != nullptr) *index_out = static_cast<int32_t>(chosen);
    if (value_out != nullptr) *value_out = whole[chosen];
  }
  __syncthreads();
}

// ---- argmax alone: a pure read stream, one cluster barrier per row ------------------------------
template <bool kVec>
__global__ void __launch_bounds__(kThreads)
argmax_kernel(const LogitsParams p) {
  grid_dependency_sync();
  __shared__ Best s_warp_best[kWarps];
  __shared__ Best s_cta_best[2];  // by row parity; read by the peers after the barrier
  __shared__ Best s_row_best;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const unsigned cluster_size = cluster.num_blocks();
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint64_t cluster_id = blockIdx.x / cluster_size;
  const uint64_t cluster_count = gridDim.x / cluster_size;
  const uint32_t begin = min(rank * p.slice, p.cols);
  const uint32_t end = min(begin + p.slice, p.cols);
  const uint32_t n = end - begin;
  int parity = 0;
  for (uint64_t row = cluster_id; row < p.rows; row += cluster_count, parity ^= 1) {
    const float *src = p.in + row * p.cols + begin;
    Best best{-CUDART_INF_F, kNoIndex};
    if constexpr (kVec) {
      const uint32_t vectors = n / 4;
      for (uint32_t v0 = t; v0 < vectors; v0 += kThreads * kLoadBatch) {
        float4 x[kLoadBatch];
#pragma unroll
        for (int k = 0; k < kLoadBatch; ++k)
          if (v0 + k * kThreads < vectors) x[k] = ld_stream(reinterpret_cast<const float4 *>(src) + v0 + k * kThreads);
#pragma unroll
        for (int k = 0; k < kLoadBatch; ++k) {
          const uint32_t v = v0 + k * kThreads;
          if (v < vectors) {
            const uint32_t i = begin + v * 4;
            consider(x[k].x, i, best);
            consider(x[k].y, i + 1, best);
            consider(x[k].z, i + 2, best);
            consider(x[k].w, i + 3, best);
          }
        }
      }
    } else {
      for (uint32_t i = t; i < n; i += kThreads) consider(ld_stream(src + i), begin + i, best);
    }
    best = warp_best(best);
    if (lane == 0) s_warp_best[warp] = best;
    __syncthreads();
    if (t == 0) {
      Best b = s_warp_best[0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) b = better_of(b, s_warp_best[w]);
      s_cta_best[parity] = b;
    }
    cluster.sync();
    if (rank == 0) {  // only the CTA that writes the result gathers the peers' slots
      if (warp == 0) {
        Best b{-CUDART_INF_F, kNoIndex};
        if (lane < cluster_size) b = *cluster.map_shared_rank(&s_cta_best[parity], lane);
        b = warp_best(b);
        if (lane == 0) s_row_best = b;
      }
      __syncthreads();
      const Best row_best = s_row_best;
      if (row_best.index != kNoIndex) {
        if (t == 0) {
          if (p.index != nullptr) p.index[row] = static_cast<int32_t>(row_best.index);
          if (p.value != nullptr) p.value[row] = row_best.value;
        }
      } else {
        rescan_argmax(p.in + row * p.cols, p.cols, p.index != nullptr ? p.index + row : nullptr,
                      p.value != nullptr ? p.value + row : nullptr);
      }
    }
  }
  cluster.sync();  // no CTA leaves while a peer may still read its shared memory
}

// ---- fused lse / softmax / argmax ---------------------------------------------------------------
struct SumSlot {
  double sum;
  uint32_t index;  // lowest index in this CTA's slice holding the row maximum, or kNoIndex
  uint32_t pad;
};

template <int kMode, bool kVec>
__global__ void __launch_bounds__(kThreads)
logits_kernel(const LogitsParams p) {
  grid_dependency_sync();
  extern __shared__ __align__(16) float slice_data[];
  __shared__ float s_warp_max[kWarps];
  __shared__ double s_warp_sum[kWarps];
  __shared__ uint32_t s_warp_index[kWarps];
  __shared__ float s_cta_max;      // read by the peers after barrier 1
  __shared__ SumSlot s_cta_sum;    // read by the peers after barrier 2
  __shared__ float s_row_max;      // cluster-wide results, broadcast inside the CTA
  __shared__ SumSlot s_row_sum;

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const unsigned cluster_size = cluster.num_blocks();
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint64_t cluster_id = blockIdx.x / cluster_size;
  const uint64_t cluster_count = gridDim.x / cluster_size;
  const bool want_index = p.index != nullptr || p.value != nullptr;

  const uint32_t begin = min(rank * p.slice, p.cols);
  const uint32_t end = min(begin + p.slice, p.cols);
  const uint32_t n = end - begin;

  for (uint64_t row = cluster_id; row < p.rows; row += cluster_count) {
    const float *src = p.in + row * p.cols + begin;

    // ---- phase A: global -> shared, NaN-propagating maximum ------------------------------------
    float maximum = -CUDART_INF_F;
    if constexpr (kVec) {
      const uint32_t vectors = n / 4;
      for (uint32_t v0 = t; v0 < vectors; v0 += kThreads * kLoadBatch) {
        float4 x[kLoadBatch];
#pragma unroll
        for (int k = 0; k < kLoadBatch; ++k)
          if (v0 + k * kThreads < vectors) x[k] = ld_stream(reinterpret_cast<const float4 *>(src) + v0 + k * kThreads);
#pragma unroll
        for (int k = 0; k < kLoadBatch; ++k) {
          const uint32_t v = v0 + k * kThreads;
          if (v < vectors) {
            reinterpret_cast<float4 *>(slice_data)[v] = x[k];
            maximum = max_nan(max_nan(maximum, x[k].x), max_nan(x[k].y, max_nan(x[k].z, x[k].w)));
          }
        }
      }
    } else {
      for (uint32_t i = t; i < n; i += kThreads) {
        const float x = ld_stream(src + i);
        slice_data[i] = x;
        maximum = max_nan(maximum, x);
      }
    }
    maximum = warp_max_nan(maximum);
    if (lane == 0) s_warp_max[warp] = maximum;
    __syncthreads();
    if (t == 0) {
      float m = s_warp_max[0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) m = max_nan(m, s_warp_max[w]);
      s_cta_max = m;
    }
    cluster.sync();  // barrier 1 (also a CTA barrier: the slice is visible to every thread)
    if (warp == 0) {
      float m = lane < cluster_size ? *cluster.map_shared_rank(&s_cta_max, lane) : -CUDART_INF_F;
#pragma unroll
      for (int o = kMaxCluster / 2; o > 0; o >>= 1) m = max_nan(m, __shfl_xor_sync(kFullMask, m, o));
      if (lane == 0) s_row_max = m;
    }
    __syncthreads();
    maximum = s_row_max;
    // NaN or +inf anywhere, or nothing above -inf: the softmax outputs of the row are NaN.
    const bool valid = maximum > -CUDART_INF_F && maximum < CUDART_INF_F;
    const bool has_nan = maximum != maximum;

    // ---- phase B: exponentials back into shared memory, sums, position of the maximum -----------
    float thread_sum = 0.0f;
    uint32_t thread_index = kNoIndex;
    if (valid || (want_index && !has_nan)) {
      if constexpr (kVec) {
        for (uint32_t v = t; v < n / 4; v += kThreads) {
          float4 x = reinterpret_cast<const float4 *>(slice_data)[v];
          if (want_index && (x.x == maximum || x.y == maximum || x.z == maximum || x.w == maximum) &&
              thread_index == kNoIndex) {
            const uint32_t i = begin + v * 4;
            thread_index = x.x == maximum ? i : x.y == maximum ? i + 1 : x.z == maximum ? i + 2 : i + 3;
          }
          if (valid) {
            x = make_float4(expf(x.x - maximum), expf(x.y - maximum), expf(x.z - maximum), expf(x.w - maximum));
            if constexpr (kMode != kLogF32) reinterpret_cast<float4 *>(slice_data)[v] = x;
            thread_sum += (x.x + x.y) + (x.z + x.w);
          }
        }
      } else {
        for (uint32_t i = t; i < n; i += kThreads) {
          const float x = slice_data[i];
          if (want_index && x == maximum && thread_index == kNoIndex) thread_index = begin + i;
          if (valid) {
            const float e = expf(x - maximum);
            if constexpr (kMode != kLogF32) slice_data[i] = e;
            thread_sum += e;
          }
        }
      }
    }
    const double warp_total = warp_sum(static_cast<double>(thread_sum));
    const uint32_t warp_index = __reduce_min_sync(kFullMask, thread_index);
    if (lane == 0) {
      s_warp_sum[warp] = warp_total;
      s_warp_index[warp] = warp_index;
    }
    __syncthreads();
    if (t == 0) {
      SumSlot slot{s_warp_sum[0], s_warp_index[0], 0u};
#pragma unroll
      for (int w = 1; w < kWarps; ++w) {
        slot.sum += s_warp_sum[w];
        slot.index = min(slot.index, s_warp_index[w]);
      }
      s_cta_sum = slot;
    }
    cluster.sync();  // barrier 2
    if (warp == 0) {
      SumSlot slot{0.0, kNoIndex, 0u};
      if (lane < cluster_size) slot = *cluster.map_shared_rank(&s_cta_sum, lane);
#pragma unroll
      for (int o = kMaxCluster / 2; o > 0; o >>= 1) {  // fixed tree over the ranks
        slot.sum += __shfl_xor_sync(kFullMask, slot.sum, o);
        slot.index = min(slot.index, __shfl_xor_sync(kFullMask, slot.index, o));
      }
      if (lane == 0) s_row_sum = slot;
    }
    __syncthreads();
    const double total = s_row_sum.sum;

    if (rank == 0 && want_index) {
      if (!has_nan) {
        if (t == 0) {
          if (p.index != nullptr) p.index[row] = static_cast<int32_t>(s_row_sum.index);
          if (p.value != nullptr) p.value[row] = element_at(p, row, s_row_sum.index, maximum);
        }
      } else {
        rescan_argmax(p.in + row * p.cols, p.cols, p.index != nullptr ? p.index + row : nullptr,
                      p.value != nullptr ? p.value + row : nullptr);
      }
    }

    // ---- phase C: shared -> global -----------------------------------------------------------------
    const float nan = CUDART_NAN_F;
    const float inverse = valid ? static_cast<float>(1.0 / total) : nan;
    const float shift = valid ? maximum + static_cast<float>(log(total)) : nan;
    if (rank == 0 && t == 0 && p.lse != nullptr) p.lse[row] = shift;
    if (p.out != nullptr) {
      if constexpr (kMode == kProbsBf16) {
        unsigned short *dst = static_cast<unsigned short *>(p.out) + row * p.cols + begin;
        if constexpr (kVec) {
          for (uint32_t g = t; g < n / 8; g += kThreads) {
            const float4 a = reinterpret_cast<const float4 *>(slice_data)[2 * g];
            const float4 b = reinterpret_cast<const float4 *>(slice_data)[2 * g + 1];
            const uint4 o = valid ? make_uint4(pack_bf16x2(a.x * inverse, a.y * inverse),
                                               pack_bf16x2(a.z * inverse, a.w * inverse),
                                               pack_bf16x2(b.x * inverse, b.y * inverse),
                                               pack_bf16x2(b.z * inverse, b.w * inverse))
                                  : make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
            st_stream(reinterpret_cast<uint4 *>(dst) + g, o);
          }
        } else {
          for (uint32_t i = t; i < n; i += kThreads)
            dst[i] = valid ? f32_to_bf16(slice_data[i] * inverse) : static_cast<unsigned short>(0x7fc0);
        }
      } else {
        float *dst = static_cast<float *>(p.out) + row * p.cols + begin;
        if constexpr (kVec) {
          for (uint32_t v = t; v < n / 4; v += kThreads) {
            const float4 a = reinterpret_cast<const float4 *>(slice_data)[v];
            float4 o;
            if constexpr (kMode == kProbsF32) o = make_float4(a.x * inverse, a.y * inverse, a.z * inverse, a.w * inverse);
            else o = make_float4(a.x - shift, a.y - shift, a.z - shift, a.w - shift);
            if (!valid) o = make_float4(nan, nan, nan, nan);
            st_stream(reinterpret_cast<float4 *>(dst) + v, o);
          }
        } else {
          for (uint32_t i = t; i < n; i += kThreads) {
            const float o = kMode == kProbsF32 ? slice_data[i] * inverse : slice_data[i] - shift;
            dst[i] = valid ? o : nan;
          }
        }
      }
    }
    // The next row's phase A rewrites the slice.  Peer reads of s_cta_max (after barrier 1) and
    // s_cta_sum (after barrier 2) are ordered before their next writes by barrier 2 of this row
    // and barrier 1 of the next row respectively.
    __syncthreads();
  }
  cluster.sync();  // no CTA leaves while a peer may still read its shared memory
}

// ================================================================================================
// Fast path: the row lives in REGISTERS.  512 threads x 10 float4 = 20 480 values per CTA, so a
// cluster of eight covers a 151 936-wide row with one float4 slot to spare per thread, and two
// CTAs share an SM.  Per row and CTA:
//   [row i+1 streams into shared memory by cp.async while row i is processed]
//   shared -> registers (each thread reads back exactly the 10 x 16 B it fetched itself, so no
//   CTA barrier is involved)
//   -> thread max (remembering the slot) -> warp max (shuffles) -> [the lane holding the warp max
//      re-reads that one float4 from the staging buffer to find the position] -> refill issued
//   -> e = 2^(x log2e - c_warp) in place, thread sum -> warp sum -> warp entry (m, s, index)
//   == CTA barrier ==  warp 0 folds the 16 warp entries into the CTA entry
//   == cluster barrier ==  every warp reads the (at most eight) CTA entries through distributed
//      shared memory and folds them (M = max m;  S = sum s 2^(c - C);  index = min index at m == M)
//   -> p = e * 2^(c_warp - C) / S -> bf16/f32 -> global
// Each warp works against its OWN maximum, so nothing waits on another warp before the exchange;
// the constants c = fl(max * log2e) are formed once and reused, so their rounding cancels between
// numerator and denominator.  About 12 instructions and one ex2 per value.
//
// Measured alternatives on 256 x 151 936 (kept out of the code):
//   every warp reading all 128 warp entries through DSMEM          104 us  (remote reads dominate)
//   entries pushed by remote stores, split arrive/wait              54 us
//   st.async + transaction mbarriers instead of the cluster barrier 60 us  (warp 0's serial fold
//                                                                           and logf stall the CTA)
//   warp-specialised exchange warp, two rows in registers, 1 CTA/SM 56 us  (only 15 clusters of 8
//                                                                           fit at one CTA per SM)
//   this version                                                    53 us; 5.1 TB/s at 1024 rows
// ================================================================================================
constexpr int kRegVectors = 10;
constexpr uint32_t kRegSlice = kThreads * kRegVectors * 4;  // 20480 values per CTA
constexpr float kLog2e = 1.4426950408889634f;

struct __align__(16) WarpEntry {
  float maximum;
  float sum;
  uint32_t index;
  uint32_t pad;
};

__device__ __forceinline__ float exp2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void cp_async_16(void *shared_dst, const void *global_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst))),
               "l"(global_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr size_t kRegStageBytes = static_cast<size_t>(kThreads) * kRegVectors * sizeof(float4);  // 80 KB

// Fold one (maximum, sum relative to 2^(maximum log2e), index) entry per lane into the warp-wide
// result.  Lanes without an entry pass (-inf, 0, none).  Fixed shuffle tree: every caller with the
// same inputs gets the same bits.
struct Combined {
  float maximum;
  float total;
  uint32_t index;
};
__device__ __forceinline__ Combined combine(WarpEntry mine) {
  Combined r;
  r.maximum = warp_max_nan(mine.maximum);
  const float row_c = __fmul_rn(r.maximum, kLog2e);
  // an entry at -inf carries sum 0; its weight must not become 0 * inf
  const float weight = mine.maximum == -CUDART_INF_F ? 0.0f : exp2_approx(__fmul_rn(mine.maximum, kLog2e) - row_c);
  r.total = warp_sum(mine.sum * weight);
  r.index = __reduce_min_sync(kFullMask, mine.maximum == r.maximum ? mine.index : kNoIndex);
  return r;
}

template <int kMode, int kFull>
__global__ void __launch_bounds__(kThreads, 2)
logits_regs_kernel(const LogitsParams p) {
  grid_dependency_sync();
  extern __shared__ __align__(16) float4 stage[];  // [kRegVectors][kThreads]: slot (j, t) belongs to thread t
  __shared__ WarpEntry s_entry[kWarps];  // this CTA's warps; read by warp 0 before the cluster barrier
  __shared__ WarpEntry s_cta[2];         // this CTA's entry, by row parity; read by the peers after it
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const unsigned cluster_size = cluster.num_blocks();
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint64_t cluster_id = blockIdx.x / cluster_size;
  const uint64_t cluster_count = gridDim.x / cluster_size;
  const bool want_index = p.index != nullptr || p.value != nullptr;
  const uint32_t begin = min(rank * p.slice, p.cols);
  const uint32_t end = min(begin + p.slice, p.cols);
  const uint32_t vectors = (end - begin) / 4;
  // float4 slots of this thread that lie inside the slice: slot j is valid when j < slots
  const int slots = vectors > static_cast<uint32_t>(t) ? static_cast<int>((vectors - t + kThreads - 1) / kThreads) : 0;
  const float neg_inf = -CUDART_INF_F;

  auto prefetch = [&](uint64_t row) {
    const float4 *src = reinterpret_cast<const float4 *>(p.in + row * p.cols + begin);
#pragma unroll
    for (int j = 0; j < kRegVectors; ++j)
      if (j < kFull || j < slots) cp_async_16(&stage[j * kThreads + t], src + j * kThreads + t);
    cp_async_commit();
  };
  if (cluster_id < p.rows) prefetch(cluster_id);

  int parity = 0;
  for (uint64_t row = cluster_id; row < p.rows; row += cluster_count, parity ^= 1) {
    cp_async_wait_all();  // this thread's own copies have landed; nobody else touches its slots
    float4 x[kRegVectors];
#pragma unroll
    for (int j = 0; j < kRegVectors; ++j)
      x[j] = (j < kFull || j < slots) ? stage[j * kThreads + t] : make_float4(neg_inf, neg_inf, neg_inf, neg_inf);
    float thread_max = neg_inf;
    int best_slot = 0;
#pragma unroll
    for (int j = 0; j < kRegVectors; ++j) {
      const float slot_max = max_nan(max_nan(x[j].x, x[j].y), max_nan(x[j].z, x[j].w));
      if (slot_max > thread_max) best_slot = j;
      thread_max = max_nan(thread_max, slot_max);
    }
    const float warp_max = warp_max_nan(thread_max);
    uint32_t index = kNoIndex;
    if (want_index) {
      if (thread_max == warp_max) {
        const float4 v = stage[best_slot * kThreads + t];
        const uint32_t base = begin + (best_slot * kThreads + t) * 4;
        index = v.x == warp_max ? base : v.y == warp_max ? base + 1 : v.z == warp_max ? base + 2 : base + 3;
      }
      index = __reduce_min_sync(kFullMask, index);
    }
    if (row + cluster_count < p.rows) prefetch(row + cluster_count);

    // Exponentials against the warp's own maximum (0 stands in when the warp saw only -inf), as
    // 2^(x log2e - c) with c = fl(max * log2e): one fused multiply-add and one ex2 per value.  The
    // same c is used again when the warp's weight is formed below, so its rounding cancels.
    const float reference = warp_max == neg_inf ? 0.0f : warp_max;
    const float neg_c = -__fmul_rn(reference, kLog2e);
    float thread_sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kRegVectors; ++j) {
      const float4 e = make_float4(exp2_approx(fmaf(x[j].x, kLog2e, neg_c)), exp2_approx(fmaf(x[j].y, kLog2e, neg_c)),
                                   exp2_approx(fmaf(x[j].z, kLog2e, neg_c)), exp2_approx(fmaf(x[j].w, kLog2e, neg_c)));
      thread_sum += (e.x + e.y) + (e.z + e.w);
      if constexpr (kMode != kLogF32) x[j] = e;
    }
    const float warp_total = warp_sum(thread_sum);
    if (lane == 0) s_entry[warp] = WarpEntry{warp_max, warp_total, index, 0u};

    // Two-level exchange.  Inside the CTA: warp 0 folds the 16 warp entries into one CTA entry.
    // Across the cluster: after the barrier every warp reads the (at most eight) CTA entries, one
    // per lane, through distributed shared memory and folds them itself -- eight small remote
    // reads per warp.  (Letting every warp read every warp's entry costs 128 remote reads per
    // warp and more than doubles the kernel time.)
    __syncthreads();
    if (warp == 0) {
      const Combined cta = combine(lane < kWarps ? s_entry[lane] : WarpEntry{neg_inf, 0.0f, kNoIndex, 0u});
      if (lane == 0) s_cta[parity] = WarpEntry{cta.maximum, cta.total, cta.index, 0u};
    }
    cluster.sync();  // the only cluster barrier of the row: every CTA has published its entry
    const Combined all = combine(lane < cluster_size ? *cluster.map_shared_rank(&s_cta[parity], lane)
                                                     : WarpEntry{neg_inf, 0.0f, kNoIndex, 0u});
    const float maximum = all.maximum, total = all.total, row_c = __fmul_rn(all.maximum, kLog2e);
    const uint32_t best_index = all.index;

    const bool valid = maximum > neg_inf && maximum < CUDART_INF_F;  // false for NaN too
    const bool has_nan = maximum != maximum;
    const float nan = CUDART_NAN_F;
    // total is relative to 2^row_c with row_c = fl(maximum * log2e); the rounding of that product
    // (up to 3e-5 for |maximum| of a few hundred) is taken back out of the logarithm.
    const float residual = fmaf(maximum, kLog2e, -row_c);
    const float shift = valid ? maximum + (logf(total) - residual * 0.6931471805599453f) : nan;
    if (rank == 0 && warp == 0 && lane == 0) {
      if (p.lse != nullptr) p.lse[row] = shift;
      if (want_index && !has_nan) {
        if (p.index != nullptr) p.index[row] = static_cast<int32_t>(best_index);
        if (p.value != nullptr) p.value[row] = element_at(p, row, best_index, maximum);
      }
    }

    if (p.out != nullptr) {
      float scale = nan;
      if (valid) scale = warp_max == neg_inf ? 0.0f : __fdiv_rn(exp2_approx(-neg_c - row_c), total);
      if constexpr (kMode == kProbsBf16) {
        uint2 *dst = reinterpret_cast<uint2 *>(static_cast<unsigned short *>(p.out) + row * p.cols + begin);
#pragma unroll
        for (int j = 0; j < kRegVectors; ++j) {
          if (j < kFull || j < slots)
            st_stream(dst + j * kThreads + t, make_uint2(pack_bf16x2(x[j].x * scale, x[j].y * scale),
                                          pack_bf16x2(x[j].z * scale, x[j].w * scale)));
        }
      } else {
        float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.out) + row * p.cols + begin);
#pragma unroll
        for (int j = 0; j < kRegVectors; ++j) {
          if (j < kFull || j < slots) {
            float4 o;
            if constexpr (kMode == kProbsF32) o = make_float4(x[j].x * scale, x[j].y * scale, x[j].z * scale, x[j].w * scale);
            else o = make_float4(x[j].x - shift, x[j].y - shift, x[j].z - shift, x[j].w - shift);
            st_stream(dst + j * kThreads + t, o);
          }
        }
      }
    }
    // NaN rows take the full TopK order from global memory.  Placed last, when the row's registers
    // are dead, so the rare path costs the common one no register pressure.  CTA-uniform condition.
    if (rank == 0 && want_index && has_nan)  // CTA-uniform: NaN rows take the full TopK order
      rescan_argmax(p.in + row * p.cols, p.cols, p.index != nullptr ? p.index + row : nullptr,
                    p.value != nullptr ? p.value + row : nullptr);
  }
  cluster.sync();  // no CTA leaves while a peer may still read its shared memory
}

// ================================================================================================
// Streaming path for many rows: two passes over a row, the second one out of L2.
//
// The cluster path above keeps 33 rows in flight and every row pays a chain of barriers; with
// hundreds of rows there is a better trade.  The row is cut into chunks of at most 10 240 values
// (256 threads x 10 float4, held in registers for the length of one task) and the kernel works
// through a global, ordered list of chunk TASKS handed out by an atomic counter:
//   first pass  (row, chunk): chunk maximum, first index of it, sum of 2^(x log2e - c) against
//                each warp's own maximum -> one partial (three tagged 8-byte words, no fence)
//   second pass (row, chunk): every warp reads the row's partials (bounded wait for the tags),
//                folds them, and writes the probabilities of the chunk (streaming stores).
//                Chunk 0 also writes lse / argmax.
// A task's chunk reaches the CTA by ONE bulk copy (TMA, cp.async.bulk) into shared memory, issued
// a whole task ahead: while the CTA computes on registers, the next chunk is in flight.  First-pass
// copies carry an L2 evict-last policy, second-pass copies evict-first: the second pass finds the
// row in L2 (measured: DRAM reads = the logits once), so HBM sees every logit once and every
// probability once, as in the cluster path.
// The list interleaves the passes with a fixed lag of `window` rows:
//   P1(0) ... P1(w-1), P2(0), P1(w), P2(1), P1(w+1), ...            (each entry = all its chunks)
// so a second-pass task is claimed w x chunks claims after the first-pass tasks it depends on, by
// which time those have finished (they never wait on anything, and a claimed task is running):
// the wait is almost always satisfied on the first look and can never deadlock.  The window
// (64 rows = 39 MB) stays far below the 126 MB of L2.  No cluster, no barrier between CTAs.
// ================================================================================================
constexpr int kStreamThreads = 256;
constexpr int kStreamWarps = kStreamThreads / 32;
// A task's chunk is kStreamVectors float4 per thread (10 240 values, 40 KB of staging, 4 CTAs per
// SM), held in registers for the length of the task.  Half-size chunks (5 float4, measured on
// 64 / 256 / 1024 rows of 151 936) lose a quarter of the throughput to the per-task overhead: 0.56
// against 0.76 of the copy peak at 256 rows.
constexpr int kStreamVectors = 10;
__host__ __device__ constexpr uint32_t stream_chunk_values(int vectors) { return kStreamThreads * vectors * 4; }
constexpr size_t stream_stage_bytes(int vectors) { return static_cast<size_t>(kStreamThreads) * vectors * sizeof(float4); }
constexpr int kStreamCtasPerSm = 4;
constexpr uint32_t kStreamMaxChunks = 32;  // one partial per lane
// Rows between a row's two passes must cover the tasks in flight (two per resident CTA), or
// second-pass tasks find their partials missing; and must stay inside L2 (126 MB).  Measured at
// 256 / 1024 rows of 151 936 with 10 240-value chunks: 32 rows -> 0.71 / 0.88 of the copy peak,
// 40..64 -> 0.77-0.79 / 0.94-0.95, 96 -> 0.72 / 0.83 (the window no longer stays in L2).
constexpr uint32_t kStreamWindowMax = 64;
constexpr uint64_t kStreamWindowBytes = 40ull << 20;  // of f32 logits between the passes
constexpr uint64_t kStreamMinRows = 64;  // below this the cluster kernel is as fast or faster
// A second-pass warp polls this often for a partial before it computes the missing one itself, and
// this often again before it gives up (which needs a lost store: it cannot be waiting for a CTA that
// is not running, see the kernel).
constexpr uint32_t kStreamHelpAfter = 1u << 12;
constexpr uint32_t kStreamPollLimit = 1u << 22;
constexpr uint64_t kStreamHeaderBytes = 64;

enum StreamPass : uint32_t { kStreamFirst = 0, kStreamSecond = 1, kStreamEnd = 2 };
struct StreamTask {
  uint64_t row;
  uint32_t chunk_id;
  uint32_t pass;
};

// One first-pass result.  Three 8-byte words, each carrying the launch tag in its upper half: an
// 8-byte store is atomic, so a word whose tag matches holds valid data -- the writer needs no
// fence and no counter, the reader polls the words themselves (the idea of NCCL's LL protocol).
struct __align__(32) StreamPartial {
  unsigned long long maximum, sum, index, pad;
};

struct StreamParams {
  LogitsParams p;
  uint32_t chunks;  // per row
  uint32_t chunk;   // values per chunk, a multiple of 16
  uint32_t window;  // rows between the passes, at most p.rows
  uint32_t fixed;   // tasks per CTA taken by position (0..2) instead of from the counter
  uint32_t help_after;  // polls before a second-pass warp reduces a missing chunk itself
  unsigned long long *next_task;
  uint32_t *ticket;
  uint32_t *epoch;          // launches so far on this workspace; tag = epoch + 1, never 0
  StreamPartial *partials;  // [rows][chunks]
};

// Position `task` of the ordered list -> (pass, row, chunk):
//   P1(0) ... P1(w-1), P2(0), P1(w), P2(1), P1(w+1), ..., P2(rows-w) ... P2(rows-1)      (each entry = all its chunks)
__host__ __device__ inline StreamTask stream_decode(uint64_t task, uint64_t rows, uint32_t chunks, uint32_t window) {
  const uint64_t paired = rows - window;  // rows whose first pass is interleaved with a second pass
  StreamTask r;
  if (task >= 2 * rows * chunks) {
    r.row = 0;
    r.chunk_id = 0;
    r.pass = kStreamEnd;
    return r;
  }
  const uint64_t entry = task / chunks;
  r.chunk_id = static_cast<uint32_t>(task - entry * chunks);
  if (entry < window) {
    r.pass = kStreamFirst;
    r.row = entry;
  } else if (entry < window + 2 * paired) {
    const bool second = ((entry - window) & 1) == 0;
    r.pass = second ? kStreamSecond : kStreamFirst;
    r.row = (entry - window) / 2 + (second ? 0 : window);
  } else {
    r.pass = kStreamSecond;
    r.row = paired + (entry - window - 2 * paired);
  }
  return r;
}

__host__ __device__ inline uint32_t stream_chunks(uint64_t cols, int vectors) {
  const uint64_t chunk = stream_chunk_values(vectors);
  return static_cast<uint32_t>((cols + chunk - 1) / chunk);
}

// L2 policies for the two passes: a first-pass line should survive until the second pass reads it
// again (evict-last); the second pass is the last use (evict-first).
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ float4 load_hinted(const float4 *p, uint64_t policy) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p), "l"(policy));
  return v;
}

__device__ __forceinline__ uint32_t shared_address(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(uint64_t *barrier, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(barrier)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbarrier_expect(uint64_t *barrier, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(barrier)), "r"(bytes) : "memory");
}
// The hint lets the hardware keep the thread suspended (no issue slots used) until the phase
// completes or the time runs out; the caller's loop bounds the total wait.
constexpr uint32_t kSuspendHint = 20000;  // nanoseconds
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t *barrier, uint32_t phase) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(shared_address(barrier)), "r"(phase), "r"(kSuspendHint)
      : "memory");
  return done != 0;
}
// One bulk copy (TMA, untiled) global -> this CTA's shared memory with an L2 policy; the bytes are
// counted on `barrier`.  Both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void *shared_dst, const void *global_src, uint32_t bytes, uint64_t *barrier,
                                          uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          shared_address(shared_dst)),
      "l"(global_src), "r"(bytes), "r"(shared_address(barrier)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void store_relaxed(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long load_relaxed(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
constexpr uint32_t kStreamLoadPollLimit = 1u << 20;  // x up to 20 us each

// One warp reduces chunk `chunk_id` of `row` by itself, from global memory, and publishes the partial.
// The slow path of a second-pass task whose partial is missing: whoever holds the first-pass task
// may not be running (a grid larger than what is resident), so the waiter must not depend on it.
// Two writers of one partial store the same maximum and index and sums that agree to rounding, and
// each word is stored whole, so a reader may combine words of either.
__device__ __forceinline__ void stream_help_chunk(const float *row_in, uint32_t cols, uint32_t chunk_values, uint32_t chunk_id,
                                               StreamPartial *out, unsigned long long tag, bool want_index) {
  const int lane = threadIdx.x & 31;
  const uint32_t begin = chunk_id * chunk_values;
  const uint32_t vectors = (min(begin + chunk_values, cols) - begin) / 4;
  const float4 *src = reinterpret_cast<const float4 *>(row_in + begin);
  const uint64_t policy = policy_evict_last();
  float maximum = -CUDART_INF_F;
  for (uint32_t v = lane; v < vectors; v += 32) {
    const float4 x = load_hinted(src + v, policy);
    maximum = max_nan(maximum, max_nan(max_nan(x.x, x.y), max_nan(x.z, x.w)));
  }
  maximum = warp_max_nan(maximum);
  const float reference = maximum == -CUDART_INF_F ? 0.0f : maximum;
  const float neg_c = -__fmul_rn(reference, kLog2e);
  float sum = 0.0f;
  uint32_t index = kNoIndex;
  for (uint32_t v = lane; v < vectors; v += 32) {
    const float4 x = load_hinted(src + v, policy);
    sum += (exp2_approx(fmaf(x.x, kLog2e, neg_c)) + exp2_approx(fmaf(x.y, kLog2e, neg_c))) +
           (exp2_approx(fmaf(x.z, kLog2e, neg_c)) + exp2_approx(fmaf(x.w, kLog2e, neg_c)));
    if (want_index && index == kNoIndex) {
      const uint32_t base = begin + v * 4;
      index = x.x == maximum ? base : x.y == maximum ? base + 1 : x.z == maximum ? base + 2 : x.w == maximum ? base + 3 : kNoIndex;
    }
  }
  sum = warp_sum(sum);
  index = __reduce_min_sync(kFullMask, index);
  if (lane == 0) {
    store_relaxed(&out->maximum, tag | __float_as_uint(maximum));
    store_relaxed(&out->sum, tag | __float_as_uint(sum));
    store_relaxed(&out->index, tag | index);
  }
}

template <int kMode, int kVectors, int kFull>
__global__ void __launch_bounds__(kStreamThreads, kStreamCtasPerSm)
logits_stream_kernel(const StreamParams s) {
  // What needs no global memory (task decoding, barrier set-up) runs before the wait for the
  // previous grid: it overlaps that grid's tail.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ __align__(128) float4 stream_stage[];  // the chunk of the task that comes next
  __shared__ __align__(8) uint64_t s_full;                 // counts the bytes of the bulk load in flight
  __shared__ WarpEntry s_entry[kStreamWarps];
  __shared__ StreamTask s_tasks[3];                        // ring: current, next (being loaded), the one after
  __shared__ uint32_t s_flag;
  const LogitsParams &p = s.p;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const bool want_index = p.index != nullptr || p.value != nullptr;
  const float neg_inf = -CUDART_INF_F;
  const WarpEntry nothing{neg_inf, 0.0f, kNoIndex, 0u};

  // One thread decodes a list position (a 64-bit division) two tasks ahead, while the CTA works.
  auto decode = [&](uint64_t task) { return stream_decode(task, p.rows, s.chunks, s.window); };
  // A CTA's first `fixed` tasks are given by its position (no atomic before the first load), the
  // rest are claimed.  The host keeps fixed tasks inside the first-pass head of the list: a fixed
  // second-pass task would start beside the first pass it depends on.
  auto claim = [&]() { return static_cast<unsigned long long>(s.fixed) * gridDim.x + atomicAdd(s.next_task, 1ull); };
  // The chunk of `task` -> shared memory, one bulk copy issued by one thread.
  auto issue_load = [&](const StreamTask &task) {
    if (task.pass == kStreamEnd) return;
    const uint32_t begin = task.chunk_id * s.chunk;
    const uint32_t bytes = (min(begin + s.chunk, p.cols) - begin) * 4u;
    mbarrier_expect(&s_full, bytes);
    bulk_load(stream_stage, p.in + task.row * p.cols + begin, bytes, &s_full,
              task.pass == kStreamFirst ? policy_evict_last() : policy_evict_first());
  };

  if (t == 0) {
    mbarrier_init(&s_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (s.fixed >= 1u) s_tasks[0] = decode(blockIdx.x);
  }
  if (t == 64 && s.fixed >= 2u) s_tasks[1] = decode(static_cast<uint64_t>(gridDim.x) + blockIdx.x);
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous grid has completed and flushed
  // A CTA's tasks must come in list order (the loop stops at the first position past the end), so
  // the claims that fill the ring at the start are made by ONE thread: a pair of positions at once
  // when nothing is fixed.
  if (t == 0) {
    if (s.fixed == 0u) {
      const unsigned long long pair = atomicAdd(s.next_task, 2ull);
      s_tasks[0] = decode(pair);
      s_tasks[1] = decode(pair + 1);
    }
    issue_load(s_tasks[0]);
    if (s.fixed == 1u) s_tasks[1] = decode(claim());
  }
  const unsigned long long tag = static_cast<unsigned long long>(*s.epoch + 1u) << 32;
  __syncthreads();

  uint32_t phase = 0;
  int slot = 0;  // position of the current task in the ring
  for (;;) {
    const StreamTask now = s_tasks[slot];
    if (now.pass == kStreamEnd) break;
    const int slot_next = slot == 2 ? 0 : slot + 1, slot_after = slot_next == 2 ? 0 : slot_next + 1;
    const bool second = now.pass == kStreamSecond;
    const uint64_t row = now.row;
    const uint32_t chunk_id = now.chunk_id;
    const uint32_t begin = chunk_id * s.chunk;
    const uint32_t vectors = (min(begin + s.chunk, p.cols) - begin) / 4;

    // The chunk has been on its way since the previous task; take it into registers.
    bool landed = mbarrier_try_wait(&s_full, phase);
    for (uint32_t polls = 0; !landed && polls < kStreamLoadPollLimit; ++polls) landed = mbarrier_try_wait(&s_full, phase);
    phase ^= 1u;
    float4 x[kVectors];
#pragma unroll
    for (int j = 0; j < kVectors; ++j)
      x[j] = (j < kFull || j * kStreamThreads + t < vectors) ? stream_stage[j * kStreamThreads + t]
                                                             : make_float4(neg_inf, neg_inf, neg_inf, neg_inf);
    if (!landed) x[0].x = CUDART_NAN_F;  // the load never completed: the row is reported as NaN
    __syncthreads();  // everyone holds its values: the stage is free for the next chunk
    if (t == 32) issue_load(s_tasks[slot_next]);  // in flight during everything below
    // The claim for the task after the next: the atomic is issued now and its result is used at
    // the end of this task, so nobody waits for the round trip.
    unsigned long long claimed = 0;
    if (t == 64) claimed = claim();

    if (!second) {
      float thread_max = neg_inf;
      int best_slot = 0;
#pragma unroll
      for (int j = 0; j < kVectors; ++j) {
        const float slot_max = max_nan(max_nan(x[j].x, x[j].y), max_nan(x[j].z, x[j].w));
        if (slot_max > thread_max) best_slot = j;
        thread_max = max_nan(thread_max, slot_max);
      }
      const float warp_max = warp_max_nan(thread_max);
      uint32_t index = kNoIndex;
      if (want_index) {
        if (thread_max == warp_max) {  // a few lanes; never true for NaN.  The float4 is in L2.
          const float4 v = load_hinted(reinterpret_cast<const float4 *>(p.in + row * p.cols + begin) + best_slot * kStreamThreads + t,
                                       policy_evict_last());
          const uint32_t base = begin + (best_slot * kStreamThreads + t) * 4;
          index = v.x == warp_max ? base : v.y == warp_max ? base + 1 : v.z == warp_max ? base + 2 : base + 3;
        }
        index = __reduce_min_sync(kFullMask, index);
      }
      const float reference = warp_max == neg_inf ? 0.0f : warp_max;
      const float neg_c = -__fmul_rn(reference, kLog2e);
      float thread_sum = 0.0f;
#pragma unroll
      for (int j = 0; j < kVectors; ++j)
        thread_sum += (exp2_approx(fmaf(x[j].x, kLog2e, neg_c)) + exp2_approx(fmaf(x[j].y, kLog2e, neg_c))) +
                      (exp2_approx(fmaf(x[j].z, kLog2e, neg_c)) + exp2_approx(fmaf(x[j].w, kLog2e, neg_c)));
      const float warp_total = warp_sum(thread_sum);
      if (lane == 0) s_entry[warp] = WarpEntry{warp_max, warp_total, index, 0u};
      __syncthreads();
      if (warp == 0) {
        const Combined cta = combine(lane < kStreamWarps ? s_entry[lane] : nothing);
        if (lane == 0) {
          StreamPartial *out = s.partials + row * s.chunks + chunk_id;
          store_relaxed(&out->maximum, tag | __float_as_uint(cta.maximum));
          store_relaxed(&out->sum, tag | __float_as_uint(cta.total));
          store_relaxed(&out->index, tag | cta.index);
        }
      }
    } else {
      WarpEntry mine = nothing;
      bool complete = true;
      // Every warp fetches the row's partials itself, one per lane, and polls until all carry this
      // launch's tag.  They were written `window` rows ago: the first look almost always succeeds.
      // A partial still missing after kStreamHelpAfter looks may belong to a CTA that is not running
      // (the grid is sized to be co-resident, but nothing guarantees it: another kernel may hold SMs),
      // so the warp then reduces its share of the missing chunks ITSELF, from global memory, and
      // polls on for the chunks its sibling warps are reducing.  Nothing here waits for a CTA other
      // than its own, so the kernel completes, with right results, whatever is resident.
      const StreamPartial *in = s.partials + row * s.chunks + (lane < s.chunks ? lane : 0);
      unsigned long long m = 0, q = 0, i = 0;
      auto look = [&]() {
        if (lane >= s.chunks) return true;
        m = load_relaxed(&in->maximum);
        q = load_relaxed(&in->sum);
        i = load_relaxed(&in->index);
        return (m ^ tag) >> 32 == 0 && (q ^ tag) >> 32 == 0 && (i ^ tag) >> 32 == 0;
      };
      bool have = look();
      for (uint32_t polls = 0; !__all_sync(kFullMask, have) && polls < s.help_after; ++polls)
        if (!have) have = look();
      uint32_t missing = __ballot_sync(kFullMask, !have);
      if (missing != 0u) {  // warp-uniform, rare
        for (uint32_t rest = missing; rest != 0u; rest &= rest - 1u) {
          const uint32_t chunk = __ffs(rest) - 1;
          if (chunk % kStreamWarps == static_cast<uint32_t>(warp))
            stream_help_chunk(p.in + row * p.cols, p.cols, s.chunk, chunk, s.partials + row * s.chunks + chunk, tag, want_index);
        }
        for (uint32_t polls = 0; !__all_sync(kFullMask, have) && polls < kStreamPollLimit; ++polls)
          if (!have) have = look();
        // The chunk's values are read again (from L2) rather than kept alive across the slow path above:
        // kept, their forty registers would have to coexist with its working set, and the common path
        // would pay for the rare one in spills (measured: 45 -> 67 us at 256 x 151 936).
        const float4 *again = reinterpret_cast<const float4 *>(p.in + row * p.cols + begin) + t;
        const uint64_t once = policy_evict_first();
#pragma unroll
        for (int j = 0; j < kVectors; ++j)
          x[j] = (j < kFull || j * kStreamThreads + t < vectors) ? load_hinted(again + j * kStreamThreads, once)
                                                                 : make_float4(neg_inf, neg_inf, neg_inf, neg_inf);
        if (!landed) x[0].x = CUDART_NAN_F;
      }
      complete = __all_sync(kFullMask, have);
      if (lane < s.chunks)
        mine = WarpEntry{__uint_as_float(static_cast<uint32_t>(m)), __uint_as_float(static_cast<uint32_t>(q)),
                         static_cast<uint32_t>(i), 0u};
      if ((!complete || !landed) && t == 0 && p.status != nullptr) atomicOr(p.status, HYLE_B200_STATUS_STREAM_WAIT_TIMEOUT);
      const Combined all = combine(mine);
      const float maximum = all.maximum, total_sum = all.total, row_c = __fmul_rn(all.maximum, kLog2e);
      const bool valid = complete && landed && maximum > neg_inf && maximum < CUDART_INF_F;  // false for NaN too
      const bool has_nan = maximum != maximum;
      const float nan = CUDART_NAN_F;
      const float residual = fmaf(maximum, kLog2e, -row_c);
      const float shift = valid ? maximum + (logf(total_sum) - residual * 0.6931471805599453f) : nan;
      if (chunk_id == 0 && t == 0) {
        if (p.lse != nullptr) p.lse[row] = shift;
        if (want_index && !has_nan && complete) {
          if (p.index != nullptr) p.index[row] = static_cast<int32_t>(all.index);
          if (p.value != nullptr) p.value[row] = element_at(p, row, all.index, maximum);
        }
      }
      const float inverse = valid ? __fdiv_rn(1.0f, total_sum) : nan;
      const float neg_row_c = -row_c;
      if constexpr (kMode == kProbsBf16) {
        uint2 *dst = reinterpret_cast<uint2 *>(static_cast<unsigned short *>(p.out) + row * p.cols + begin) + t;
#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
          if (j < kFull || j * kStreamThreads + t < vectors)
            st_stream(dst + j * kStreamThreads,
                      make_uint2(pack_bf16x2(exp2_approx(fmaf(x[j].x, kLog2e, neg_row_c)) * inverse,
                                             exp2_approx(fmaf(x[j].y, kLog2e, neg_row_c)) * inverse),
                                 pack_bf16x2(exp2_approx(fmaf(x[j].z, kLog2e, neg_row_c)) * inverse,
                                             exp2_approx(fmaf(x[j].w, kLog2e, neg_row_c)) * inverse)));
        }
      } else {
        float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.out) + row * p.cols + begin) + t;
#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
          if (j < kFull || j * kStreamThreads + t < vectors) {
            float4 o;
            if constexpr (kMode == kProbsF32)
              o = make_float4(exp2_approx(fmaf(x[j].x, kLog2e, neg_row_c)) * inverse, exp2_approx(fmaf(x[j].y, kLog2e, neg_row_c)) * inverse,
                              exp2_approx(fmaf(x[j].z, kLog2e, neg_row_c)) * inverse, exp2_approx(fmaf(x[j].w, kLog2e, neg_row_c)) * inverse);
            else
              o = make_float4(x[j].x - shift, x[j].y - shift, x[j].z - shift, x[j].w - shift);
            st_stream(dst + j * kStreamThreads, o);
          }
        }
      }
      // NaN rows take the full TopK order from global memory (CTA-uniform condition).
      if (chunk_id == 0 && want_index && has_nan)
        rescan_argmax(p.in + row * p.cols, p.cols, p.index != nullptr ? p.index + row : nullptr,
                      p.value != nullptr ? p.value + row : nullptr);
    }
    // No barrier here: the next task's first barrier separates this task's shared-memory reads
    // from the next one's writes, and a ring entry is read two tasks after it is written.
    if (t == 64) s_tasks[slot_after] = decode(claimed);
    slot = slot_next;
  }

  // The CTA that leaves last re-arms the workspace for the next stream-ordered launch.  The barrier
  // orders the claiming thread's last atomic (consumed before it left the loop) before the ticket,
  // so no claim can land on the counter after it has been reset.
  __syncthreads();
  if (t == 0) {
    __threadfence();
    s_flag = atomicAdd(s.ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_flag != 0u && t == 0) {
    *s.next_task = 0ull;
    *s.ticket = 0u;
    *s.epoch = *s.epoch >= 0xfffffffeu ? 0u : *s.epoch + 1u;  // the next launch's partials carry another tag
  }
}

struct Plan {
  int cluster;
  uint32_t slice;
  size_t shared_bytes;
};

bool make_plan(uint64_t cols, Plan &plan) {
  for (int c = 1; c <= kMaxCluster; c *= 2) {
    const uint64_t slice = ((cols + c - 1) / c + 7) / 8 * 8;
    const size_t bytes = slice * sizeof(float);
    if (bytes <= kTwoCtaSliceBytes || (c == kMaxCluster && bytes <= kMaxSliceBytes)) {
      plan = {c, static_cast<uint32_t>(slice), bytes};
      return true;
    }
  }
  return false;
}

int launch_cluster_kernel(cudaStream_t stream, void (*kernel)(const LogitsParams), const LogitsParams &p,
                          int cluster, uint64_t clusters, size_t shared) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(clusters * cluster));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attributes[2]{};
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = cluster;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = 2;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, p));
}

// Clusters of `cluster` CTAs that can be resident at once (two CTAs per SM), cached per size.
template <int kMode>
int resident_clusters(int cluster) {
  static int cached[4][64] = {};
  int device = 0;
  cudaGetDevice(&device);
  int slot = cluster == 1 ? 0 : cluster == 2 ? 1 : cluster == 4 ? 2 : 3;
  if (device < 0 || device >= 64) device = 0;
  if (cached[slot][device] == 0) {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(cluster * 1024);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kRegStageBytes;
    cudaFuncSetAttribute(logits_regs_kernel<kMode, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(kRegStageBytes));
    cudaFuncSetAttribute(logits_regs_kernel<kMode, 9>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(kRegStageBytes));
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = cluster;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int count = 0;
    if (cudaOccupancyMaxActiveClusters(&count, logits_regs_kernel<kMode, 0>, &config) != cudaSuccess || count <= 0)
      count = sm_count() * 2 / cluster;
    cached[slot][device] = count;
  }
  return cached[slot][device];
}

// What the streaming kernel will do for a shape: chunk size, window, grid.  Host arithmetic only.
struct StreamPlan {
  int vectors = 0;        // float4 per thread and task (0 = the shape is not eligible)
  uint32_t chunks = 0;    // per row
  uint32_t chunk = 0;     // values per chunk, a multiple of 16
  uint32_t window = 0;    // rows between the passes
  uint32_t fixed = 0;     // tasks per CTA taken by position
  uint32_t help_after = kStreamHelpAfter;
  int ctas_per_sm = 0;
  unsigned grid = 0;
};

inline bool stream_eligible(uint64_t rows, uint64_t cols, int vectors) {
  return rows >= kStreamMinRows && cols % 16 == 0 && cols >= kStreamThreads * 4 && cols <= 0x7fffffffull &&
         stream_chunks(cols, vectors) <= kStreamMaxChunks;
}

uint64_t stream_workspace_bytes(uint64_t rows, uint64_t cols) {
  return kStreamHeaderBytes + rows * stream_chunks(cols, kStreamVectors) * sizeof(StreamPartial);
}

// CTAs of one instantiation that fit an SM, by the occupancy calculator, cached per device.
template <class Kernel>
int stream_resident_ctas(Kernel kernel, size_t shared_bytes, int slot) {
  static int cached[4][64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64) device = 0;
  if (cached[slot][device] == 0) {
    int count = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&count, kernel, kStreamThreads, shared_bytes) != cudaSuccess || count <= 0)
      count = 1;
    cached[slot][device] = count;
  }
  return cached[slot][device];
}

// `resident` = CTAs per SM the kernel can hold (occupancy calculator).  `tuning` may be null.
StreamPlan make_stream_plan(uint64_t rows, uint64_t cols, const hyle_b200_stream_tuning *tuning, int sms, int resident) {
  StreamPlan plan{};
  if (tuning != nullptr && tuning->chunk_vectors != 0 && tuning->chunk_vectors != kStreamVectors) return plan;
  const int vectors = kStreamVectors;
  if (!stream_eligible(rows, cols, vectors)) return plan;
  plan.vectors = vectors;
  plan.chunks = stream_chunks(cols, vectors);
  plan.chunk = static_cast<uint32_t>((cols / plan.chunks + 15) / 16 * 16);
  if (static_cast<uint64_t>(plan.chunk) * plan.chunks < cols) plan.chunk += 16;
  int per_sm = kStreamCtasPerSm;
  if (tuning != nullptr && tuning->ctas_per_sm > 0 && tuning->ctas_per_sm < per_sm) per_sm = tuning->ctas_per_sm;
  if (per_sm > resident) per_sm = resident;
  plan.ctas_per_sm = per_sm;
  const uint64_t tasks = 2 * rows * plan.chunks;
  plan.grid = clamp_grid(tasks, static_cast<uint64_t>(sms) * per_sm);
  // window: cover the tasks in flight (one computing, one loading per CTA), stay inside L2
  uint64_t window = (2ull * plan.grid + plan.chunks - 1) / plan.chunks;
  const uint64_t by_bytes = kStreamWindowBytes / (cols * sizeof(float));
  if (window > by_bytes) window = by_bytes;
  if (window > kStreamWindowMax) window = kStreamWindowMax;
  if (window < 8) window = 8;
  if (tuning != nullptr && tuning->window_rows != 0) window = tuning->window_rows;
  if (window > rows) window = rows;
  plan.window = static_cast<uint32_t>(window);
  const uint64_t head = window * plan.chunks;  // first-pass tasks before the first second-pass task
  plan.fixed = 2ull * plan.grid <= head ? 2u : plan.grid <= head ? 1u : 0u;
  if (tuning != nullptr && tuning->help_after_polls != 0) plan.help_after = tuning->help_after_polls;
  return plan;
}

template <int kMode>
int launch_stream(cudaStream_t stream, const LogitsParams &p, void *workspace, const hyle_b200_stream_tuning *tuning) {
  constexpr int kAlmost = kStreamVectors - 1;
  constexpr size_t kStage = stream_stage_bytes(kStreamVectors);
  const int resident = stream_resident_ctas(logits_stream_kernel<kMode, kStreamVectors, 0>, kStage, kMode);
  const StreamPlan plan = make_stream_plan(p.rows, p.cols, tuning, sm_count(), resident);
  if (plan.vectors == 0) return HYLE_B200_INVALID_VALUE;
  StreamParams s{};
  s.p = p;
  s.chunks = plan.chunks;
  s.chunk = plan.chunk;
  s.window = plan.window;
  s.fixed = plan.fixed;
  s.help_after = plan.help_after;
  unsigned char *base = static_cast<unsigned char *>(workspace);
  s.next_task = reinterpret_cast<unsigned long long *>(base);
  s.ticket = reinterpret_cast<uint32_t *>(base + 8);
  s.epoch = reinterpret_cast<uint32_t *>(base + 12);
  s.partials = reinterpret_cast<StreamPartial *>(base + kStreamHeaderBytes);
  const uint32_t last = p.cols - (s.chunks - 1) * s.chunk;  // the shortest chunk
  const bool almost_full = s.chunk / 4 >= static_cast<uint32_t>(kAlmost) * kStreamThreads &&
                           last / 4 >= static_cast<uint32_t>(kAlmost) * kStreamThreads;
  return launch(almost_full ? logits_stream_kernel<kMode, kStreamVectors, kAlmost> : logits_stream_kernel<kMode, kStreamVectors, 0>,
                dim3(plan.grid), dim3(kStreamThreads), kStage, stream, s);
}

template <int kMode>
int launch_logits(cudaStream_t stream, LogitsParams p, bool vec, void *workspace, uint64_t workspace_bytes,
                  const hyle_b200_stream_tuning *tuning) {
  if (p.cols == 0) return HYLE_B200_NOT_SUPPORTED;
  if constexpr (kMode != kArgmaxOnly) {
    // Many rows with an output tensor: the two-pass streaming kernel (needs the caller's workspace).
    if (vec && p.out != nullptr && p.out != static_cast<const void *>(p.in) && workspace != nullptr &&
        stream_eligible(p.rows, p.cols, kStreamVectors) && workspace_bytes >= stream_workspace_bytes(p.rows, p.cols))
      return launch_stream<kMode>(stream, p, workspace, tuning);
    if (tuning != nullptr) return HYLE_B200_INVALID_VALUE;  // tuning is for the streaming kernel only
  }
  if constexpr (kMode != kArgmaxOnly) {
    // Register-resident fast path: aligned rows of at most 8 x 20480 values.
    if (vec && p.cols <= static_cast<uint64_t>(kMaxCluster) * kRegSlice) {
      int cluster = 1;
      while (static_cast<uint64_t>(cluster) * kRegSlice < p.cols) cluster *= 2;
      p.slice = static_cast<uint32_t>(((p.cols + cluster - 1) / cluster + 7) / 8 * 8);
      const uint64_t resident = static_cast<uint64_t>(resident_clusters<kMode>(cluster));
      const uint64_t last = p.cols - static_cast<uint64_t>(cluster - 1) * p.slice;
      const bool nine_full = p.cols > static_cast<uint64_t>(cluster - 1) * p.slice && last / 4 >= 9ull * kThreads;
      return launch_cluster_kernel(stream, nine_full ? logits_regs_kernel<kMode, 9> : logits_regs_kernel<kMode, 0>, p, cluster,
                                   p.rows < resident ? p.rows : resident, kRegStageBytes);
    }
  }
  Plan plan{};
  if (!make_plan(p.cols, plan)) return HYLE_B200_NOT_SUPPORTED;
  p.slice = plan.slice;
  const size_t shared = kMode == kArgmaxOnly ? 0 : plan.shared_bytes;
  void (*kernel)(const LogitsParams);
  if constexpr (kMode == kArgmaxOnly) kernel = vec ? argmax_kernel<true> : argmax_kernel<false>;
  else kernel = vec ? logits_kernel<kMode, true> : logits_kernel<kMode, false>;
  if (shared > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return launch_cluster_kernel(stream, kernel, p, plan.cluster, p.rows < 65536 ? p.rows : 65536, shared);
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" uint64_t hyle_b200_logits_workspace_bytes(uint64_t rows, uint64_t cols) {
  return stream_workspace_bytes(rows, cols);
}

extern "C" int hyle_b200_logits_reduce_f32_tuned(hyle_b200_stream_t stream, const float *logits, uint64_t rows, uint64_t cols,
                                                 float *lse, void *probs_bf16, int32_t *argmax_index, float *argmax_value,
                                                 void *workspace, uint64_t workspace_bytes, uint32_t *status_word,
                                                 const hyle_b200_stream_tuning *tuning) {
  if (rows == 0) return HYLE_B200_OK;
  if (logits == nullptr || cols == 0 || cols > 0x7fffffffull) return HYLE_B200_INVALID_VALUE;
  if (workspace != nullptr && !aligned_to(workspace, 16)) return HYLE_B200_INVALID_VALUE;
  LogitsParams p{logits, rows, static_cast<uint32_t>(cols), 0, lse, probs_bf16, argmax_index, argmax_value, status_word};
  const bool vec = aligned_to(logits, 16) && cols % 8 == 0 && (probs_bf16 == nullptr || aligned_to(probs_bf16, 16));
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (lse == nullptr && probs_bf16 == nullptr)
    return tuning != nullptr ? HYLE_B200_INVALID_VALUE : launch_logits<kArgmaxOnly>(s, p, vec, nullptr, 0, nullptr);
  return launch_logits<kProbsBf16>(s, p, vec, workspace, workspace_bytes, tuning);
}

extern "C" int hyle_b200_logits_reduce_f32(hyle_b200_stream_t stream, const float *logits,
                                           uint64_t rows, uint64_t cols, float *lse,
                                           void *probs_bf16, int32_t *argmax_index,
                                           float *argmax_value, void *workspace,
                                           uint64_t workspace_bytes, uint32_t *status_word) {
  return hyle_b200_logits_reduce_f32_tuned(stream, logits, rows, cols, lse, probs_bf16, argmax_index, argmax_value, workspace,
                                           workspace_bytes, status_word, nullptr);
}

extern "C" int hyle_b200_softmax_f32(hyle_b200_stream_t stream, int kind, const float *in,
                                     float *out, uint64_t rows, uint64_t cols, void *workspace,
                                     uint64_t workspace_bytes, uint32_t *status_word) {
  if (rows == 0 || cols == 0) return HYLE_B200_OK;
  if (in == nullptr || out == nullptr || cols > 0x7fffffffull) return HYLE_B200_INVALID_VALUE;
  if (workspace != nullptr && !aligned_to(workspace, 16)) return HYLE_B200_INVALID_VALUE;
  LogitsParams p{in, rows, static_cast<uint32_t>(cols), 0, nullptr, out, nullptr, nullptr, status_word};
  const bool vec = aligned_to(in, 16) && aligned_to(out, 16) && cols % 8 == 0;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (kind == HYLE_B200_SOFTMAX) return launch_logits<kProbsF32>(s, p, vec, workspace, workspace_bytes, nullptr);
  if (kind == HYLE_B200_LOG_SOFTMAX) return launch_logits<kLogF32>(s, p, vec, workspace, workspace_bytes, nullptr);
  return HYLE_B200_INVALID_VALUE;
}

// Host-side introspection of the streaming kernel's schedule (no launch, no device access beyond the
// cached SM count and occupancy query): what tests and tuning sweeps read.
extern "C" int hyle_b200_logits_stream_plan(uint64_t rows, uint64_t cols, const hyle_b200_stream_tuning *tuning,
                                            hyle_b200_stream_plan *plan_out) {
  if (plan_out == nullptr) return HYLE_B200_INVALID_VALUE;
  const int resident = stream_resident_ctas(logits_stream_kernel<kProbsBf16, kStreamVectors, 0>, stream_stage_bytes(kStreamVectors),
                                            kProbsBf16);
  const StreamPlan plan = make_stream_plan(rows, cols, tuning, sm_count(), resident);
  *plan_out = hyle_b200_stream_plan{plan.vectors, plan.chunks, plan.chunk, plan.window, plan.fixed, plan.ctas_per_sm,
                                    plan.grid, plan.help_after};
  return plan.vectors == 0 ? HYLE_B200_NOT_SUPPORTED : HYLE_B200_OK;
}

extern "C" int hyle_b200_logits_stream_task(uint64_t rows, uint32_t chunks, uint32_t window, uint64_t task,
                                            uint32_t *pass_out, uint64_t *row_out, uint32_t *chunk_out) {
  if (rows == 0 || chunks == 0 || window == 0 || window > rows || pass_out == nullptr || row_out == nullptr || chunk_out == nullptr)
    return HYLE_B200_INVALID_VALUE;
  const StreamTask decoded = stream_decode(task, rows, chunks, window);
  *pass_out = decoded.pass;
  *row_out = decoded.row;
  *chunk_out = decoded.chunk_id;
  return HYLE_B200_OK;
}

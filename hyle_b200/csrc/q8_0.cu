// Q8_0 block quantise / dequantise and the global sum of squares.
//
// A Q8_0 block is 34 bytes: little-endian f16 scale, then 32 int8 codes
// (src/compute_ops/low_precision.cc:28-29).  Arithmetic, per block of 32 inputs
// (src/compute_provider_ggml/ggml_cpu_provider.cc:585-615 around ggml's reference row quantiser):
//   amax = max|x|;  d = amax / 127.0f;  id = 1.0f / d;  q = roundf(x * id);  scale = f16_rne(d)
//   f16 scale == 0, or any |x| non-finite or > 65504*127  ->  34 zero bytes (+ status bit)
//   decode: bf16_rne(f32(scale) * q)
//
// Tiling: a CTA of 256 threads takes 256 consecutive blocks (8192 values, 16 KB of bf16) at a time.
// Thread t owns the 16-byte vectors k*256+t, k = 0..3; four neighbouring lanes share a block, so
// amax is two xor shuffles.  The 34-byte blocks are only 2-byte aligned, so the 8704 bytes a tile
// produces are staged in shared memory and leave as 16-byte coalesced stores.
#include "common.cuh"

#include <math_constants.h>
#include <type_traits>

#include <cstring>

namespace hb {
namespace {

constexpr int kThreads = 256;
constexpr int kVectorsPerThread = 4;
constexpr int kTileBlocks = 256;
constexpr int kTileBytes = kTileBlocks * 34;  // 8704 = 544 * 16
constexpr int kMaxPartials = 4096;
constexpr uint64_t kWorkspaceBytes = 64 + sizeof(double) * kMaxPartials;  // static scheme: header + CTA partials

// |x| <= 65504*127 as an integer comparison on the magnitude bits; NaN and inf compare above it
// (ggml_cpu_provider.cc:563-584).
constexpr uint32_t kLimitBitsF32 = 0x4afde040u;  // bits of 8319008.0f = 65504 * 127

// Round half away from zero WITHOUT the conversion unit (F2I/I2F run at a quarter of the FP32 rate
// and this kernel needs one rounding per value).  For |p| < 2^22:
//   s = RZ(|p| + 0.5)            never crosses an integer upward (0.49999997 + 0.5 stays below 1)
//   f = RZ(s + 2^23)             = 2^23 + floor(s): the integer sits in the low mantissa bits
//   magnitude = f - 2^23         exact
// The signed integer is then formed as 1.5 * 2^23 + sign * magnitude, whose bit pattern holds the
// two's-complement code in its low byte; subtracting 1.5 * 2^23 again gives the code as a float.
// The signed integer is the magnitude with p's sign bit (one logic operation); added to 1.5 * 2^23 it
// gives a bit pattern whose low byte is the two's-complement code.  Five FP32-pipe operations per value.
struct Rounded {
  float value;     // roundf(p) as a float; -0 when p < 0 rounds to 0: the decode adds +0 (see decoded_value)
  uint32_t bits;   // bit pattern whose low byte is the int8 code
};
__device__ __forceinline__ Rounded round_half_away(float p) {
  const float f = __fadd_rz(__fadd_rz(fabsf(p), 0.5f), 8388608.0f);
  const float magnitude = __fadd_rn(f, -8388608.0f);
  Rounded r;
  r.value = __uint_as_float(__float_as_uint(magnitude) | (__float_as_uint(p) & 0x80000000u));
  r.bits = __float_as_uint(__fadd_rn(r.value, 12582912.0f));  // 1.5 * 2^23 + signed integer, exact
  return r;
}
// scale * (float)code as the CPU forms it: the code 0 is +0 there, so a product of -0 becomes +0
// (x + +0 is x for every other x, and (-0) + (+0) is +0 in round-to-nearest).
__device__ __forceinline__ float decoded_value(float scale, float rounded) { return __fmaf_rn(scale, rounded, 0.0f); }

// amax / 127 and 1 / d, correctly rounded like the CPU's two IEEE divisions, without the division
// sequence: q0 = RN(a * y) with y = RN(1 / 127), r = a - 127 * q0 exactly (one fma), d = RN(q0 + r * y)
// (Markstein's correction: with a correctly rounded reciprocal and a faithful q0 the result is the correctly
// rounded quotient); __frcp_rn is the IEEE reciprocal.  hyle_b200_selfcheck_q8_0_scale compares both with
// __fdiv_rn for EVERY magnitude the kernel accepts (tests/test_gpu_parity.py).
__device__ __forceinline__ float scale_quotient(float amax) {
  constexpr float kReciprocal127 = 0.00787401574803149606f;
  const float q0 = __fmul_rn(amax, kReciprocal127);
  const float r = __fmaf_rn(-127.0f, q0, amax);
  return __fmaf_rn(r, kReciprocal127, q0);
}

// Eight consecutive values as f32 plus the largest magnitude bit pattern among them.
template <int kDtype>
__device__ __forceinline__ void load8(const void *in, uint64_t element, float v[8], uint32_t &amax_bits) {
  if constexpr (kDtype == HYLE_B200_BF16) {
    const uint4 raw = ld_stream(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(in) + element));
    v[0] = bf16_lo(raw.x); v[1] = bf16_hi(raw.x); v[2] = bf16_lo(raw.y); v[3] = bf16_hi(raw.y);
    v[4] = bf16_lo(raw.z); v[5] = bf16_hi(raw.z); v[6] = bf16_lo(raw.w); v[7] = bf16_hi(raw.w);
    const uint32_t m = __vmaxu2(__vmaxu2(raw.x & 0x7fff7fffu, raw.y & 0x7fff7fffu),
                                __vmaxu2(raw.z & 0x7fff7fffu, raw.w & 0x7fff7fffu));
    amax_bits = max(m & 0xffffu, m >> 16) << 16;
  } else if constexpr (kDtype == HYLE_B200_F16) {
    const uint4 raw = ld_stream(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(in) + element));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    amax_bits = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = f16_to_f32(static_cast<unsigned short>(w[i] & 0xffffu));
      v[2 * i + 1] = f16_to_f32(static_cast<unsigned short>(w[i] >> 16));
      amax_bits = max(amax_bits, max(__float_as_uint(v[2 * i]) & 0x7fffffffu,
                                     __float_as_uint(v[2 * i + 1]) & 0x7fffffffu));
    }
  } else {
    const float4 a = ld_stream(reinterpret_cast<const float4 *>(static_cast<const float *>(in) + element));
    const float4 b = ld_stream(reinterpret_cast<const float4 *>(static_cast<const float *>(in) + element) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    amax_bits = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7fffffffu);
  }
}

struct SumSquaresState {
  uint32_t *ticket;
  double *partials;
};

__device__ __forceinline__ SumSquaresState workspace_state(void *workspace) {
  return {static_cast<uint32_t *>(workspace),
          reinterpret_cast<double *>(static_cast<unsigned char *>(workspace) + 64)};
}

// ---- dynamic tile scheduling with an order-independent result ---------------------------------
// On this GPU a persistent grid that pulls tiles from one atomic counter finishes the 4 GiB sweep
// point 6 % sooner than a static tile-to-CTA assignment (all CTAs stay within a narrow window of
// addresses and nobody waits for the slowest SM).  The price is that "which CTA summed which tile"
// is no longer fixed, so the sum of squares is built from per-TILE sums instead of per-CTA sums:
//   tile_sums[tile]   f32 per thread over its 32 values, f32 warp tree, 8 warp values added in f64;
//                     a plain store, no fence and no atomic per tile (a fence would wait for the
//                     tile's streaming stores: measured, that cost more than the scheduling gains)
//   *sum_out          the CTA that leaves last adds all tile sums: thread t takes t, t+256, ... in
//                     order, then the fixed warp / CTA tree (2 MB of f64 at the largest point)
// Every value is a function of the data only, so the result is bit-identical from run to run and
// for any grid size.  The tile sums live after the static scheme's area of the workspace.
struct DynamicState {
  uint32_t *ticket;                 // CTAs that have left
  unsigned long long *next_tile;    // tile counter (tiles gridDim.x.. are handed out through it)
  double *tile_sums;
};
__host__ __device__ inline uint64_t dynamic_bytes(uint64_t tiles) { return tiles * 8; }
__device__ __forceinline__ DynamicState dynamic_state(void *workspace) {
  unsigned char *base = static_cast<unsigned char *>(workspace);
  return {reinterpret_cast<uint32_t *>(base), reinterpret_cast<unsigned long long *>(base + 16),
          reinterpret_cast<double *>(base + kWorkspaceBytes)};
}

// ---- sum of squares across GPUs: the exchange fused into the kernel's tail -----------------------
// When the tensor is row-sharded over several GPUs, each GPU's finishing CTA holds that GPU's sum.
// Instead of ending the kernel and launching a collective, the finishing CTA's first warp sends the
// eight bytes straight into every peer's mailbox (plain stores to peer-mapped memory, over NVLink)
// and waits for the peers' values in its own.  Lane r talks to rank r.
//   mailbox of one rank: words[2 parities][kMaxRanks senders][2], 8 bytes each.  A value travels as
//   two words {low half, epoch} and {high half, epoch}: an 8-byte store is atomic, so a word whose
//   epoch matches carries valid data and no fence or separate flag is needed (the same idea as
//   NCCL's LL protocol).  Consecutive epochs use different parities, so a fast rank that is already
//   one call ahead never overwrites a word a slow rank is still waiting for; it cannot be two
//   calls ahead, because its previous call needed the slow rank's word of that call.
//   The received values are added in rank order, so every rank gets the same bits.
// Every wait is bounded: after `poll_limit` polls the rank gives up, reports NaN and sets
// HYLE_B200_STATUS_EXCHANGE_TIMEOUT; the kernel ends normally and the context stays usable.
constexpr int kMaxRanks = HYLE_B200_EXCHANGE_MAX_RANKS;
struct Exchange {
  unsigned long long *mailbox[kMaxRanks];  // mailbox[r]: rank r's mailbox as this GPU addresses it
  uint32_t world = 0, rank = 0, epoch = 0, poll_limit = 0;
};
static_assert(HYLE_B200_EXCHANGE_MAILBOX_BYTES == 2 * kMaxRanks * 2 * 8, "mailbox layout");

__device__ __forceinline__ void store_relaxed_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long load_relaxed_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(__cvta_generic_to_global(p)) : "memory");
  return v;
}

// Called by one full warp.  Returns the sum over all ranks (NaN after a timeout) in every lane.
__device__ __forceinline__ double exchange_sum(double mine, const Exchange &ex, uint32_t *status_word) {
  const uint32_t lane = threadIdx.x & 31;
  const unsigned long long epoch = static_cast<unsigned long long>(ex.epoch) << 32;
  const uint32_t slot = (ex.epoch & 1u) * kMaxRanks;
  double value = 0.0;
  bool arrived = true;
  if (lane < ex.world) {
    const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(mine));
    unsigned long long *peer = nullptr;
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (lane == r) peer = ex.mailbox[r];
    unsigned long long *dst = peer + (slot + ex.rank) * 2;
    store_relaxed_sys(dst, (bits & 0xffffffffull) | epoch);
    store_relaxed_sys(dst + 1, (bits >> 32) | epoch);
    unsigned long long *own = nullptr;
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (ex.rank == r) own = ex.mailbox[r];
    const unsigned long long *src = own + (slot + lane) * 2;
    unsigned long long low = load_relaxed_sys(src), high = load_relaxed_sys(src + 1);
    for (uint32_t polls = 0; ((low ^ epoch) >> 32 != 0 || (high ^ epoch) >> 32 != 0) && polls < ex.poll_limit; ++polls) {
      __nanosleep(64);
      low = load_relaxed_sys(src);
      high = load_relaxed_sys(src + 1);
    }
    arrived = (low ^ epoch) >> 32 == 0 && (high ^ epoch) >> 32 == 0;
    value = __longlong_as_double(static_cast<long long>((low & 0xffffffffull) | (high << 32)));
  }
  arrived = __all_sync(kFullMask, arrived);
  double total = 0.0;
  for (uint32_t r = 0; r < ex.world; ++r) total += __shfl_sync(kFullMask, value, r);  // rank order
  if (!arrived) {
    total = __longlong_as_double(0x7ff8000000000000ll);
    if (lane == 0 && status_word != nullptr) atomicOr(status_word, HYLE_B200_STATUS_EXCHANGE_TIMEOUT);
  }
  return total;
}

// Deterministic grid-wide sum: fixed-order CTA reduction, one partial per CTA, and the CTA that
// takes the last ticket adds the partials in index order.  Which CTA is last does not matter.
__device__ __forceinline__ void finish_sum(double thread_sum, SumSquaresState ws, double *sum_out) {
  __shared__ double s_warp[kThreads / 32];
  __shared__ bool s_last;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const double w = warp_sum(thread_sum);
  if (lane == 0) s_warp[warp] = w;
  __syncthreads();
  if (t == 0) {
    double total = s_warp[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) total += s_warp[i];
    ws.partials[blockIdx.x] = total;
    __threadfence();
    const uint32_t taken = atomicAdd(ws.ticket, 1u);
    s_last = taken == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last && warp == 0) {
    __threadfence();
    double acc = 0.0;
    for (uint32_t i = lane; i < gridDim.x; i += 32) acc += __ldcg(ws.partials + i);
    acc = warp_sum(acc);
    if (lane == 0) {
      *sum_out = acc;
      *ws.ticket = 0;  // the workspace is ready for the next stream-ordered launch
    }
  }
}

// kEncode: write Q8_0 blocks.  kDecode: write decoded bf16.  kSumSquares: accumulate sum x^2.
// kDynamic (needs kEncode and kSumSquares): tiles come from the workspace's counter.
template <int kDtype, bool kEncode, bool kDecode, bool kSumSquares, bool kDynamic = false>
__global__ void __launch_bounds__(kThreads, 4)  // four CTAs per SM: 64 registers
q8_0_kernel(const void *__restrict__ in, uint64_t blocks, unsigned char *__restrict__ blocks_out,
            unsigned short *__restrict__ decoded, double *sum_out, uint32_t *status_word,
            void *workspace, int out_aligned, const Exchange exchange) {
  grid_dependency_sync();
  __shared__ __align__(16) unsigned char staged[2][kTileBytes];
  const int t = threadIdx.x;
  const int sub = t & 3;  // which quarter of a block this lane holds
  const uint64_t tiles = (blocks + kTileBlocks - 1) / kTileBlocks;
  static_assert(!kDynamic || (kEncode && kSumSquares), "the dynamic scheme rides on the encode barrier");
  __shared__ float s_warp_sum[2][kThreads / 32];
  __shared__ unsigned long long s_next_tile[2];
  DynamicState dynamic{};
  if constexpr (kDynamic) dynamic = dynamic_state(workspace);
  double sum = 0.0;
  bool invalid_seen = false;
  int buffer = 0;
  for (uint64_t tile = blockIdx.x; tile < tiles; buffer ^= 1) {
    // The next tile is requested now and read after this tile's barrier: no barrier of its own.
    if constexpr (kDynamic) {
      if (t == 0) s_next_tile[buffer] = gridDim.x + atomicAdd(dynamic.next_tile, 1ull);
    }
    const uint64_t first_block = tile * kTileBlocks;
    const uint32_t tile_blocks = static_cast<uint32_t>(min(static_cast<uint64_t>(kTileBlocks), blocks - first_block));
    const bool full = tile_blocks == kTileBlocks;
    // The tile's work, compiled twice: a full tile (all but the last) carries no per-block bounds test, so its
    // loads, staging stores and decoded stores sit in straight-line code (the tests cost three branches with
    // their convergence barriers per eight values).
    float tile_sum = 0.0f;
    auto process = [&](auto full_tag) {
      constexpr bool kFullTile = decltype(full_tag)::value;
      float v[kVectorsPerThread][8];
      uint32_t amax_bits[kVectorsPerThread];
#pragma unroll
      for (int k = 0; k < kVectorsPerThread; ++k) {
        const uint32_t block = k * 64 + (t >> 2);
        if (kFullTile || block < tile_blocks) {
          load8<kDtype>(in, (first_block + block) * 32 + sub * 8, v[k], amax_bits[k]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[k][i] = 0.0f;
          amax_bits[k] = 0;
        }
      }
      // Block maxima: after two xor shuffles all four lanes of a group hold the maximum of each of
      // their four blocks.  The two IEEE divisions per block are then done ONCE: lane `sub` of the
      // group handles block `sub` and the group shares the results by shuffle.
      uint32_t mine = 0;
#pragma unroll
      for (int k = 0; k < kVectorsPerThread; ++k) {
        uint32_t m = amax_bits[k];
        m = max(m, __shfl_xor_sync(kFullMask, m, 1));
        m = max(m, __shfl_xor_sync(kFullMask, m, 2));
        if (k == sub) mine = m;
      }
      const bool valid = mine <= kLimitBitsF32;
      const float d = scale_quotient(__uint_as_float(mine));
      const unsigned short scale = f32_to_f16(d);
      // inverse 0: a block whose scale rounds to zero (all its products are +-0, all its codes and decoded
      // values come out as zeros by themselves); inverse NaN: invalid input, patched below
      const float my_inverse = !valid ? CUDART_NAN_F : (scale == 0 ? 0.0f : __frcp_rn(d));
      const uint32_t my_scale = valid ? static_cast<uint32_t>(scale) : 0u;
      invalid_seen |= !valid;
      // Invalid input (NaN, infinity, a magnitude beyond 65504 * 127) makes its block all zeros.  No valid block
      // needs a select, so the patch is compiled into a second copy of the loop below that a warp enters only
      // when one of the 32 blocks it handles in this tile is invalid (one vote per tile).
      auto emit = [&](auto patch_tag) {
      constexpr bool kPatch = decltype(patch_tag)::value;
#pragma unroll
      for (int k = 0; k < kVectorsPerThread; ++k) {
        const uint32_t block = k * 64 + (t >> 2);
        const int source = (threadIdx.x & 28) + k;  // lane within the warp that divided for block k
        const float inverse = __shfl_sync(kFullMask, my_inverse, source);
        const uint32_t stored_scale = __shfl_sync(kFullMask, my_scale, source);
        if constexpr (kSumSquares) {
#pragma unroll
          for (int i = 0; i < 8; ++i) tile_sum = fmaf(v[k][i], v[k][i], tile_sum);
        }
        Rounded q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = round_half_away(__fmul_rn(v[k][i], inverse));
        // two codes per 16-bit store (a block starts on a 2-byte boundary only): the low bytes of two words
        uint32_t pair[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pair[i] = __byte_perm(q[2 * i].bits, q[2 * i + 1].bits, 0x0040);
        if constexpr (kPatch) {
          if (inverse != inverse) {
#pragma unroll
            for (int i = 0; i < 4; ++i) pair[i] = 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i].value = 0.0f;
          }
        }
        if constexpr (kEncode) {
          if (kFullTile || block < tile_blocks) {
            unsigned short *dst = reinterpret_cast<unsigned short *>(staged[buffer] + block * 34);
            if (sub == 0) dst[0] = static_cast<unsigned short>(stored_scale);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[1 + sub * 4 + i] = static_cast<unsigned short>(pair[i]);
          }
        }
        if constexpr (kDecode) {
          if (kFullTile || block < tile_blocks) {
            const float s = f16_to_f32(static_cast<unsigned short>(stored_scale));
            uint4 out = make_uint4(pack_bf16x2(decoded_value(s, q[0].value), decoded_value(s, q[1].value)),
                                   pack_bf16x2(decoded_value(s, q[2].value), decoded_value(s, q[3].value)),
                                   pack_bf16x2(decoded_value(s, q[4].value), decoded_value(s, q[5].value)),
                                   pack_bf16x2(decoded_value(s, q[6].value), decoded_value(s, q[7].value)));
            st_stream(reinterpret_cast<uint4 *>(decoded + (first_block + block) * 32 + sub * 8), out);
          }
        }
      }
      };
      if (__builtin_expect(__any_sync(kFullMask, !valid), 0)) emit(std::true_type{});
      else emit(std::false_type{});
    };
    if (full) process(std::true_type{});
    else process(std::false_type{});
    if constexpr (kSumSquares && !kDynamic) sum += static_cast<double>(tile_sum);
    if constexpr (kDynamic) {
      const float warp_total = warp_sum(tile_sum);
      if ((t & 31) == 0) s_warp_sum[buffer][t >> 5] = warp_total;
    }
    uint64_t next_tile = tile + gridDim.x;
    if constexpr (kEncode) {
      // One barrier per tile: the staging buffer alternates, and this barrier also orders the
      // previous tile's reads of the other buffer before the next tile's writes to it.
      __syncthreads();
      if constexpr (kDynamic) {
        next_tile = s_next_tile[buffer];
        if (t == 0) {
          double tile_total = static_cast<double>(s_warp_sum[buffer][0]);
#pragma unroll
          for (int w = 1; w < kThreads / 32; ++w) tile_total += static_cast<double>(s_warp_sum[buffer][w]);
          dynamic.tile_sums[tile] = tile_total;
        }
      }
      unsigned char *dst = blocks_out + first_block * 34;
      if (full && out_aligned) {
        const uint4 *src = reinterpret_cast<const uint4 *>(staged[buffer]);
        for (int i = t; i < kTileBytes / 16; i += kThreads) st_stream(reinterpret_cast<uint4 *>(dst) + i, src[i]);
      } else {
        const unsigned short *src = reinterpret_cast<const unsigned short *>(staged[buffer]);
        for (uint32_t i = t; i < tile_blocks * 17; i += kThreads) st_stream(reinterpret_cast<unsigned short *>(dst) + i, src[i]);
      }
    }
    tile = next_tile;
  }
  if (status_word != nullptr && invalid_seen) atomicOr(status_word, HYLE_B200_STATUS_INVALID_Q8_INPUT);
  if constexpr (kDynamic) {
    // The CTA that leaves last adds the tile sums in a fixed order and re-arms the workspace.
    __shared__ bool s_last;
    __shared__ double s_final[kThreads / 32];
    __syncthreads();
    if (t == 0) {
      __threadfence();  // this CTA's tile sums are visible before its ticket
      s_last = atomicAdd(dynamic.ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      double acc = 0.0;
      for (uint64_t i = t; i < tiles; i += kThreads) acc += __ldcg(dynamic.tile_sums + i);
      acc = warp_sum(acc);
      if ((t & 31) == 0) s_final[t >> 5] = acc;
      __syncthreads();
      if (t < 32) {
        double total = s_final[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) total += s_final[w];
        if (exchange.world > 1) total = exchange_sum(total, exchange, status_word);
        if (t == 0) {
          *sum_out = total;
          *dynamic.ticket = 0u;
          *dynamic.next_tile = 0ull;
        }
      }
    }
  } else if constexpr (kSumSquares) {
    finish_sum(sum, workspace_state(workspace), sum_out);
  }
}

// Decode-only: a tile's 8704 bytes are pulled into shared memory with 16-byte loads, then every
// thread rebuilds its four vectors.
__global__ void __launch_bounds__(kThreads)
q8_0_decode_kernel(const unsigned char *__restrict__ blocks_in, uint64_t blocks,
                   unsigned short *__restrict__ decoded, int in_aligned) {
  grid_dependency_sync();
  __shared__ __align__(16) unsigned char staged[2][kTileBytes];
  const int t = threadIdx.x, sub = t & 3;
  const uint64_t tiles = (blocks + kTileBlocks - 1) / kTileBlocks;
  int buffer = 0;
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, buffer ^= 1) {
    const uint64_t first_block = tile * kTileBlocks;
    const uint32_t tile_blocks = static_cast<uint32_t>(min(static_cast<uint64_t>(kTileBlocks), blocks - first_block));
    const bool full = tile_blocks == kTileBlocks;
    const unsigned char *src = blocks_in + first_block * 34;
    if (full && in_aligned) {
      uint4 *dst = reinterpret_cast<uint4 *>(staged[buffer]);
      uint4 held[3];
#pragma unroll
      for (int j = 0; j < 3; ++j)
        if (t + j * kThreads < kTileBytes / 16) held[j] = ld_stream(reinterpret_cast<const uint4 *>(src) + t + j * kThreads);
#pragma unroll
      for (int j = 0; j < 3; ++j)
        if (t + j * kThreads < kTileBytes / 16) dst[t + j * kThreads] = held[j];
    } else {
      unsigned short *dst = reinterpret_cast<unsigned short *>(staged[buffer]);
      for (uint32_t i = t; i < tile_blocks * 17; i += kThreads) dst[i] = ld_stream(reinterpret_cast<const unsigned short *>(src) + i);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kVectorsPerThread; ++k) {
      const uint32_t block = k * 64 + (t >> 2);
      if (full || block < tile_blocks) {
        const unsigned short *b = reinterpret_cast<const unsigned short *>(staged[buffer] + block * 34);
        const float s = f16_to_f32(b[0]);
        uint32_t out[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned short pair = b[1 + sub * 4 + i];
          const float lo = static_cast<float>(static_cast<int>(static_cast<signed char>(pair & 0xffu)));
          const float hi = static_cast<float>(static_cast<int>(static_cast<signed char>(pair >> 8)));
          out[i] = pack_bf16x2(__fmul_rn(s, lo), __fmul_rn(s, hi));
        }
        st_stream(reinterpret_cast<uint4 *>(decoded + (first_block + block) * 32 + sub * 8),
                  make_uint4(out[0], out[1], out[2], out[3]));
      }
    }
  }
}

// Sum of squares alone: a pure read stream.
__global__ void __launch_bounds__(kThreads)
sum_squares_bf16_kernel(const uint4 *__restrict__ in, uint64_t vectors,
                        const unsigned short *__restrict__ tail, uint32_t tail_count, double *sum_out,
                        void *workspace) {
  grid_dependency_sync();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  double sum = 0.0;
  auto squares8 = [](uint4 v, float acc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = bf16_lo(w[j]), hi = bf16_hi(w[j]);
      acc = fmaf(hi, hi, fmaf(lo, lo, acc));
    }
    return acc;
  };
  for (; i + 3 * stride < vectors; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = ld_stream(in + i + k * stride);
    float part = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) part = squares8(v[k], part);
    sum += static_cast<double>(part);
  }
  for (; i < vectors; i += stride) sum += static_cast<double>(squares8(ld_stream(in + i), 0.0f));
  if (blockIdx.x == 0 && threadIdx.x < tail_count) {
    const float f = bf16_to_f32(tail[threadIdx.x]);
    sum += static_cast<double>(f * f);
  }
  finish_sum(sum, workspace_state(workspace), sum_out);
}

unsigned q8_grid(uint64_t blocks) {
  const uint64_t tiles = (blocks + kTileBlocks - 1) / kTileBlocks;
  return clamp_grid(tiles, min(static_cast<uint64_t>(kMaxPartials), static_cast<uint64_t>(sm_count()) * 6));
}

}  // namespace
}  // namespace hb

using namespace hb;

// Every magnitude the encoder accepts (bit patterns 0 ... 65504 * 127), and for each the scale it leads to:
// the two shortcuts against the IEEE divisions they replace.
__global__ void __launch_bounds__(kThreads) selfcheck_scale_kernel(unsigned long long *mismatches) {
  unsigned long long bad = 0;
  for (uint64_t bits = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; bits <= kLimitBitsF32;
       bits += static_cast<uint64_t>(gridDim.x) * kThreads) {
    const float amax = __uint_as_float(static_cast<uint32_t>(bits));
    const float d = scale_quotient(amax);
    bad += __float_as_uint(d) != __float_as_uint(__fdiv_rn(amax, 127.0f));
    if (f32_to_f16(d) != 0) bad += __float_as_uint(__frcp_rn(d)) != __float_as_uint(__fdiv_rn(1.0f, d));
  }
  bad = __reduce_add_sync(kFullMask, static_cast<unsigned>(bad));
  if ((threadIdx.x & 31) == 0 && bad != 0) atomicAdd(mismatches, bad);
}

extern "C" int hyle_b200_selfcheck_q8_0_scale(hyle_b200_stream_t stream, unsigned long long *mismatches) {
  if (mismatches == nullptr || !aligned_to(mismatches, 8)) return HYLE_B200_INVALID_VALUE;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const cudaError_t cleared = cudaMemsetAsync(mismatches, 0, sizeof(unsigned long long), s);
  if (cleared != cudaSuccess) return static_cast<int>(cleared);
  return launch(selfcheck_scale_kernel, dim3(static_cast<unsigned>(sm_count()) * 8), dim3(kThreads), 0, s, mismatches);
}

extern "C" uint64_t hyle_b200_sum_squares_workspace_bytes(uint64_t count) {
  const uint64_t tiles = (count / 32 + kTileBlocks - 1) / kTileBlocks;
  return kWorkspaceBytes + dynamic_bytes(tiles);
}

extern "C" int hyle_b200_q8_0_encode(hyle_b200_stream_t stream, int dtype, const void *in,
                                     uint64_t count, void *blocks_out, uint32_t *status_word) {
  if (count == 0) return HYLE_B200_OK;
  if (in == nullptr || blocks_out == nullptr || count % 32 != 0 || !aligned_to(blocks_out, 2))
    return HYLE_B200_INVALID_VALUE;
  if (!aligned_to(in, 16)) return HYLE_B200_NOT_SUPPORTED;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const uint64_t blocks = count / 32;
  const unsigned grid = q8_grid(blocks);
  const int out_aligned = aligned_to(blocks_out, 16);
  auto *out = static_cast<unsigned char *>(blocks_out);
  int launch_status = HYLE_B200_OK;
  if (dtype == HYLE_B200_BF16)
    launch_status = launch(q8_0_kernel<HYLE_B200_BF16, true, false, false>, dim3(grid), dim3(kThreads), 0, s, in, blocks, out, nullptr, nullptr, status_word, nullptr, out_aligned, Exchange{});
  else if (dtype == HYLE_B200_F16)
    launch_status = launch(q8_0_kernel<HYLE_B200_F16, true, false, false>, dim3(grid), dim3(kThreads), 0, s, in, blocks, out, nullptr, nullptr, status_word, nullptr, out_aligned, Exchange{});
  else if (dtype == HYLE_B200_F32)
    launch_status = launch(q8_0_kernel<HYLE_B200_F32, true, false, false>, dim3(grid), dim3(kThreads), 0, s, in, blocks, out, nullptr, nullptr, status_word, nullptr, out_aligned, Exchange{});
  else
    return HYLE_B200_INVALID_VALUE;
  return launch_status;
}

extern "C" int hyle_b200_q8_0_decode_bf16(hyle_b200_stream_t stream, const void *blocks,
                                          uint64_t count, void *out_bf16) {
  if (count == 0) return HYLE_B200_OK;
  if (blocks == nullptr || out_bf16 == nullptr || count % 32 != 0 || !aligned_to(blocks, 2))
    return HYLE_B200_INVALID_VALUE;
  if (!aligned_to(out_bf16, 16)) return HYLE_B200_NOT_SUPPORTED;
  const uint64_t n = count / 32;
  return launch(q8_0_decode_kernel, dim3(q8_grid(n)), dim3(kThreads), 0, reinterpret_cast<cudaStream_t>(stream), 
      static_cast<const unsigned char *>(blocks), n, static_cast<unsigned short *>(out_bf16),
      aligned_to(blocks, 16));
}

extern "C" int hyle_b200_sum_squares_bf16(hyle_b200_stream_t stream, const void *in, uint64_t count,
                                          double *sum_out, void *workspace, uint64_t workspace_bytes) {
  if (sum_out == nullptr || workspace == nullptr || workspace_bytes < kWorkspaceBytes ||
      !aligned_to(workspace, 8) || (in == nullptr && count != 0))
    return HYLE_B200_INVALID_VALUE;
  if (!aligned_to(in, 16)) return HYLE_B200_NOT_SUPPORTED;
  const uint64_t vectors = count / 8;
  const uint32_t tail = static_cast<uint32_t>(count % 8);
  const unsigned grid = clamp_grid((vectors + kThreads * 4 - 1) / (kThreads * 4),
                                   min(static_cast<uint64_t>(kMaxPartials), static_cast<uint64_t>(sm_count()) * 8));
  return launch(sum_squares_bf16_kernel, dim3(grid), dim3(kThreads), 0, reinterpret_cast<cudaStream_t>(stream), 
      static_cast<const uint4 *>(in), vectors, static_cast<const unsigned short *>(in) + vectors * 8, tail,
      sum_out, workspace);
}

namespace {
// About ten seconds of polling (each poll sleeps at least 64 ns and reads two words through L2).
constexpr uint32_t kDefaultPollLimit = 1u << 23;

int roundtrip(hyle_b200_stream_t stream, const void *in, uint64_t count, void *blocks_out, void *decoded_bf16,
              double *sum_squares_out, uint32_t *status_word, void *workspace, uint64_t workspace_bytes,
              const Exchange &exchange) {
  if (in == nullptr && count != 0) return HYLE_B200_INVALID_VALUE;
  if (blocks_out == nullptr || decoded_bf16 == nullptr || sum_squares_out == nullptr ||
      workspace == nullptr || workspace_bytes < hyle_b200_sum_squares_workspace_bytes(count) ||
      !aligned_to(workspace, 8) || count % 32 != 0 || !aligned_to(blocks_out, 2))
    return HYLE_B200_INVALID_VALUE;
  if (!aligned_to(in, 16) || !aligned_to(decoded_bf16, 16)) return HYLE_B200_NOT_SUPPORTED;
  const uint64_t blocks = count / 32;
  const uint64_t tiles = (blocks + kTileBlocks - 1) / kTileBlocks;
  // Persistent grid of what fits at once (four CTAs per SM at 64 registers); the rest of the tiles
  // are pulled from the workspace's counter.
  const unsigned grid = clamp_grid(tiles, static_cast<uint64_t>(sm_count()) * 4);
  return launch(q8_0_kernel<HYLE_B200_BF16, true, true, true, true>, dim3(grid), dim3(kThreads), 0,
                reinterpret_cast<cudaStream_t>(stream), in, blocks, static_cast<unsigned char *>(blocks_out),
                static_cast<unsigned short *>(decoded_bf16), sum_squares_out, status_word, workspace,
                aligned_to(blocks_out, 16), exchange);
}

}  // namespace

extern "C" int hyle_b200_q8_0_roundtrip_bf16(hyle_b200_stream_t stream, const void *in,
                                             uint64_t count, void *blocks_out, void *decoded_bf16,
                                             double *sum_squares_out, uint32_t *status_word,
                                             void *workspace, uint64_t workspace_bytes) {
  return roundtrip(stream, in, count, blocks_out, decoded_bf16, sum_squares_out, status_word, workspace,
                   workspace_bytes, Exchange{});
}

extern "C" int hyle_b200_q8_0_roundtrip_bf16_exchange(
    hyle_b200_stream_t stream, const void *in, uint64_t count, void *blocks_out, void *decoded_bf16,
    double *sum_squares_out, uint32_t *status_word, void *workspace, uint64_t workspace_bytes,
    void *const *mailboxes, uint32_t world, uint32_t rank, uint32_t epoch, uint32_t poll_limit) {
  if (world == 0 || world > HYLE_B200_EXCHANGE_MAX_RANKS || rank >= world || epoch == 0 || mailboxes == nullptr)
    return HYLE_B200_INVALID_VALUE;
  Exchange exchange{};
  for (uint32_t r = 0; r < world; ++r) {
    if (mailboxes[r] == nullptr || !aligned_to(mailboxes[r], 8)) return HYLE_B200_INVALID_VALUE;
    exchange.mailbox[r] = static_cast<unsigned long long *>(mailboxes[r]);
  }
  exchange.world = world;
  exchange.rank = rank;
  exchange.epoch = epoch;
  exchange.poll_limit = poll_limit != 0 ? poll_limit : kDefaultPollLimit;
  return roundtrip(stream, in, count, blocks_out, decoded_bf16, sum_squares_out, status_word, workspace,
                   workspace_bytes, exchange);
}

extern "C" int hyle_b200_exchange_create(void **mailbox, unsigned char *handle_out) {
  if (mailbox == nullptr || handle_out == nullptr) return HYLE_B200_INVALID_VALUE;
  static_assert(sizeof(cudaIpcMemHandle_t) == HYLE_B200_EXCHANGE_HANDLE_BYTES, "handle size");
  void *pointer = nullptr;
  cudaError_t error = cudaMalloc(&pointer, HYLE_B200_EXCHANGE_MAILBOX_BYTES);
  if (error != cudaSuccess) return static_cast<int>(error);
  error = cudaMemset(pointer, 0, HYLE_B200_EXCHANGE_MAILBOX_BYTES);
  cudaIpcMemHandle_t handle;
  if (error == cudaSuccess) error = cudaIpcGetMemHandle(&handle, pointer);
  if (error != cudaSuccess) {
    cudaFree(pointer);
    return static_cast<int>(error);
  }
  memcpy(handle_out, &handle, sizeof handle);
  *mailbox = pointer;
  return HYLE_B200_OK;
}

extern "C" int hyle_b200_exchange_open(const unsigned char *handle, void **peer_mailbox) {
  if (handle == nullptr || peer_mailbox == nullptr) return HYLE_B200_INVALID_VALUE;
  cudaIpcMemHandle_t copy;
  memcpy(&copy, handle, sizeof copy);
  return static_cast<int>(cudaIpcOpenMemHandle(peer_mailbox, copy, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int hyle_b200_exchange_close(void *peer_mailbox) {
  return peer_mailbox == nullptr ? HYLE_B200_INVALID_VALUE : static_cast<int>(cudaIpcCloseMemHandle(peer_mailbox));
}

extern "C" int hyle_b200_exchange_destroy(void *mailbox) {
  return mailbox == nullptr ? HYLE_B200_INVALID_VALUE : static_cast<int>(cudaFree(mailbox));
}

// ------------------------------------------------------------------------------------------------
// Round trip for callers that cannot allocate.
//
// Some hosts of this library never get to call cudaMalloc: code running inside a framework that
// owns every byte of device memory through its own pool, a provider whose enqueue() contract
// forbids allocation and that was handed no workspace, or a process that must not disturb a
// memory budget fixed at start-up.  For them the per-CTA partial sums and the ticket counter of
// the sum of squares live in the library image itself: a file-scope device array of fixed size,
// resident on every GPU that loads the library until the process exits.
//
// The array bounds the launch: at most kStaticPartials CTAs, and the entry point accepts at most
// HYLE_B200_STATIC_MAX_VALUES values per call.  All calls on a device share the one array, so two
// calls whose kernels may run at the same time (different streams) race on it; calls ordered on
// one stream are fine.  The array keeps what the previous call left behind, so the ticket counter
// is cleared on the stream before every launch.
// ------------------------------------------------------------------------------------------------
namespace hb {
namespace {

constexpr int kStaticPartials = 1024;
constexpr uint64_t kStaticScratchBytes = 64 + sizeof(double) * kStaticPartials;  // 8256 bytes
static_assert(kStaticPartials <= kMaxPartials, "the kernel indexes partials by CTA");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` names a host-side shadow of the symbol, not device memory.  The
// device address comes from cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_address(void **address) {
  constexpr int kMaxDevices = 64;
  static void *cached[kMaxDevices] = {};
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return static_cast<int>(error);
  if (device < 0 || device >= kMaxDevices) return HYLE_B200_NOT_SUPPORTED;
  if (cached[device] == nullptr) {
    void *pointer = nullptr;
    error = cudaGetSymbolAddress(&pointer, g_static_scratch);
    if (error != cudaSuccess) return static_cast<int>(error);
    if (pointer == nullptr) return HYLE_B200_NOT_SUPPORTED;
    cached[device] = pointer;  // benign race: every thread stores the same address
  }
  *address = cached[device];
  return HYLE_B200_OK;
}

}  // namespace
}  // namespace hb

extern "C" int hyle_b200_q8_0_roundtrip_bf16_static(hyle_b200_stream_t stream, const void *in,
                                                    uint64_t count, void *blocks_out,
                                                    void *decoded_bf16, double *sum_squares_out,
                                                    uint32_t *status_word) {
  if (count > HYLE_B200_STATIC_MAX_VALUES) return HYLE_B200_STATIC_SCRATCH_EXCEEDED;
  if (in == nullptr && count != 0) return HYLE_B200_INVALID_VALUE;
  if (blocks_out == nullptr || decoded_bf16 == nullptr || sum_squares_out == nullptr ||
      count % 32 != 0 || !aligned_to(blocks_out, 2))
    return HYLE_B200_INVALID_VALUE;
  if (!aligned_to(in, 16) || !aligned_to(decoded_bf16, 16)) return HYLE_B200_NOT_SUPPORTED;
  void *scratch = nullptr;
  const int status = static_scratch_address(&scratch);
  if (status != HYLE_B200_OK) return status;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  // The ticket counter must start at zero whatever an earlier call (or an aborted one) left.
  const cudaError_t cleared = cudaMemsetAsync(scratch, 0, 64, s);
  if (cleared != cudaSuccess) return static_cast<int>(cleared);
  const uint64_t blocks = count / 32;
  const uint64_t tiles = (blocks + kTileBlocks - 1) / kTileBlocks;
  const unsigned grid = clamp_grid(tiles, min(static_cast<uint64_t>(kStaticPartials), static_cast<uint64_t>(sm_count()) * 6));
  return launch(q8_0_kernel<HYLE_B200_BF16, true, true, true>, dim3(grid), dim3(kThreads), 0, s, 
      in, blocks, static_cast<unsigned char *>(blocks_out), static_cast<unsigned short *>(decoded_bf16),
      sum_squares_out, status_word, scratch, aligned_to(blocks_out, 16), Exchange{});
}

// Pieces shared by the decode kernels of aten::_weight_int8pack_mm (qmm8.cu: one product per launch; qmm8_chain.cu: a list
// of products per launch): the shared-memory stage layout, the exact int8 -> 16-bit float widening, the split of the
// (tile, k chunk) units into per-CTA ranges, and the constants of the arrival counters of sharded products.
#pragma once

#include <cuda.h>

#include <cstdint>

#include "../core/common.h"
#include "numerics.cuh"
#include "ptx.cuh"

namespace tvb {
namespace {

constexpr int kChunkK = 128;  // k values (= bytes of a weight row) per pipeline stage
constexpr size_t kCounterBytes = 65536;                                   // scratch: tile counters first
constexpr int kMaxTiles = static_cast<int>(kCounterBytes / sizeof(int)) - 1;  // (the last int counts finished CTAs)

template <int NT, int RW, int NWARPS>
struct SkinnyCfg {
  static constexpr int kRowsPerTile = NWARPS * RW * 16;
  static constexpr int kTokens = NT * 8;
  static constexpr int kWeightBytes = kRowsPerTile * kChunkK;   // one TMA box
  static constexpr int kTokenBoxBytes = kTokens * 128;          // 64 k of 16-bit values per row: two boxes per stage
  static constexpr int kStageBytes = kWeightBytes + 2 * kTokenBoxBytes;
  static constexpr int kStages = (224 * 1024 - kTokens * kRowsPerTile * 2) / kStageBytes < 8 ? (224 * 1024 - kTokens * kRowsPerTile * 2) / kStageBytes : 8;
  static constexpr int kThreads = (NWARPS + 2) * 32;  // consumers, the producer warp, the agent warp
  static constexpr int kOutTileBytes = kTokens * kRowsPerTile * 2;  // one tile's outputs, staged for coalesced stores
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */ + kOutTileBytes;
  static constexpr int kPartialFloats = NWARPS * RW * NT * 32 * 4;  // one CTA's accumulators
};

// int8 x 4 (one 32-bit word, k ascending) -> two packed pairs of 16-bit floats, exactly.
// bf16: the low 7 bits ride a 2^7 exponent (0x4300 | l = 128 + l); the same exponent with
// the sign bit as its top mantissa bit is 128 or 256; their difference is the int8 value.
// f16: 0x6400 | (x + 128) = 1024 + 128 + x; subtract 1152.
template <int DT>
__device__ __forceinline__ void widen_int8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  if (DT == TVB_BF16) {
    uint32_t l = w & 0x7f7f7f7fu, s = w & 0x80808080u;
    lo = ptx::sub_bf16x2(ptx::prmt(l, 0x43434343u, 0x4140u), ptx::prmt(s, 0x43434343u, 0x4140u));
    hi = ptx::sub_bf16x2(ptx::prmt(l, 0x43434343u, 0x4342u), ptx::prmt(s, 0x43434343u, 0x4342u));
  } else {
    uint32_t u = w ^ 0x80808080u;
    lo = ptx::sub_f16x2(ptx::prmt(u, 0x64646464u, 0x4140u), 0x64806480u);
    hi = ptx::sub_f16x2(ptx::prmt(u, 0x64646464u, 0x4342u), 0x64806480u);
  }
}

template <int DT>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  if (DT == TVB_BF16) ptx::mma_bf16_16816(d, a0, a1, a2, a3, b0, b1);
  else ptx::mma_f16_16816(d, a0, a1, a2, a3, b0, b1);
}

constexpr int kMaxRanks = 8;

// Arrival counters of sharded products (and of the products of a chain). Every rank owns kArriveSlots x kMaxRanks
// counters. Product number q of a channel (counted from zero, the same on every rank) is reported in slot q % 4: each CTA of
// rank s, once its columns are stored on every rank, adds its share to counter [q % 4][s] of every rank; the shares of one
// rank and product add up to kArriveWeight whatever the grid. So product q has arrived from rank s when counter [q % 4][s]
// has reached (q / 4 + 1) * kArriveWeight. Slots keep products that may be in flight together apart: a product waits at
// least for all products more than three before it, so a counter never holds shares of two unfinished products at once.
constexpr uint32_t kArriveWeight = 1024;
constexpr int kArriveSlots = 4;
constexpr int kArriveWords = kArriveSlots * kMaxRanks;

__device__ __forceinline__ uint32_t arrive_share() {
  return (blockIdx.x + 1) * kArriveWeight / gridDim.x - blockIdx.x * kArriveWeight / gridDim.x;
}

// Adds `share` for product q to this rank's counters on every rank. The caller's earlier stores must be ordered before the
// call by a fence of the calling thread: system scope, or GPU scope when there is one rank.
__device__ __forceinline__ void arrive_publish(uint32_t* const* flags, int nranks, int rank, uint32_t q, uint32_t share) {
  const int index = static_cast<int>(q & 3u) * kMaxRanks + rank;
  if (nranks == 1) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(flags[0] + index), "r"(share) : "memory");
    return;
  }
  for (int r = 0; r < nranks; r++)
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(flags[r] + index), "r"(share) : "memory");
}

// The product that slot `slot` must show for "all products up to number `upto` have arrived" (-1: none to show: those further
// back are implied), and the counter value that shows it.
__device__ __forceinline__ long long arrive_slot_product(long long upto, int slot) {
  if (upto < 0) return -1;
  return upto - ((upto - slot) & 3);
}
__device__ __forceinline__ uint32_t arrive_target(long long q) { return (static_cast<uint32_t>(q >> 2) + 1u) * kArriveWeight; }

// One thread's check that all products up to number `upto` have arrived in `mine` (this rank's counters) from all ranks.
// On success the thread has acquired what the arriving CTAs released. With one rank everything stays at GPU scope
// (system-scope loads and fences are several times slower while HBM is busy).
__device__ __forceinline__ bool arrivals_complete(const uint32_t* mine, int nranks, long long upto) {
  bool all = true;
#pragma unroll
  for (int slot = 0; slot < kArriveSlots; slot++) {
    const long long q = arrive_slot_product(upto, slot);
    if (q < 0) continue;
    const uint32_t target = arrive_target(q);
    if (nranks == 1) {
      uint32_t v;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + slot * kMaxRanks) : "memory");
      all = all && static_cast<int32_t>(v - target) >= 0;
      continue;
    }
    uint32_t v[kMaxRanks];
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(mine + slot * kMaxRanks) : "memory");
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(mine + slot * kMaxRanks + 4) : "memory");
#pragma unroll
    for (int r = 0; r < kMaxRanks; r++)
      if (r < nranks) all = all && static_cast<int32_t>(v[r] - target) >= 0;
  }
  if (all) {
    if (nranks == 1) __threadfence();
    else __threadfence_system();
  }
  return all;
}

// The same check by a whole warp, one counter per lane.
__device__ __forceinline__ bool arrivals_complete_warp(const uint32_t* mine, int nranks, long long upto) {
  const int lane = threadIdx.x & 31, slot = lane / kMaxRanks, r = lane % kMaxRanks;
  const long long q = arrive_slot_product(upto, slot);
  bool ok = true;
  if (q >= 0 && r < nranks) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + lane) : "memory");
    ok = static_cast<int32_t>(v - arrive_target(q)) >= 0;
  }
  return __all_sync(0xffffffffu, ok);
}

template <int DT>
__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
  return DT == TVB_BF16 ? __uint_as_float(static_cast<uint32_t>(h) << 16) : __half2float(__ushort_as_half(h));
}
template <int DT>
__device__ __forceinline__ uint16_t float_to_half_bits(float v) {
  return DT == TVB_BF16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
}

// First unit of CTA c when `units` units are cut into `grid` contiguous ranges. (32-bit arithmetic whenever the products
// fit, which the kernel checks once: 64-bit division is a long instruction sequence, and these run between segments.)
__device__ __forceinline__ long long range_start(long long c, long long units, long long grid, bool small) {
  if (small) return static_cast<unsigned>(c) * static_cast<unsigned>(units) / static_cast<unsigned>(grid);
  return c * units / grid;
}
// The CTA whose range holds unit x.
__device__ __forceinline__ int range_owner(long long x, long long units, long long grid, bool small) {
  if (small)
    return static_cast<int>((static_cast<unsigned>(x + 1) * static_cast<unsigned>(grid) + static_cast<unsigned>(units) - 1u) /
                            static_cast<unsigned>(units)) - 1;
  return static_cast<int>(((x + 1) * grid + units - 1) / units - 1);
}

// The tile that holds unit u.
__device__ __forceinline__ int unit_tile(long long u, int chunks, bool small) {
  return small ? static_cast<int>(static_cast<unsigned>(u) / static_cast<unsigned>(chunks)) : static_cast<int>(u / chunks);
}

}  // namespace
}  // namespace tvb

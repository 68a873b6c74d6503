// A list of int8 weight-only decode products in one launch (tvb_qmm8_chain_*): the decode kernel of qmm8.cu made
// persistent over a whole sequence of products, such as the Linears of a decoder stack for one token step
// (aten::_weight_int8pack_mm after aten::_weight_int8pack_mm; the reference issues one dispatch per product,
// crates/pyvk/csrc/quant.cpp:86-117, and has no counterpart to this).
//
// Why: a decode product is a few microseconds of weight streaming; launched one by one, every product pays for the
// start of its CTAs, the fill of its shared-memory ring and the completion of the tiles that several CTAs share, during
// which HBM idles (about 8 us per launch, more than the streaming time of a sharded product). Here one CTA per SM walks
// the list:
//  * the producer lane keeps two cursors. Weights have no dependencies, so their TMA copies run ahead through the ring
//    across product boundaries, as far as the ring has room; the activation slices of a stage follow as soon as the
//    product they belong to may start. While the consumers finish a product's shared tiles, the ring already fills
//    with the next product's weights.
//  * a product may start when all earlier products of the list (all but its latest `independent` ones) are complete on
//    every rank: completion is counted per CTA in the same arrival counters that tvb_qmm8_gather uses (one counter per
//    source rank, 1024 per product and rank), so the same kernel runs on one GPU (its own counters) and sharded over
//    the GPUs of a node (every CTA stores its columns into every rank's buffer and adds its share to every rank's
//    counter; plain stores and reductions to peer memory, no TMA multicast).
//  * CTAs wait for one another here (a product needs the outputs of the one before), so the launch is cooperative: all
//    CTAs are resident together. Every wait is bounded and gives up through the status word.
// Arithmetic, tile shapes, the split of (tile, k chunk) units over the CTAs and the fixed order of additions are those of
// qmm8_skinny_kernel: a chain's outputs are bit for bit those of the products launched one by one.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "numerics.cuh"
#include "ptx.cuh"
#include "qmm8_skinny.cuh"

namespace tvb {

extern std::atomic<long long> g_wait_limit_cycles;  // (qmm8.cu; tvb_set_wait_limit_ms)

namespace {

constexpr int kChainSets = 4;           // scratch sets used in turn: product i of a launch uses set i % 4
constexpr int kChainTileSlots = 8192;   // tile counters per set

struct ChainItemDev {
  const void* scales;
  void* c[kMaxRanks];   // every rank's output buffer [m, c_ld] (entry 0 only without sharding)
  int m, m0, n, k;      // rows of A, first row of this pass, this rank's output columns, k
  int tiles, chunks;
  int c_ld, c_col0;
  uint32_t independent;  // how many of the latest earlier products this one need not wait for (at most kChainSets - 1)
  uint32_t pad[5];
};
static_assert(sizeof(ChainItemDev) == 128, "ChainItemDev layout");

struct ChainParams {
  const CUtensorMap* maps;    // [count][2]: weights, activations
  const ChainItemDev* items;  // [count]
  int count;
  uint32_t* flags[kMaxRanks];  // every rank's arrival counters (entry `rank` of each is this GPU's to add to)
  int nranks, rank;
  uint32_t* seq;      // device counter of the products this rank has completed on the channel
  int* done;          // counter of finished CTAs (zero between launches)
  int* counters;      // [kChainSets][kChainTileSlots], zero between launches
  float* partials;    // [kChainSets][grid][2][kPartialFloats]
  int* status;
  long long wait_limit;
  int wait_at_end;    // CTA 0 ends only when every rank's columns of the last product have arrived here
};

// This CTA's range of product `d` (empty for CTAs beyond the product's units).
struct ItemRange {
  long long units, g, u0, u1;
  bool small, active;
};

__device__ __forceinline__ ItemRange item_range(const ChainItemDev& d) {
  ItemRange r;
  r.units = static_cast<long long>(d.tiles) * d.chunks;
  r.g = r.units < static_cast<long long>(gridDim.x) ? r.units : static_cast<long long>(gridDim.x);
  r.small = (r.units + 1) * (r.g + 1) < (1ll << 31);
  r.active = static_cast<long long>(blockIdx.x) < r.g;
  r.u0 = r.active ? range_start(blockIdx.x, r.units, r.g, r.small) : 0;
  r.u1 = r.active ? range_start(blockIdx.x + 1, r.units, r.g, r.small) : 0;
  return r;
}

// Adds this CTA's share of the completion of product number q to this rank's counters on every rank. Called by one thread
// once everything the CTA stores for the product is ordered before it (the CTA's barriers, then this thread's fence).
__device__ __forceinline__ void chain_publish(const ChainParams& p, uint32_t q) {
  if (p.nranks == 1) __threadfence();
  else __threadfence_system();
  arrive_publish(p.flags, p.nranks, p.rank, q, arrive_share());
}

struct ChainCursor {
  int item;
  long long u, u1, it;
  int tile, chunk, chunks, m0;
};

// Moves the cursor to the first product from c.item on in which this CTA has units.
__device__ __forceinline__ void chain_enter(const ChainParams& p, ChainCursor& c) {
  while (c.item < p.count) {
    const ChainItemDev& d = p.items[c.item];
    const ItemRange r = item_range(d);
    if (r.active && r.u0 < r.u1) {
      c.u = r.u0;
      c.u1 = r.u1;
      c.chunks = d.chunks;
      c.m0 = d.m0;
      c.tile = unit_tile(r.u0, d.chunks, r.small);
      c.chunk = static_cast<int>(r.u0 - static_cast<long long>(c.tile) * d.chunks);
      return;
    }
    c.item++;
  }
}

__device__ __forceinline__ void chain_advance(const ChainParams& p, ChainCursor& c) {
  c.it++;
  c.u++;
  if (++c.chunk == c.chunks) {
    c.chunk = 0;
    c.tile++;
  }
  if (c.u == c.u1) {
    c.item++;
    chain_enter(p, c);
  }
}

template <int DT, int NT, int RW, int NWARPS>
__global__ void __launch_bounds__((NWARPS + 2) * 32, 1) qmm8_chain_kernel(const ChainParams p) {
  using Cfg = SkinnyCfg<NT, RW, NWARPS>;
  extern __shared__ uint8_t smem_raw[];
  // stages need 1024-byte alignment for the 128-byte swizzle pattern
  uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + Cfg::kStages * Cfg::kStageBytes);
  const uint32_t full0 = ptx::smem_u32(bars), empty0 = full0 + 8 * Cfg::kStages;
  const uint32_t agent_bar = empty0 + 8 * Cfg::kStages;  // the consumers have stored the partial sums of a segment they leave behind
  const uint32_t item_bar = agent_bar + 8;               // the consumers have stored everything of a product
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * Cfg::kStages + 2);
  int* last_flag = const_cast<int*>(abort_flag) + 1;  // two slots
  int* early_flag = last_flag + 2;  // set when every other contributor of the segment's tile was seen to have arrived
  volatile int* agent_passed = early_flag + 1;  // how many of the consumers' hand-overs of a tile the agent warp has taken up
  volatile int* agent_items = early_flag + 2;   // how many of the consumers' end-of-product reports it has taken up
  static_assert((2 * Cfg::kStages + 2) * 8 + (1 + 2 + 1 + 2) * 4 <= 256, "barrier area too small");
  uint16_t* out_tile = reinterpret_cast<uint16_t*>(base_ptr + Cfg::kStages * Cfg::kStageBytes + 256);  // [tokens][rows of a tile]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, NWARPS);
    }
    ptx::mbar_init(agent_bar, NWARPS);
    ptx::mbar_init(item_bar, NWARPS);
    *abort_flag = 0;
    last_flag[0] = last_flag[1] = 0;
    *early_flag = 0;
    *agent_passed = 0;
    *agent_items = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  // products completed on the channel before this launch (the previous launch of the stream has ended: the count is final)
  const uint32_t seq0 = *reinterpret_cast<const volatile uint32_t*>(p.seq);
  const size_t partial_set = static_cast<size_t>(gridDim.x) * 2 * Cfg::kPartialFloats;

  if (warp == NWARPS) {
    // ---------------- producer: one lane issues every TMA copy
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();  // weights are read once
      const uint64_t keep_policy = ptx::policy_evict_last();     // every CTA re-reads A
      ChainCursor w{}, a{};
      chain_enter(p, w);
      chain_enter(p, a);
      int ready_item = -1;  // the highest product known to be allowed to start
      long long idle_since = -1;
      bool ok = true;
      while (a.item < p.count) {
        bool progress = false;
        // activations: only once their product may start
        if (a.it < w.it) {
          if (a.item > ready_item) {
            const long long upto = static_cast<long long>(seq0) + a.item - 1 - static_cast<long long>(p.items[a.item].independent);
            if (arrivals_complete(p.flags[p.rank], p.nranks, upto)) {
              ready_item = a.item;
              asm volatile("fence.proxy.async.global;" ::: "memory");  // (the copies below read what other CTAs and ranks stored)
            }
          }
          while (a.item <= ready_item && a.it < w.it && a.item < p.count) {
            const int s = static_cast<int>(a.it % Cfg::kStages);
            const uint32_t dst = base + s * Cfg::kStageBytes + Cfg::kWeightBytes;
            const CUtensorMap* map_a = p.maps + 2 * a.item + 1;
            ptx::tma_load_2d_hint(dst, map_a, a.chunk * kChunkK, a.m0, full0 + 8 * s, keep_policy);
            ptx::tma_load_2d_hint(dst + Cfg::kTokenBoxBytes, map_a, a.chunk * kChunkK + 64, a.m0, full0 + 8 * s, keep_policy);
            chain_advance(p, a);
            progress = true;
          }
        }
        // weights: as far ahead as the ring has room, whatever product they belong to
        while (w.item < p.count) {
          const int s = static_cast<int>(w.it % Cfg::kStages);
          const uint32_t ph = static_cast<uint32_t>((w.it / Cfg::kStages) & 1);
          if (!ptx::mbar_test_wait(empty0 + 8 * s, ph ^ 1u)) break;  // (a test, not a wait: the activations below must not be held up)
          ptx::mbar_expect_tx(full0 + 8 * s, Cfg::kStageBytes);
          ptx::tma_load_2d_hint(base + s * Cfg::kStageBytes, p.maps + 2 * w.item,
                                w.chunk * kChunkK, w.tile * Cfg::kRowsPerTile, full0 + 8 * s, stream_policy);
          chain_advance(p, w);
          progress = true;
        }
        if (progress) {
          idle_since = -1;
        } else {
          // Nothing to issue right now. Sleep on the ring slot the next weights need (the usual thing to wait for; the
          // thread is suspended, so it does not compete with the consumers for the shared-memory pipe) for at most half a
          // microsecond, then look at both cursors again: activations may be waiting for other CTAs or ranks.
          if (w.item < p.count)
            ptx::mbar_try_wait_for(empty0 + 8 * static_cast<int>(w.it % Cfg::kStages), static_cast<uint32_t>((w.it / Cfg::kStages) & 1) ^ 1u,
                                   a.it < w.it ? 100 : 500);
          else
            __nanosleep(200);
          if (*abort_flag != 0) { ok = false; break; }
          const long long now = clock64();
          if (idle_since < 0) idle_since = now;
          else if (now - idle_since > p.wait_limit) {
            *abort_flag = 1;
            atomicExch(p.status, 5);
            ok = false;
            break;
          }
        }
      }
      // Leave no copy in flight behind. A stage whose weights were requested but whose activations were not (the kernel
      // is giving up) gets them now, so that its barrier completes; then every stage that was armed is waited for.
      while (a.it < w.it && a.item < p.count) {
        const int s = static_cast<int>(a.it % Cfg::kStages);
        const uint32_t dst = base + s * Cfg::kStageBytes + Cfg::kWeightBytes;
        const CUtensorMap* map_a = p.maps + 2 * a.item + 1;
        ptx::tma_load_2d_hint(dst, map_a, a.chunk * kChunkK, a.m0, full0 + 8 * s, keep_policy);
        ptx::tma_load_2d_hint(dst + Cfg::kTokenBoxBytes, map_a, a.chunk * kChunkK + 64, a.m0, full0 + 8 * s, keep_policy);
        chain_advance(p, a);
      }
      const long long first = w.it > Cfg::kStages ? w.it - Cfg::kStages : 0;
      for (long long j = first; j < w.it; j++) {
        volatile int never = 0;
        ptx::mbar_wait(full0 + 8 * static_cast<int>(j % Cfg::kStages), static_cast<uint32_t>((j / Cfg::kStages) & 1), &never);
      }
      if (ok && p.wait_at_end != 0 && blockIdx.x == 0) {
        // the launch ends only when the last product's columns from every rank are in this rank's buffers
        const long long upto = static_cast<long long>(seq0) + p.count - 1;
        const long long start = clock64();
        for (int spins = 0; !arrivals_complete(p.flags[p.rank], p.nranks, upto); spins++) {
          if ((spins & 15) == 15 && (*reinterpret_cast<volatile int*>(p.status) != 0 || clock64() - start > p.wait_limit)) {
            atomicExch(p.status, 5);
            break;
          }
        }
      }
    }
    return;
  }

  if (warp == NWARPS + 1) {
    // ---------------- agent: what would otherwise hold the consumers up between two products
    // (Completing tiles here as a rule, so that the consumers never stop for one, was measured: one warp doing eight warps'
    // additions is several times too slow.)
    // (1) A range that starts inside a tile and goes on beyond it leaves that tile's partial sums in scratch and moves on
    // at once; this warp counts the arrival in the consumers' stead. Should it turn out to be the tile's last arrival
    // (the other contributors normally come much later), this warp alone completes the tile. (2) When the consumers have
    // stored everything of a product, this warp orders those stores (a fence that takes microseconds while HBM is busy)
    // and adds the CTA's share to the arrival counters. (3) For a product in which the CTA has no units it reports as
    // soon as the product may start: a counter must never hold shares of products four apart.
    int uses = 0, reports = 0;
    for (int item = 0; item < p.count; item++) {
      const ChainItemDev& d = p.items[item];
      const ItemRange rg_ = item_range(d);
      if (!rg_.active) {
        bool go = true;
        if (lane == 0) {
          const long long upto = static_cast<long long>(seq0) + item - 1 - static_cast<long long>(d.independent);
          const long long start = clock64();
          for (int spins = 0; !arrivals_complete(p.flags[p.rank], p.nranks, upto); spins++) {
            if ((spins & 15) == 15 && (*abort_flag != 0 || clock64() - start > p.wait_limit)) {
              if (*abort_flag == 0) atomicExch(p.status, 5);
              *abort_flag = 1;
              go = false;
              break;
            }
            __nanosleep(100);
          }
          if (go) chain_publish(p, seq0 + static_cast<uint32_t>(item));
        }
        if (!__shfl_sync(0xffffffffu, go, 0)) break;
        continue;
      }
      const bool small = rg_.small;
      const long long units = rg_.units, grid = rg_.g, u0 = rg_.u0, u1 = rg_.u1;
      const int tile = unit_tile(u0, d.chunks, small), c0 = static_cast<int>(u0 - static_cast<long long>(tile) * d.chunks);
      const int c1 = static_cast<int>(min(static_cast<long long>(d.chunks), c0 + (u1 - u0)));
      const bool left_behind = !(c0 == 0 && c1 == d.chunks) && u0 + (c1 - c0) < u1;
      // Counts this CTA's arrival at `tile` and, should it be the tile's last, completes the tile.
      auto see_to_tile = [&](int tile) {
        int* counters = p.counters + (item % kChainSets) * kChainTileSlots;
        const float* partials = p.partials + (item % kChainSets) * partial_set;
        const long long tile_first_unit = static_cast<long long>(tile) * d.chunks;
        const int cta_first = range_owner(tile_first_unit, units, grid, small);
        const int cta_last = range_owner(tile_first_unit + d.chunks - 1, units, grid, small);
        int last = 0;
        if (lane == 0) {
          __threadfence();  // (cumulative over the consumers' stores, which the barrier ordered before this)
          last = atomicAdd(&counters[tile], 1) == cta_last - cta_first;
          if (last) atomicExch(&counters[tile], 0);
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          const int g = lane >> 2, t = lane & 3, rg = (g >> 1) | ((g & 1) << 2);
          for (int w = 0; w < NWARPS; w++)  // this warp plays every consumer warp's part in turn
#pragma unroll
            for (int rb = 0; rb < RW; rb++)
#pragma unroll
              for (int nt = 0; nt < NT; nt++) {
                float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int cta = cta_last; cta >= cta_first; cta--) {  // the one fixed order of additions
                  const bool cta_first_segment = unit_tile(range_start(cta, units, grid, small), d.chunks, small) == tile;
                  const float4* theirs = reinterpret_cast<const float4*>(
                      partials + (static_cast<size_t>(cta) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
                  const float4 v = __ldcg(&theirs[((w * RW + rb) * NT + nt) * 32 + lane]);
                  sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int half = 0; half < 2; half++) {
                  const int col = tile * Cfg::kRowsPerTile + (w * RW + rb) * 16 + rg + 8 * half;
                  if (col >= d.n) continue;
                  const float scale = load_float<DT>(d.scales, col);
#pragma unroll
                  for (int i = 0; i < 2; i++) {
                    const int token = d.m0 + nt * 8 + 2 * t + i;
                    if (token >= d.m) continue;
                    const uint16_t bits = float_to_half_bits<DT>(vals[2 * half + i] * scale);
                    const int64_t off = static_cast<int64_t>(token) * d.c_ld + d.c_col0 + col;
                    for (int r = 0; r < p.nranks; r++) static_cast<uint16_t*>(d.c[r])[off] = bits;
                  }
                }
              }
        }
      };
      if (left_behind) {
        if (!ptx::mbar_wait(agent_bar, static_cast<uint32_t>(uses & 1), abort_flag)) break;
        uses++;
        if (lane == 0) *agent_passed = uses;  // (the consumers may now complete the barrier's next phase)
        see_to_tile(tile);
      }
      // the consumers' stores of this product are out (the barrier's release and acquire order them before the fence below)
      if (!ptx::mbar_wait(item_bar, static_cast<uint32_t>(reports & 1), abort_flag)) break;
      reports++;
      __syncwarp();
      if (lane == 0) {
        *agent_items = reports;
        chain_publish(p, seq0 + static_cast<uint32_t>(item));
      }
    }
    return;
  }

  // ---------------- consumers
  const int g = lane >> 2, t = lane & 3;
  // MMA row g of a 16-row block reads weight row rg (and rg + 8): a permutation chosen so that the two values of g in a
  // quarter-warp differ in bit 2 of the row, which sends their 16-byte chunks to disjoint banks under the 128-byte swizzle.
  const int rg = (g >> 1) | ((g & 1) << 2);
  float acc[RW][NT][4];
  long long it = 0;
  bool ok = true;
  int segment = 0;
  int handovers = 0;  // tiles left to the agent warp so far
  int reported = 0;   // products whose end was reported to the agent warp so far
  for (int item = 0; item < p.count && ok; item++) {
    const ChainItemDev& d = p.items[item];
    const ItemRange range = item_range(d);
    if (!range.active) continue;  // (the agent warp reports for the CTA)
    const bool small = range.small;
    const long long units = range.units, grid = range.g, u0 = range.u0, u1 = range.u1;
    const int chunks = d.chunks, n = d.n, m = d.m, m0 = d.m0;
    int* counters = p.counters + (item % kChainSets) * kChainTileSlots;
    float* partials = p.partials + (item % kChainSets) * partial_set;
    long long u = u0;
    while (u < u1 && ok) {
      const int tile = unit_tile(u, chunks, small), c0 = static_cast<int>(u - static_cast<long long>(tile) * chunks);
      const int c1 = static_cast<int>(min(static_cast<long long>(chunks), c0 + (u1 - u)));
      const bool first_segment = (u == u0);
      const bool whole_tile = c0 == 0 && c1 == chunks;
      const bool hand_over = !whole_tile && u + (c1 - c0) < u1;  // (a first segment with more of the range to follow)
      // The ranges that share this tile (consecutive CTAs). Their partial sums are always added in descending CTA order.
      const long long tile_first_unit = static_cast<long long>(tile) * chunks;
      const int cta_first = whole_tile ? static_cast<int>(blockIdx.x) : range_owner(tile_first_unit, units, grid, small);
      const int cta_last = whole_tile ? static_cast<int>(blockIdx.x) : range_owner(tile_first_unit + chunks - 1, units, grid, small);
      // A CTA that holds the tile's first k (the usual case for the last tile of its range) is added last. If, shortly
      // before its segment ends, it sees that all the others have already arrived, it is certain to finish the tile: it
      // then fetches their sums while its last chunks are in flight and skips the exchange through scratch altogether.
      const bool may_be_early = !whole_tile && !hand_over && cta_first == static_cast<int>(blockIdx.x) && c1 - c0 >= 3;
      bool early = false;
      int peeked = 0;
      float pre[RW][NT][4];
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) acc[rb][nt][i] = pre[rb][nt][i] = 0.0f;

      // This thread's columns' scales, asked for now: each is read once per product, so the load goes to DRAM, and at the
      // end of the segment (where the finished sums need it) it would wait in line behind the other SMs' weight traffic.
      float scale_pre[RW][2];
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int col = tile * Cfg::kRowsPerTile + (warp * RW + rb) * 16 + rg + 8 * half;
          scale_pre[rb][half] = col < n ? load_float<DT>(d.scales, col) : 0.0f;
        }

      for (int chunk = c0; chunk < c1; chunk++, it++) {
        const int s = static_cast<int>(it % Cfg::kStages);
        const uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
        ok = ptx::mbar_wait(full0 + 8 * s, ph, abort_flag);
        if (!ok) break;
        if (may_be_early) {
          if (chunk == c1 - 3) {
            if (threadIdx.x == 0) asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(peeked) : "l"(counters + tile) : "memory");
          } else if (chunk == c1 - 2) {
            if (threadIdx.x == 0) *early_flag = peeked == cta_last - cta_first;
          } else if (chunk == c1 - 1) {
            ptx::named_bar_sync(1, NWARPS * 32);
            early = *early_flag != 0;
            if (early) {
              // the highest contributor's sums: requested now, first needed after this segment's last chunk
              const bool cta_first_segment = unit_tile(range_start(cta_last, units, grid, small), chunks, small) == tile;
              const float4* theirs = reinterpret_cast<const float4*>(
                  partials + (static_cast<size_t>(cta_last) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
#pragma unroll
              for (int rb = 0; rb < RW; rb++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                  float4 v = __ldcg(&theirs[((warp * RW + rb) * NT + nt) * 32 + lane]);
                  pre[rb][nt][0] = v.x; pre[rb][nt][1] = v.y; pre[rb][nt][2] = v.z; pre[rb][nt][3] = v.w;
                }
            }
          }
        }
        const uint32_t wbase = base + s * Cfg::kStageBytes;
        const uint32_t tbase = wbase + Cfg::kWeightBytes;
#pragma unroll
        for (int h = 0; h < 2; h++) {
          // this lane's 16 k of every token row: 32 bytes = swizzled 16-byte chunks 2t and 2t+1 of row nt*8+g
          uint32_t tok[NT][8];
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            uint32_t row = tbase + h * Cfg::kTokenBoxBytes + (nt * 8 + g) * 128;
            uint4 x = ptx::lds128(row + (((2 * t) ^ g) << 4));
            uint4 y = ptx::lds128(row + (((2 * t + 1) ^ g) << 4));
            tok[nt][0] = x.x; tok[nt][1] = x.y; tok[nt][2] = x.z; tok[nt][3] = x.w;
            tok[nt][4] = y.x; tok[nt][5] = y.y; tok[nt][6] = y.z; tok[nt][7] = y.w;
          }
#pragma unroll
          for (int rb = 0; rb < RW; rb++) {
            // rows rg and rg+8 of this warp's 16-row block; both have (row & 7) == rg
            uint32_t r0 = wbase + ((warp * RW + rb) * 16 + rg) * 128 + (((4 * h + t) ^ rg) << 4);
            uint4 w0 = ptx::lds128(r0);
            uint4 w1 = ptx::lds128(r0 + 8 * 128);
            const uint32_t w0v[4] = {w0.x, w0.y, w0.z, w0.w};
            const uint32_t w1v[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              uint32_t a0, a1, a2, a3;
              widen_int8x4<DT>(w0v[j], a0, a2);
              widen_int8x4<DT>(w1v[j], a1, a3);
#pragma unroll
              for (int nt = 0; nt < NT; nt++) mma_16816<DT>(acc[rb][nt], a0, a1, a2, a3, tok[nt][2 * j], tok[nt][2 * j + 1]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(empty0 + 8 * s);
      }
      if (!ok) break;

      // ---- the segment's sums are complete: finish the tile, alone or with the other CTAs that share it
      bool finish = true;
      if (early) {
        // every other contributor was counted before this CTA looked: nobody else will touch the counter again
        if (threadIdx.x == 0) atomicExch(&counters[tile], 0);
        // the same additions in the same order as the general path below: from zero, descending, this CTA's sums last
#pragma unroll
        for (int rb = 0; rb < RW; rb++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) pre[rb][nt][i] = 0.0f + pre[rb][nt][i];
        for (int cta = cta_last - 1; cta > cta_first; cta--) {
          const bool cta_first_segment = unit_tile(range_start(cta, units, grid, small), chunks, small) == tile;
          const float4* theirs = reinterpret_cast<const float4*>(
              partials + (static_cast<size_t>(cta) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
#pragma unroll
          for (int rb = 0; rb < RW; rb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              float4 v = __ldcg(&theirs[((warp * RW + rb) * NT + nt) * 32 + lane]);
              pre[rb][nt][0] += v.x; pre[rb][nt][1] += v.y; pre[rb][nt][2] += v.z; pre[rb][nt][3] += v.w;
            }
        }
#pragma unroll
        for (int rb = 0; rb < RW; rb++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[rb][nt][i] = pre[rb][nt][i] + acc[rb][nt][i];
      } else if (!whole_tile) {
        float4* mine = reinterpret_cast<float4*>(partials + (static_cast<size_t>(blockIdx.x) * 2 + (first_segment ? 0 : 1)) *
                                                                Cfg::kPartialFloats);
#pragma unroll
        for (int rb = 0; rb < RW; rb++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
            __stcg(&mine[((warp * RW + rb) * NT + nt) * 32 + lane],
                   make_float4(acc[rb][nt][0], acc[rb][nt][1], acc[rb][nt][2], acc[rb][nt][3]));
        if (hand_over) {
          // More of the range follows: leave the tile to the agent warp (which counts this arrival) and go on at once.
          // (The agent must have seen the previous hand-over complete before this one may: a barrier tells two phases
          // apart, not three. It almost always has.)
          __syncwarp();
          if (lane == 0) {
            const long long start = clock64();
            while (*agent_passed < handovers) {
              if (*abort_flag != 0 || clock64() - start > p.wait_limit) {
                *abort_flag = 1;
                break;
              }
            }
            ptx::mbar_arrive(agent_bar);
          }
          handovers++;
          finish = false;

        } else {
          // All consumer threads have stored their partial sums once they pass the barrier; one thread then publishes
          // them: its gpu-scope fence is cumulative over what the barrier ordered before it.
          ptx::named_bar_sync(1, NWARPS * 32);
          int* flag = last_flag + (segment & 1);  // (alternating slots: no barrier needed before the next segment rewrites it)
          if (threadIdx.x == 0) {
            __threadfence();
            int arrived = atomicAdd(&counters[tile], 1);
            int last = arrived == cta_last - cta_first;
            if (last) atomicExch(&counters[tile], 0);  // zero again for the next product that uses this set
            *flag = last;
          }
          ptx::named_bar_sync(1, NWARPS * 32);
          finish = *flag != 0;
          segment++;
          if (finish) {
            __threadfence();
#pragma unroll
            for (int rb = 0; rb < RW; rb++)
#pragma unroll
              for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[rb][nt][i] = 0.0f;
            for (int cta = cta_last; cta >= cta_first; cta--) {  // fixed order: the sum does not depend on who came last
              const bool cta_first_segment = unit_tile(range_start(cta, units, grid, small), chunks, small) == tile;
              const float4* theirs = reinterpret_cast<const float4*>(
                  partials + (static_cast<size_t>(cta) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
#pragma unroll
              for (int rb = 0; rb < RW; rb++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                  float4 v = __ldcg(&theirs[((warp * RW + rb) * NT + nt) * 32 + lane]);
                  acc[rb][nt][0] += v.x; acc[rb][nt][1] += v.y; acc[rb][nt][2] += v.z; acc[rb][nt][3] += v.w;
                }
            }
          }
        }
      }
      if (finish) {
        // Scale, round once, and stage the tile's [tokens][columns] in shared memory, so that what goes to global
        // memory (this GPU's output and, with sharding, every peer's over NVLink) is 16-byte, fully coalesced stores.
#pragma unroll
        for (int rb = 0; rb < RW; rb++) {
          const int lrow0 = (warp * RW + rb) * 16 + rg;
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int lcol = lrow0 + 8 * half;  // column within the tile (weight row = output column)
            const float scale = scale_pre[rb][half];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
              for (int i = 0; i < 2; i++)
                out_tile[(nt * 8 + 2 * t + i) * Cfg::kRowsPerTile + lcol] = float_to_half_bits<DT>(acc[rb][nt][2 * half + i] * scale);
          }
        }
        ptx::named_bar_sync(1, NWARPS * 32);
        const int col_base = tile * Cfg::kRowsPerTile;
        const int c_ld = d.c_ld, c_col0 = d.c_col0;
        const bool vec = (c_ld % 8 == 0) && (c_col0 % 8 == 0);
        for (int v = threadIdx.x; v < Cfg::kTokens * (Cfg::kRowsPerTile / 8); v += NWARPS * 32) {
          const int tok = v / (Cfg::kRowsPerTile / 8), chunk = v % (Cfg::kRowsPerTile / 8);
          const int token = m0 + tok, col = col_base + chunk * 8;
          if (token >= m || col >= n) continue;
          const uint4 val = *reinterpret_cast<const uint4*>(out_tile + tok * Cfg::kRowsPerTile + chunk * 8);
          const int64_t off = static_cast<int64_t>(token) * c_ld + c_col0 + col;
          if (vec && col + 8 <= n) {
            for (int r = 0; r < p.nranks; r++) {
              uint16_t* dst = static_cast<uint16_t*>(d.c[r]) + off;
              if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                *reinterpret_cast<uint4*>(dst) = val;
              } else {
                const uint16_t* e = reinterpret_cast<const uint16_t*>(&val);
                for (int j = 0; j < 8; j++) dst[j] = e[j];
              }
            }
          } else {
            const uint16_t* e = reinterpret_cast<const uint16_t*>(&val);
            for (int r = 0; r < p.nranks; r++)
              for (int j = 0; j < 8 && col + j < n; j++) (static_cast<uint16_t*>(d.c[r]) + off)[j] = e[j];
          }
        }
        ptx::named_bar_sync(1, NWARPS * 32);  // (the staging tile is free again)
      }
      u += c1 - c0;
    }
    if (!ok) break;
    // Everything this warp stores for the product is out (and it has read all of A it ever will): tell the agent warp, which
    // reports for the CTA once all consumer warps have. (It must have taken up the previous product's report first: a
    // barrier tells two phases apart, not three. It almost always has.)
    __syncwarp();
    if (lane == 0) {
      const long long start = clock64();
      while (*agent_items < reported) {
        if (*abort_flag != 0 || clock64() - start > p.wait_limit) {
          *abort_flag = 1;
          break;
        }
      }
      ptx::mbar_arrive(item_bar);
    }
    reported++;
  }
  if (ok && threadIdx.x == 0) {
    // the last CTA to get here counts the products (the next launch of the stream reads the count after this one has ended)
    if (atomicAdd(p.done, 1) == static_cast<int>(gridDim.x) - 1) {
      atomicExch(p.done, 0);
      *reinterpret_cast<volatile uint32_t*>(p.seq) = seq0 + static_cast<uint32_t>(p.count);
    }
  }
}

// ------------------------------------------------------------------ host side

struct Chain {
  int device = 0, dtype = 0, nt = 1, rw = 1, count = 0, grid = 0;
  void* block = nullptr;  // one device allocation: tensor maps, product descriptors, scratch, the chain's own channel
  ChainParams params{};
};

template <int DT, int NT, int RW>
int chain_launch(const Chain& c, cudaStream_t stream) {
  using Cfg = SkinnyCfg<NT, RW, 8>;
  auto kernel = qmm8_chain_kernel<DT, NT, RW, 8>;
  {
    static std::mutex mutex;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> lock(mutex);
    if (!configured[c.device & 63]) {
      TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      int per_sm = 0;
      TVB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, Cfg::kThreads, Cfg::kSmemBytes));
      if (per_sm < 1) return fail("tvb_qmm8_chain_run: the kernel does not fit an SM of this device");
      configured[c.device & 63] = true;
    }
  }
  ChainParams p = c.params;
  p.wait_limit = g_wait_limit_cycles.load();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(c.grid);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // the CTAs wait for one another: all of them must be resident together
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TVB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return launched("qmm8_chain", dim3(c.grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

template <int DT>
int chain_launch_dt(const Chain& c, cudaStream_t stream) {
  if (c.nt == 1) return c.rw == 1 ? chain_launch<DT, 1, 1>(c, stream) : chain_launch<DT, 1, 2>(c, stream);
  return c.rw == 1 ? chain_launch<DT, 2, 1>(c, stream) : chain_launch<DT, 2, 2>(c, stream);
}

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" int tvb_qmm8_chain_create(int device, int dtype, const TvbChainItem* items, int count, uint32_t* const* flag_ranks,
                                     int world, int rank, uint32_t* seq_counter, int wait_at_end, void** chain_out) {
  TVB_REQUIRE(chain_out != nullptr && items != nullptr && count >= 1 && count <= 65536, "tvb_qmm8_chain_create: 1 to 65536 products");
  TVB_REQUIRE(dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8_chain_create: A must be float16 or bfloat16");
  TVB_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "tvb_qmm8_chain_create: 1 to 8 ranks");
  TVB_REQUIRE(world == 1 || (flag_ranks != nullptr && seq_counter != nullptr), "tvb_qmm8_chain_create: a sharded chain needs a channel");
  TVB_REQUIRE((flag_ranks == nullptr) == (seq_counter == nullptr), "tvb_qmm8_chain_create: counters and product count go together");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  const int grid = sm_count(device);
  TVB_REQUIRE(grid >= 1 && grid <= static_cast<int>(kArriveWeight), "tvb_qmm8_chain_create: unsupported SM count");

  // shapes: 16 rows of A per pass, every pass a product of its own; one tile shape and token count for the whole chain
  int nt = 1, rw = 2;
  int64_t passes_total = 0;
  for (int i = 0; i < count; i++) {
    const TvbChainItem& it = items[i];
    TVB_REQUIRE(it.m >= 1 && it.m <= 64 && it.n_local >= 1 && it.k >= kChunkK && it.k % kChunkK == 0 && it.k < (int64_t(1) << 31),
                "tvb_qmm8_chain_create: 1 <= m <= 64, k a positive multiple of 128");
    TVB_REQUIRE(it.a != nullptr && it.b != nullptr && it.scales != nullptr && it.c_ranks != nullptr, "tvb_qmm8_chain_create: NULL pointer");
    TVB_REQUIRE((reinterpret_cast<uintptr_t>(it.a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(it.b) & 15u) == 0 &&
                    (it.a_sm % 8 == 0 || it.m == 1),
                "tvb_qmm8_chain_create: A's rows and B must be 16-byte aligned");
    TVB_REQUIRE(it.independent >= 0 && it.independent <= kArriveSlots - 1, "tvb_qmm8_chain_create: independent must be between 0 and 3");
    TVB_REQUIRE(it.n_local * world < (int64_t(1) << 31), "tvb_qmm8_chain_create: sizes beyond 32 bits");
    for (int r = 0; r < world; r++) TVB_REQUIRE(it.c_ranks[r] != nullptr, "tvb_qmm8_chain_create: NULL output buffer of a rank");
    if (std::min<int64_t>(it.m, 16) > 8) nt = 2;
    if (it.n_local * it.k < (int64_t(64) << 20)) rw = 1;  // (small matrices: 128-row tiles, as tvb_qmm8 chooses)
    passes_total += ceil_div(it.m, 16);
  }
  const int rows_per_tile = 8 * rw * 16;
  const size_t partial_floats = static_cast<size_t>(8) * rw * nt * 32 * 4;

  // layout of the device block
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t at = off; off = (off + bytes + 255) & ~size_t(255); return at; };
  const size_t maps_at = take(static_cast<size_t>(passes_total) * 2 * sizeof(CUtensorMap));
  const size_t items_at = take(static_cast<size_t>(passes_total) * sizeof(ChainItemDev));
  const size_t done_at = take(256);
  const size_t counters_at = take(static_cast<size_t>(kChainSets) * kChainTileSlots * sizeof(int));
  const size_t channel_at = take(256);
  const size_t zero_until = off;  // (everything up to here except maps and descriptors starts at zero)
  const size_t partials_at = take(static_cast<size_t>(kChainSets) * grid * 2 * partial_floats * sizeof(float));
  const size_t total = off;

  std::vector<CUtensorMap> maps(static_cast<size_t>(passes_total) * 2);
  std::vector<ChainItemDev> devs(static_cast<size_t>(passes_total));
  size_t at = 0;
  for (int i = 0; i < count; i++) {
    const TvbChainItem& it = items[i];
    const int passes = static_cast<int>(ceil_div(it.m, 16));
    const int64_t tiles = ceil_div(it.n_local, rows_per_tile);
    TVB_REQUIRE(tiles <= kChainTileSlots, "tvb_qmm8_chain_create: too many output columns for a chained product");
    const int64_t stride = it.m == 1 ? it.k : it.a_sm;
    for (int pass = 0; pass < passes; pass++, at++) {
      if (make_tensor_map_2d(&maps[2 * at], it.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, it.k, it.n_local, it.k, kChunkK, rows_per_tile,
                             CU_TENSOR_MAP_SWIZZLE_128B) != 0)
        return -1;
      if (make_tensor_map_2d(&maps[2 * at + 1], it.a, dtype == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                             it.k, it.m, stride * 2, 64, nt * 8, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
        return -1;
      ChainItemDev& d = devs[at];
      std::memset(&d, 0, sizeof(d));
      d.scales = it.scales;
      for (int r = 0; r < world; r++) d.c[r] = it.c_ranks[r];
      d.m = static_cast<int>(it.m);
      d.m0 = 16 * pass;
      d.n = static_cast<int>(it.n_local);
      d.k = static_cast<int>(it.k);
      d.tiles = static_cast<int>(tiles);
      d.chunks = static_cast<int>(it.k / kChunkK);
      d.c_ld = static_cast<int>(it.n_local * world);
      d.c_col0 = static_cast<int>(rank * it.n_local);
      // (the passes of one product do not depend on each other)
      d.independent = static_cast<uint32_t>(std::min(it.independent * passes + pass, kArriveSlots - 1));
    }
  }

  Chain* c = new Chain();
  c->device = device;
  c->dtype = dtype;
  c->nt = nt;
  c->rw = rw;
  c->count = static_cast<int>(passes_total);
  c->grid = grid;
  cudaError_t err = cudaMalloc(&c->block, total);
  if (err != cudaSuccess) {
    delete c;
    return fail_cuda("tvb_qmm8_chain_create: cudaMalloc", err);
  }
  uint8_t* base = static_cast<uint8_t*>(c->block);
  err = cudaMemset(base + done_at, 0, zero_until - done_at);
  if (err == cudaSuccess) err = cudaMemcpy(base + maps_at, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(base + items_at, devs.data(), devs.size() * sizeof(ChainItemDev), cudaMemcpyHostToDevice);
  int* status = nullptr;
  if (err != cudaSuccess || status_word(device, &status) != 0) {
    cudaFree(c->block);
    delete c;
    return err != cudaSuccess ? fail_cuda("tvb_qmm8_chain_create: upload", err) : -1;
  }
  ChainParams& p = c->params;
  p.maps = reinterpret_cast<const CUtensorMap*>(base + maps_at);
  p.items = reinterpret_cast<const ChainItemDev*>(base + items_at);
  p.count = c->count;
  p.nranks = world;
  p.rank = rank;
  if (flag_ranks != nullptr) {
    for (int r = 0; r < world; r++) {
      if (flag_ranks[r] == nullptr) {
        cudaFree(c->block);
        delete c;
        return fail("tvb_qmm8_chain_create: NULL counters of a rank");
      }
      p.flags[r] = flag_ranks[r];
    }
    p.seq = seq_counter;
  } else {
    p.flags[0] = reinterpret_cast<uint32_t*>(base + channel_at);
    p.seq = p.flags[0] + kArriveWords;
  }
  p.done = reinterpret_cast<int*>(base + done_at);
  p.counters = reinterpret_cast<int*>(base + counters_at);
  p.partials = reinterpret_cast<float*>(base + partials_at);
  p.status = status;
  p.wait_at_end = wait_at_end != 0 && world > 1 ? 1 : 0;
  *chain_out = c;
  return 0;
}

extern "C" int tvb_qmm8_chain_run(int device, void* chain) {
  TVB_REQUIRE(chain != nullptr, "tvb_qmm8_chain_run: NULL chain");
  const Chain& c = *static_cast<const Chain*>(chain);
  TVB_REQUIRE(c.device == device, "tvb_qmm8_chain_run: the chain was made for another device");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  return c.dtype == TVB_BF16 ? chain_launch_dt<TVB_BF16>(c, stream) : chain_launch_dt<TVB_F16>(c, stream);
}

extern "C" void tvb_qmm8_chain_destroy(void* chain) {
  if (chain == nullptr) return;
  Chain* c = static_cast<Chain*>(chain);
  cudaStream_t stream;
  if (enter(c->device, &stream) == 0) {
    if (cudaStreamSynchronize(stream) != cudaSuccess) cudaGetLastError();
    if (cudaFree(c->block) != cudaSuccess) cudaGetLastError();
  }
  delete c;
}

// aten::_weight_int8pack_mm on sm_100a: C[m, n] = A[m, k] @ (int8 B[n, k] * scales[n]).T
//
// What it computes is the reference's qmm8 shader (crates/vkcore/shaders/qmm8.slang:
// float32 accumulation of A times the dequantised weights, rounded once to A's dtype;
// launched from crates/pyvk/csrc/quant.cpp:86-117). How it computes it is not:
//
//  * qmm8_skinny_kernel (m <= 16 per pass, 16-bit A): the decode path, bound by
//    streaming B from HBM once. Persistent CTAs, one per SM. One producer lane feeds
//    a ring of shared-memory stages with TMA (128-byte-swizzled boxes of 256 weight
//    rows x 128 k, plus the matching slice of A); eight consumer warps read 16 bytes
//    per lane, widen int8 to bf16 / f16 exactly in registers (two byte permutes and a
//    packed subtract per pair) and multiply with mma.sync m16n8k16 (weights as the
//    16-row operand, tokens as the 8-column operand), float32 accumulators.
//    Work is the list of (256-row tile, 128-k chunk) units cut into equal contiguous
//    ranges, one per CTA, so every SM streams the same number of bytes whatever n is;
//    a tile shared by several CTAs is finished by the CTA that holds its first k (for which
//    they are the last units of its range): the others leave their partial sums in scratch and
//    count themselves in without waiting for an answer; the finisher waits (briefly: all started
//    together with as many units; bounded) until all are counted and adds their sums in
//    descending CTA order, its own last, from registers (deterministic). Two shortcuts keep the
//    consumers streaming: a range that leaves a shared tile behind hands the arrival to an
//    otherwise idle agent warp and goes on at once; a finisher whose tile has already been
//    reached by all other contributors fetches their sums under its last chunks. The scale
//    multiplies the finished sum: (sum a*b) * s instead of sum a*(b*s); both are within
//    the float32 rounding the reference's tests allow (tests/python/test_quant.py:36-40).
//  * qmm8_plain_kernel: any shape, stride and dtype (float32 A included), one warp per
//    output column, as the shader's matrix-vector path (qmm8.slang:78-111).
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "numerics.cuh"
#include "ptx.cuh"
#include "qmm8_skinny.cuh"

namespace tvb {

// SM cycles the waits for peers may take (tvb_set_wait_limit_ms; the default is about two seconds).
std::atomic<long long> g_wait_limit_cycles{ptx::kWaitLimitCycles};

// The tcgen05 kernel for m > 16 (qmm8_tc.cu).
bool qmm8_tc_usable(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k);
int qmm8_tc(int device, cudaStream_t stream, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales, void* c,
            int64_t m, int64_t n, int64_t k);
// Very large m: the weights widened once into scratch, then the 16-bit tcgen05 GEMM (qmm8_tc.cu).
bool qmm8_widen_gemm_usable(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k);
int qmm8_widen_gemm(int device, cudaStream_t stream, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                    void* c, int64_t m, int64_t n, int64_t k);

// float32 A on the tensor cores through an exact three-term bfloat16 split (qmm8_f32_tc.cu).
bool qmm8_f32_tc_usable(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k);
int qmm8_f32_tc(int device, cudaStream_t stream, const float* a, int64_t a_sm, const int8_t* b, const float* scales, float* c, int64_t m,
                int64_t n, int64_t k);

namespace {

// ------------------------------------------------------------------ plain kernel

constexpr int kPlainRows = 8;

template <int DT>
__global__ void __launch_bounds__(256) qmm8_plain_kernel(const void* __restrict__ a, int64_t a_sm,
                                                         const int8_t* __restrict__ b, const void* __restrict__ scales,
                                                         void* __restrict__ c, int m, int n, int k) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int col = blockIdx.x * 8 + warp;
  if (col >= n) return;
  float scale = load_float<DT>(scales, col);
  const int8_t* brow = b + static_cast<int64_t>(col) * k;
  for (int r0 = blockIdx.y * kPlainRows; r0 < m; r0 += gridDim.y * kPlainRows) {
    float acc[kPlainRows];
#pragma unroll
    for (int r = 0; r < kPlainRows; r++) acc[r] = 0.0f;
    int rows = min(kPlainRows, m - r0);
    for (int kk = lane; kk < k; kk += 32) {
      float w = static_cast<float>(static_cast<int>(brow[kk])) * scale;
#pragma unroll
      for (int r = 0; r < kPlainRows; r++)
        if (r < rows) acc[r] = fmaf(load_float<DT>(a, static_cast<int64_t>(r0 + r) * a_sm + kk), w, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kPlainRows; r++) {
      float v = acc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && r < rows) store_float<DT>(c, static_cast<int64_t>(r0 + r) * n + col, v);
    }
  }
}

// ------------------------------------------------------------------ float32 A, aligned rows
//
// float32 activations cannot ride the 16-bit tensor-core operands exactly, so this stays on the CUDA cores: a warp owns
// four output columns and up to eight rows of A; its lanes walk k together (4 values per lane and step, so that a step's
// loads are one contiguous 512 bytes of each A row and 128 bytes of each weight row), every A value is used for four
// columns, float32 fmaf accumulation, a shuffle tree at the end, the scale applied to the finished sum.
// Needs k % 4 == 0 and 16-byte aligned rows of A; 4-byte aligned rows of B follow from k % 4 == 0.
constexpr int kF32Rows = 8, kF32Cols = 4;

__global__ void __launch_bounds__(256) qmm8_f32_kernel(const float* __restrict__ a, int64_t a_sm, const int8_t* __restrict__ b,
                                                       const float* __restrict__ scales, float* __restrict__ c, int m, int n,
                                                       int k) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = (blockIdx.x * 8 + warp) * kF32Cols;
  if (col0 >= n) return;
  const uint4* brow[kF32Cols];
#pragma unroll
  for (int j = 0; j < kF32Cols; j++)  // (columns past n read the last row again; their sums are dropped)
    brow[j] = reinterpret_cast<const uint4*>(b + static_cast<int64_t>(min(col0 + j, n - 1)) * k);
  for (int r0 = blockIdx.y * kF32Rows; r0 < m; r0 += gridDim.y * kF32Rows) {
    const int rows = min(kF32Rows, m - r0);
    float acc[kF32Rows][kF32Cols];
#pragma unroll
    for (int r = 0; r < kF32Rows; r++)
#pragma unroll
      for (int j = 0; j < kF32Cols; j++) acc[r][j] = 0.0f;
    // A lane takes 16 consecutive values of k per step (a warp: 512). The weights of the step after this one are
    // requested before this step's arithmetic: their latency is the loop's.
    uint4 ahead[kF32Cols];
#pragma unroll
    for (int j = 0; j < kF32Cols; j++) ahead[j] = lane * 16 < k ? __ldcs(brow[j] + lane) : make_uint4(0u, 0u, 0u, 0u);
    for (int kk = lane * 16; kk < k; kk += 512) {
      uint4 cur[kF32Cols];
#pragma unroll
      for (int j = 0; j < kF32Cols; j++) {
        cur[j] = ahead[j];
        if (kk + 512 < k) ahead[j] = __ldcs(brow[j] + ((kk + 512) >> 4));
      }
#pragma unroll
      for (int q = 0; q < 4; q++) {  // four values of k at a time
        float w[kF32Cols][4];
#pragma unroll
        for (int j = 0; j < kF32Cols; j++) {
          const uint32_t word = q == 0 ? cur[j].x : (q == 1 ? cur[j].y : (q == 2 ? cur[j].z : cur[j].w));
#pragma unroll
          for (int i = 0; i < 4; i++) w[j][i] = static_cast<float>(static_cast<int>(static_cast<int8_t>(word >> (8 * i))));
        }
#pragma unroll
        for (int r = 0; r < kF32Rows; r++) {
          if (r < rows) {
            const float4 av = *reinterpret_cast<const float4*>(a + static_cast<int64_t>(r0 + r) * a_sm + kk + 4 * q);
#pragma unroll
            for (int j = 0; j < kF32Cols; j++) {
              acc[r][j] = fmaf(av.x, w[j][0], acc[r][j]);
              acc[r][j] = fmaf(av.y, w[j][1], acc[r][j]);
              acc[r][j] = fmaf(av.z, w[j][2], acc[r][j]);
              acc[r][j] = fmaf(av.w, w[j][3], acc[r][j]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kF32Rows; r++)
#pragma unroll
      for (int j = 0; j < kF32Cols; j++) {
        float v = acc[r][j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && r < rows && col0 + j < n) c[static_cast<int64_t>(r0 + r) * n + col0 + j] = v * scales[col0 + j];
      }
  }
}

// ------------------------------------------------------------------ skinny kernel


struct SkinnyParams {
  const void* scales;
  void* c[kMaxRanks + 1];    // output buffers [m, c_ld]: this GPU's, and with sharding every peer's (peer-mapped memory); a
                             // grouped launch may add one in page-locked host memory
  int ndest;                 // how many of them (nranks, or nranks + 1 with the host's)
  uint32_t* flags[kMaxRanks];  // with sharding: every rank's arrival counters (entry `rank` of each is this GPU's to add to)
  int* done;                 // with sharding: counter of finished CTAs (zero between launches)
  int nranks, rank;
  uint32_t* seq;             // with sharding: device counter of the sharded products this rank has completed on the channel
  uint32_t independent;      // with sharding: how many of the latest products of the channel this one need not wait for
  long long wait_limit;      // with sharding: SM cycles after which the wait for the peers gives up
  int c_ld, c_col0;          // row length of the output buffers and first column of this GPU's slice
  float* partials;   // [grid][2][kPartialFloats]
  int* counters;     // [tiles], zero between launches
  int* status;
  int m, n, k;
  int m0;            // first token row of this pass
  int tiles, chunks; // tiles = ceil(n / rows per tile), chunks = k / 128
  const void* bias;      // n values of A's dtype added to the rounded product (rounded again), or NULL
  const void* residual;  // [m, c_ld] of A's dtype, laid out like the output, added after the bias (rounded again), or NULL
};

// Several products of one shape in one launch (tvb_qmm8_group): product g has its own activations, weights, scales and
// outputs; n, k and the tiling are shared. The kernel's tiles are numbered through all products (tile = g * tiles + its
// tile within product g), so the list of (tile, chunk) units, cut into one contiguous range per CTA, runs across them: a
// CTA shares at most the two tiles at its range's ends with other CTAs however many products the launch holds.
constexpr int kMaxGroup = 4;
struct SkinnyGroup {
  CUtensorMap map_w[kMaxGroup], map_a[kMaxGroup];
  const void* scales[kMaxGroup];
  void* c[kMaxGroup][kMaxRanks + 1];
  int m[kMaxGroup];
  int count;
};
struct NoGroup {};
template <bool GROUP> struct GroupArg { using type = NoGroup; };
template <> struct GroupArg<true> { using type = SkinnyGroup; };

// What a Linear does after the product, in the thread that holds the finished value: + bias[col], then + residual[token,
// col], each sum rounded to the output type as the separate kernels would round it (so the fused result is bit for bit
// that of product, add, add).
template <int DT>
__device__ __forceinline__ uint16_t skinny_epilogue(const SkinnyParams& p, uint16_t bits, int token, int col) {
  if (p.bias != nullptr) bits = float_to_half_bits<DT>(half_bits_to_float<DT>(bits) + load_float<DT>(p.bias, col));
  if (p.residual != nullptr)
    bits = float_to_half_bits<DT>(half_bits_to_float<DT>(bits) +
                                  load_float<DT>(p.residual, static_cast<int64_t>(token) * p.c_ld + p.c_col0 + col));
  return bits;
}

// acc += the partial sums that CTAs hi, hi - 1, ..., lo left in scratch for `tile`, in that order (the one fixed order of
// additions). The addresses of a few contributors are worked out first and their loads issued together: with one
// contributor at a time, each one's index arithmetic (two divisions) and its trip to the L2 came one after the other, and
// the CTA that finishes a shared tile was the last of its launch to end by about 3 us.
template <class Cfg, int RW, int NT>
__device__ __forceinline__ void add_partials(float (&acc)[RW][NT][4], const float* partials, const int hi, const int lo, const int tile,
                                             const long long units, const long long grid, const bool small, const int chunks,
                                             const int warp, const int lane) {
  // (the configurations of large matrices and wide passes keep one contributor at a time: their registers are spoken for,
  // and a launch of theirs is long against its finish)
  constexpr int kBatch = RW * NT <= 2 ? 4 : 1;
  for (int top = hi; top >= lo; top -= kBatch) {
    const float4* theirs[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
      const int cta = top - j >= lo ? top - j : lo;  // (past the end: a valid address whose values are not added)
      const bool cta_first_segment = unit_tile(range_start(cta, units, grid, small), chunks, small) == tile;
      theirs[j] = reinterpret_cast<const float4*>(partials + (static_cast<size_t>(cta) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
    }
    float4 v[kBatch][RW][NT];
#pragma unroll
    for (int j = 0; j < kBatch; j++)
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) v[j][rb][nt] = __ldcg(&theirs[j][((warp * RW + rb) * NT + nt) * 32 + lane]);
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
      if (top - j < lo) break;
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          acc[rb][nt][0] += v[j][rb][nt].x; acc[rb][nt][1] += v[j][rb][nt].y; acc[rb][nt][2] += v[j][rb][nt].z; acc[rb][nt][3] += v[j][rb][nt].w;
        }
    }
  }
}

// ADDS: the instantiation whose epilogue also adds a bias and a residual (tvb_qmm8_linear); the plain product carries no
// code for them (with it in one kernel, behind a test of the two pointers, every launch was 0.65 us slower).
template <int DT, int NT, int RW, int NWARPS, bool ADDS = false, bool GROUP = false>
__global__ void __launch_bounds__((NWARPS + 2) * 32, 1)
    qmm8_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                       const SkinnyParams p, const __grid_constant__ typename GroupArg<GROUP>::type group) {
  using Cfg = SkinnyCfg<NT, RW, NWARPS>;
  static_assert(!(ADDS && GROUP), "grouped products carry no adds");
  // Who finishes a tile that several CTAs share: the CTA that holds its first k, which waits for the others (single
  // products: 1.3 us less per dependent launch), or whichever CTA arrives last (grouped launches, whose long ranges drift
  // apart: measured 2.3 % faster that way).
  constexpr bool kLastFinishes = GROUP;
  // product g of a grouped launch (g = 0 otherwise): which product a tile belongs to, and that product's operands
  auto split = [&](int tile, int& g, int& lt) {
    if constexpr (GROUP) {
      g = tile / p.tiles;
      lt = tile - g * p.tiles;
    } else {
      g = 0;
      lt = tile;
    }
  };
  auto weights_of = [&](int g) -> const CUtensorMap* {
    if constexpr (GROUP) return &group.map_w[g];
    else return &map_w;
  };
  auto tokens_of = [&](int g) -> const CUtensorMap* {
    if constexpr (GROUP) return &group.map_a[g];
    else return &map_a;
  };
  auto scales_of = [&](int g) -> const void* {
    if constexpr (GROUP) return group.scales[g];
    else return p.scales;
  };
  auto rows_of = [&](int g) -> int {
    if constexpr (GROUP) return group.m[g];
    else return p.m;
  };
  auto out_of = [&](int g, int r) -> void* {
    if constexpr (GROUP) return group.c[g][r];
    else return p.c[r];
  };
  int products = 1;
  if constexpr (GROUP) products = group.count;
  extern __shared__ uint8_t smem_raw[];
  // stages need 1024-byte alignment for the 128-byte swizzle pattern
  uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + Cfg::kStages * Cfg::kStageBytes);
  const uint32_t full0 = ptx::smem_u32(bars), empty0 = full0 + 8 * Cfg::kStages;
  const uint32_t agent_bar = empty0 + 8 * Cfg::kStages;  // the consumers have stored the partial sums of a segment they leave behind
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * Cfg::kStages + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;  // two slots
  int* early_flag = last_flag + 2;  // set when every other contributor of the segment's tile was seen to have arrived
  uint16_t* out_tile = reinterpret_cast<uint16_t*>(base_ptr + Cfg::kStages * Cfg::kStageBytes + 256);  // [tokens][rows of a tile]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, NWARPS);
    }
    ptx::mbar_init(agent_bar, NWARPS);
    *abort_flag = 0;
    last_flag[0] = last_flag[1] = 0;
    *early_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  ptx::grid_launch_dependents();  // the next kernel of the stream may take SMs as this one's CTAs retire

  const long long units = static_cast<long long>(p.tiles) * products * p.chunks;
  const long long grid = gridDim.x;
  const bool small = (units + 1) * (grid + 1) < (1ll << 31);
  const long long u0 = range_start(blockIdx.x, units, grid, small), u1 = range_start(blockIdx.x + 1, units, grid, small);

  if (warp == NWARPS) {
    // ---------------- producer: one lane issues every TMA copy
    const uint64_t stream_policy = ptx::policy_evict_first();  // weights are read once
    const uint64_t keep_policy = ptx::policy_evict_last();     // every CTA re-reads A
    const long long mine = u1 - u0;
    const long long ahead = mine < Cfg::kStages ? mine : Cfg::kStages;
    if (lane == 0) {
      for (int g = 0; g < products; g++) {
        ptx::prefetch_tensormap(weights_of(g));
        ptx::prefetch_tensormap(tokens_of(g));
      }
      // The weights do not depend on earlier kernels of the stream: start streaming them at once, one ring's worth.
      // A (which an earlier kernel may have produced) is fetched only after the stream's earlier work has completed.
      for (long long j = 0; j < ahead; j++) {
        const long long u = u0 + j;
        const int tile = unit_tile(u, p.chunks, small), chunk = static_cast<int>(u - static_cast<long long>(tile) * p.chunks);
        int g, lt;
        split(tile, g, lt);
        const uint32_t dst = base + static_cast<int>(j) * Cfg::kStageBytes;
        ptx::mbar_expect_tx(full0 + 8 * static_cast<int>(j), Cfg::kStageBytes);
        ptx::tma_load_2d_hint(dst, weights_of(g), chunk * kChunkK, lt * Cfg::kRowsPerTile, full0 + 8 * static_cast<int>(j), stream_policy);
      }
    }
    if (p.done != nullptr) {
      // Sharded product: before this CTA reads A or stores a column, every rank must have delivered the earlier products
      // of the channel (all but the latest `independent` ones). The previous product's output may be this one's A; and a
      // rank that has delivered has also finished reading its own A, which this product may be about to overwrite (two
      // output buffers in turn). The warp waits (bounded), one arrival counter per lane.
      ptx::grid_dependency_wait();  // (this rank's previous kernel has ended: the product count below is final)
      {
        const long long count = *reinterpret_cast<const volatile uint32_t*>(p.seq);
        const long long upto = count - 1 - static_cast<long long>(p.independent);
        const long long start = clock64();
        for (int spins = 0; !arrivals_complete_warp(p.flags[p.rank], p.nranks, upto); spins++) {
          if ((spins & 63) == 63) {
            // an earlier give-up (here or in an earlier kernel) is final: nobody waits the limit out a second time
            bool stop = *reinterpret_cast<volatile int*>(p.status) != 0;
            if (!stop && clock64() - start > p.wait_limit) {
              atomicExch(p.status, 5);
              stop = true;
            }
            if (__any_sync(0xffffffffu, stop)) break;
          }
        }
      }
      __syncwarp();
      asm volatile("fence.proxy.async.global;" ::: "memory");  // (the copies below read what the peers' stores delivered)
    }
    if (lane == 0) {
      ptx::grid_dependency_wait();
      for (long long j = 0; j < ahead; j++) {
        const int tile_j = unit_tile(u0 + j, p.chunks, small);
        const int chunk = static_cast<int>(u0 + j - static_cast<long long>(tile_j) * p.chunks);
        int g, lt;
        split(tile_j, g, lt);
        const uint32_t dst = base + static_cast<int>(j) * Cfg::kStageBytes + Cfg::kWeightBytes;
        ptx::tma_load_2d_hint(dst, tokens_of(g), chunk * kChunkK, p.m0, full0 + 8 * static_cast<int>(j), keep_policy);
        ptx::tma_load_2d_hint(dst + Cfg::kTokenBoxBytes, tokens_of(g), chunk * kChunkK + 64, p.m0, full0 + 8 * static_cast<int>(j), keep_policy);
      }
      long long it = ahead;
      bool ok = true;
      int tile, g;
      split(unit_tile(u0 + ahead, p.chunks, small), g, tile);  // (`tile` counts within product g from here on)
      int chunk = static_cast<int>(u0 + ahead - static_cast<long long>(unit_tile(u0 + ahead, p.chunks, small)) * p.chunks);
      for (long long u = u0 + ahead; u < u1 && ok; u++, it++, chunk++) {
        if (chunk == p.chunks) {
          chunk = 0;
          tile++;
          if (GROUP && tile == p.tiles) {
            tile = 0;
            g++;
          }
        }
        int s = static_cast<int>(it % Cfg::kStages);
        uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
        ok = ptx::mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag);
        if (!ok) break;
        uint32_t dst = base + s * Cfg::kStageBytes;
        ptx::mbar_expect_tx(full0 + 8 * s, Cfg::kStageBytes);
        ptx::tma_load_2d_hint(dst, weights_of(g), chunk * kChunkK, tile * Cfg::kRowsPerTile, full0 + 8 * s, stream_policy);
        ptx::tma_load_2d_hint(dst + Cfg::kWeightBytes, tokens_of(g), chunk * kChunkK, p.m0, full0 + 8 * s, keep_policy);
        ptx::tma_load_2d_hint(dst + Cfg::kWeightBytes + Cfg::kTokenBoxBytes, tokens_of(g), chunk * kChunkK + 64, p.m0,
                              full0 + 8 * s, keep_policy);
      }
      // Leave no copy in flight behind: every stage that was armed has landed before the CTA ends.
      long long first = it > Cfg::kStages ? it - Cfg::kStages : 0;
      for (long long j = first; j < it; j++) {
        int s = static_cast<int>(j % Cfg::kStages);
        uint32_t ph = static_cast<uint32_t>((j / Cfg::kStages) & 1);
        volatile int never = 0;
        ptx::mbar_wait(full0 + 8 * s, ph, &never);
      }
      if (*abort_flag != 0) atomicExch(p.status, 1);
    }
    return;
  }

  if (warp == NWARPS + 1) {
    // ---------------- agent: arrival at the tile that this CTA's first segment shares
    // A range that starts inside a tile and goes on beyond it leaves that tile's partial sums in scratch and moves on
    // at once; this warp counts the arrival in the consumers' stead.
    const int tile = unit_tile(u0, p.chunks, small), c0 = static_cast<int>(u0 - static_cast<long long>(tile) * p.chunks);
    const int c1 = static_cast<int>(min(static_cast<long long>(p.chunks), c0 + (u1 - u0)));
    const bool left_behind = !(c0 == 0 && c1 == p.chunks) && u0 + (c1 - c0) < u1;
    if (left_behind && ptx::mbar_wait(agent_bar, 0, abort_flag)) {
      ptx::grid_dependency_wait();
      if constexpr (kLastFinishes) {
      const long long tile_first_unit = static_cast<long long>(tile) * p.chunks;
      const int cta_first = range_owner(tile_first_unit, units, grid, small);
      const int cta_last = range_owner(tile_first_unit + p.chunks - 1, units, grid, small);
      int last = 0;
      if (lane == 0) {
        __threadfence();  // (cumulative over the consumers' stores, which the barrier ordered before this)
        last = atomicAdd(&p.counters[tile], 1) == cta_last - cta_first;
        if (last) atomicExch(&p.counters[tile], 0);
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence();
        int product, lt;
        split(tile, product, lt);
        const int g = lane >> 2, t = lane & 3, rg = (g >> 1) | ((g & 1) << 2);
        for (int w = 0; w < NWARPS; w++)  // this warp plays every consumer warp's part in turn
#pragma unroll
          for (int rb = 0; rb < RW; rb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
              for (int cta = cta_last; cta >= cta_first; cta--) {  // the one fixed order of additions
                const bool cta_first_segment = unit_tile(range_start(cta, units, grid, small), p.chunks, small) == tile;
                const float4* theirs = reinterpret_cast<const float4*>(
                    p.partials + (static_cast<size_t>(cta) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
                const float4 v = __ldcg(&theirs[((w * RW + rb) * NT + nt) * 32 + lane]);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
              }
              const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
              for (int half = 0; half < 2; half++) {
                const int col = lt * Cfg::kRowsPerTile + (w * RW + rb) * 16 + rg + 8 * half;
                if (col >= p.n) continue;
                const float scale = load_float<DT>(scales_of(product), col);
#pragma unroll
                for (int i = 0; i < 2; i++) {
                  const int token = p.m0 + nt * 8 + 2 * t + i;
                  if (token >= rows_of(product)) continue;
                  const float v = vals[2 * half + i] * scale;
                  uint16_t bits = DT == TVB_BF16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
                  if constexpr (ADDS) bits = skinny_epilogue<DT>(p, bits, token, col);
                  const int64_t off = static_cast<int64_t>(token) * p.c_ld + p.c_col0 + col;
                  for (int r = 0; r < p.ndest; r++) static_cast<uint16_t*>(out_of(product, r))[off] = bits;
                }
              }
            }
      }
      } else if (lane == 0) {
        __threadfence();  // (cumulative over the consumers' stores, which the barrier ordered before this)
        atomicAdd(&p.counters[tile], 1);  // (this CTA holds the tile's last k: the tile's finisher is another CTA, see below)
      }
    }
    if (p.done != nullptr) {
      __syncwarp();
      ptx::named_bar_arrive(2, (NWARPS + 1) * 32);  // (its stores come before the CTA reports its columns as delivered)
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
  long long u = u0;
  while (u < u1 && ok) {
    const int tile = unit_tile(u, p.chunks, small), c0 = static_cast<int>(u - static_cast<long long>(tile) * p.chunks);
    const int c1 = static_cast<int>(min(static_cast<long long>(p.chunks), c0 + (u1 - u)));
    const bool first_segment = (u == u0);
    const bool whole_tile = c0 == 0 && c1 == p.chunks;
    // The ranges that share this tile (consecutive CTAs). Their partial sums are always added in descending CTA order.
    const long long tile_first_unit = static_cast<long long>(tile) * p.chunks;
    const int cta_first = whole_tile ? static_cast<int>(blockIdx.x) : range_owner(tile_first_unit, units, grid, small);
    const int cta_last = whole_tile ? static_cast<int>(blockIdx.x) : range_owner(tile_first_unit + p.chunks - 1, units, grid, small);
    // A CTA that holds the tile's first k (the usual case for the last tile of its range) is added last. If, shortly
    // before its segment ends, it sees that all the others have already arrived, it is certain to finish the tile: it
    // then fetches their sums while its last chunks are in flight and skips the exchange through scratch altogether.
    const bool may_be_early = !whole_tile && cta_first == static_cast<int>(blockIdx.x) && c1 - c0 >= 3;
    int product, lt;  // the product the tile belongs to and the tile's index within it
    split(tile, product, lt);
    const int m_rows = rows_of(product);
    bool early = false;
    int peeked = 0;
    float pre[RW][NT][4];
#pragma unroll
    for (int rb = 0; rb < RW; rb++)
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[rb][nt][i] = pre[rb][nt][i] = 0.0f;

    // This thread's columns' scales, asked for now: each is read once per launch, so the load goes to DRAM, and at the
    // end of the segment (where the finished sums need it) it would wait in line behind the other SMs' weight traffic.
    float scale_pre[RW][2];
#pragma unroll
    for (int rb = 0; rb < RW; rb++)
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int col = lt * Cfg::kRowsPerTile + (warp * RW + rb) * 16 + rg + 8 * half;
        scale_pre[rb][half] = col < p.n ? load_float<DT>(scales_of(product), col) : 0.0f;
      }
    float bias_pre[ADDS ? RW : 1][2];
    uint32_t residual_pre[ADDS ? RW : 1][NT][2];  // [..][half]: the values of tokens 2t (low 16 bits) and 2t + 1

    if constexpr (ADDS) {
      // (the first stage of the segment has landed: the producer has waited for the stream's earlier kernels by then.
      // Waiting here as well as in the loop below is harmless: only the consumers release a stage.)
      const int s0 = static_cast<int>(it % Cfg::kStages);
      const uint32_t ph0 = static_cast<uint32_t>((it / Cfg::kStages) & 1);
      ok = ptx::mbar_wait(full0 + 8 * s0, ph0, abort_flag);
      if (!ok) break;
      {
      // the values this thread would add if it finishes the tile, for the same reason asked for early; the residual
      // may be the previous kernel's output, hence not before that kernel has ended
      ptx::grid_dependency_wait();
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int col = lt * Cfg::kRowsPerTile + (warp * RW + rb) * 16 + rg + 8 * half;
          bias_pre[rb][half] = p.bias != nullptr && col < p.n ? load_float<DT>(p.bias, col) : 0.0f;
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            uint32_t pair = 0;
#pragma unroll
            for (int i = 0; i < 2; i++) {
              const int token = p.m0 + nt * 8 + 2 * t + i;
              if (p.residual != nullptr && col < p.n && token < p.m)
                pair |= static_cast<uint32_t>(
                            static_cast<const uint16_t*>(p.residual)[static_cast<int64_t>(token) * p.c_ld + p.c_col0 + col])
                        << (16 * i);
            }
            residual_pre[rb][nt][half] = pair;
          }
        }
      }
    }

    for (int chunk = c0; chunk < c1; chunk++, it++) {
      const int s = static_cast<int>(it % Cfg::kStages);
      const uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
      ok = ptx::mbar_wait(full0 + 8 * s, ph, abort_flag);
      if (!ok) break;
      // (past the first stage's barrier the stream's earlier kernels have completed: the producer waited for them)
      if (may_be_early) {
        if (chunk == c1 - 3) {
          if (threadIdx.x == 0) asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(peeked) : "l"(p.counters + tile) : "memory");
        } else if (chunk == c1 - 2) {
          if (threadIdx.x == 0) *early_flag = peeked == cta_last - cta_first;
        } else if (chunk == c1 - 1) {
          ptx::named_bar_sync(1, NWARPS * 32);
          early = *early_flag != 0;
          if (early) {
            // the highest contributor's sums: requested now, first needed after this segment's last chunk
            const bool cta_first_segment = unit_tile(range_start(cta_last, units, grid, small), p.chunks, small) == tile;
            const float4* theirs = reinterpret_cast<const float4*>(
                p.partials + (static_cast<size_t>(cta_last) * 2 + (cta_first_segment ? 0 : 1)) * Cfg::kPartialFloats);
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
    ptx::grid_dependency_wait();  // (scratch, counters and C may still be in use by the stream's previous kernel)
    bool finish = true;
    if (early) {
      // every other contributor was counted before this CTA looked: nobody else will touch the counter again
      if (threadIdx.x == 0) atomicExch(&p.counters[tile], 0);
      // the same additions in the same order as the general path below: from zero, descending, this CTA's sums last
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) pre[rb][nt][i] = 0.0f + pre[rb][nt][i];
      add_partials<Cfg, RW, NT>(pre, p.partials, cta_last - 1, cta_first + 1, tile, units, grid, small, p.chunks, warp, lane);
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) acc[rb][nt][i] = pre[rb][nt][i] + acc[rb][nt][i];
    } else if (!kLastFinishes && !whole_tile && cta_first == static_cast<int>(blockIdx.x)) {
      // This CTA holds the tile's first k, which are the last units of its range: it finishes the tile. The other
      // contributors arrive at about the same time (they started together and have as many units), so the wait is
      // short, and bounded; then their sums are added in descending CTA order and this CTA's own last, from registers.
      // (With "whoever arrives last finishes", the last arriver paid for a round trip of its own sums through scratch,
      // an atomic whose answer it had to wait for and a fence before it could fetch anything: 1.3 us more per launch.)
      int* flag = last_flag + (segment & 1);
      if (threadIdx.x == 0) {
        const int want = cta_last - cta_first;
        int seen = 0, done = 0;
        const long long start = clock64();
        for (;;) {
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile) : "memory");
          if (seen == want) {
            done = 1;
            break;
          }
          if (*abort_flag != 0 || clock64() - start > ptx::kWaitLimitCycles) break;
        }
        if (done) atomicExch(&p.counters[tile], 0);  // zero again for the next launch: nobody else touches it any more
        else *abort_flag = 1;
        *flag = done;
      }
      ptx::named_bar_sync(1, NWARPS * 32);
      const bool arrived = *flag != 0;
      segment++;
      if (!arrived) {
        ok = false;
        break;
      }
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) pre[rb][nt][i] = 0.0f;
      add_partials<Cfg, RW, NT>(pre, p.partials, cta_last, cta_first + 1, tile, units, grid, small, p.chunks, warp, lane);
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) acc[rb][nt][i] = pre[rb][nt][i] + acc[rb][nt][i];
    } else if (!whole_tile) {
      float4* mine = reinterpret_cast<float4*>(p.partials + (static_cast<size_t>(blockIdx.x) * 2 + (first_segment ? 0 : 1)) *
                                                                Cfg::kPartialFloats);
#pragma unroll
      for (int rb = 0; rb < RW; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
          __stcg(&mine[((warp * RW + rb) * NT + nt) * 32 + lane],
                 make_float4(acc[rb][nt][0], acc[rb][nt][1], acc[rb][nt][2], acc[rb][nt][3]));
      if constexpr (kLastFinishes) {
      if (u + (c1 - c0) < u1) {
        // More of the range follows: leave the tile to the agent warp (which counts this arrival) and go on at once.
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(agent_bar);
        finish = false;
      } else {
        // All consumer threads have stored their partial sums once they pass the barrier; one thread then publishes
        // them: its gpu-scope fence is cumulative over what the barrier ordered before it.
        ptx::named_bar_sync(1, NWARPS * 32);
        int* flag = last_flag + (segment & 1);  // (alternating slots: no barrier needed before the next segment rewrites it)
        if (threadIdx.x == 0) {
          __threadfence();
          int arrived = atomicAdd(&p.counters[tile], 1);
          int last = arrived == cta_last - cta_first;
          if (last) atomicExch(&p.counters[tile], 0);  // zero again for the next launch
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
          // fixed order: the sum does not depend on who came last
          add_partials<Cfg, RW, NT>(acc, p.partials, cta_last, cta_first, tile, units, grid, small, p.chunks, warp, lane);
        }
      }
      } else {
      finish = false;
      if (u + (c1 - c0) < u1) {
        // More of the range follows: leave the tile to the agent warp (which counts this arrival) and go on at once.
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(agent_bar);
      } else {
        // All consumer threads have stored their partial sums once they pass the barrier; one thread then publishes
        // them: its gpu-scope fence is cumulative over what the barrier ordered before it. Nobody waits for the answer.
        ptx::named_bar_sync(1, NWARPS * 32);
        if (threadIdx.x == 0) {
          __threadfence();
          atomicAdd(&p.counters[tile], 1);
        }
      }
      }
    }
    if (finish) {
      // Scale, round once, and stage the tile's [tokens][256 columns] in shared memory, so that what goes to global
      // memory (this GPU's output and, with sharding, every peer's over NVLink) is 16-byte, fully coalesced stores.
#pragma unroll
      for (int rb = 0; rb < RW; rb++) {
        const int lrow0 = (warp * RW + rb) * 16 + rg;
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int lcol = lrow0 + 8 * half;                       // column within the tile (weight row = output column)
          const float scale = scale_pre[rb][half];
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 2; i++) {
              const float v = acc[rb][nt][2 * half + i] * scale;
              uint16_t bits = float_to_half_bits<DT>(v);
              if constexpr (ADDS) {
                if (p.bias != nullptr) bits = float_to_half_bits<DT>(half_bits_to_float<DT>(bits) + bias_pre[rb][half]);
                if (p.residual != nullptr)
                  bits = float_to_half_bits<DT>(half_bits_to_float<DT>(bits) + half_bits_to_float<DT>(static_cast<uint16_t>(residual_pre[rb][nt][half] >> (16 * i))));
              }
              out_tile[(nt * 8 + 2 * t + i) * Cfg::kRowsPerTile + lcol] = bits;
            }
        }
      }
      ptx::named_bar_sync(1, NWARPS * 32);
      const int col_base = lt * Cfg::kRowsPerTile;
      const bool vec = (p.c_ld % 8 == 0) && (p.c_col0 % 8 == 0);
      for (int v = threadIdx.x; v < Cfg::kTokens * (Cfg::kRowsPerTile / 8); v += NWARPS * 32) {
        const int tok = v / (Cfg::kRowsPerTile / 8), chunk = v % (Cfg::kRowsPerTile / 8);
        const int token = p.m0 + tok, col = col_base + chunk * 8;
        if (token >= m_rows || col >= p.n) continue;
        const uint4 val = *reinterpret_cast<const uint4*>(out_tile + tok * Cfg::kRowsPerTile + chunk * 8);
        const int64_t off = static_cast<int64_t>(token) * p.c_ld + p.c_col0 + col;
        if (vec && col + 8 <= p.n) {
          for (int r = 0; r < p.ndest; r++) {
            uint16_t* dst = static_cast<uint16_t*>(out_of(product, r)) + off;
            if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
              *reinterpret_cast<uint4*>(dst) = val;
            } else {
              const uint16_t* e = reinterpret_cast<const uint16_t*>(&val);
              for (int j = 0; j < 8; j++) dst[j] = e[j];
            }
          }
        } else {
          const uint16_t* e = reinterpret_cast<const uint16_t*>(&val);
          for (int r = 0; r < p.ndest; r++)
            for (int j = 0; j < 8 && col + j < p.n; j++) (static_cast<uint16_t*>(out_of(product, r)) + off)[j] = e[j];
        }
      }
      ptx::named_bar_sync(1, NWARPS * 32);  // (the staging tile is free again)
    }
    u += c1 - c0;
  }
  if (p.done != nullptr && ok) {
    // Sharded product: this CTA's columns are stored everywhere (and it has read all of A it will ever read): add its
    // share to this rank's arrival counter on every rank, this one included. The system-scope fence after the barrier
    // covers the stores of all the CTA's threads; no CTA waits for another, and columns count as they land.
    ptx::named_bar_sync(2, (NWARPS + 1) * 32);  // (the agent warp arrives here too, after whatever it had to store)
    if (threadIdx.x == 0) {
      if (p.nranks == 1 && p.ndest == 1) __threadfence();
      else __threadfence_system();
      // (a grouped launch holds `products` products of the channel: the CTA reports its share of each, whichever tiles
      // it had, since the counters say "every CTA of the launch is past its stores")
      const uint32_t first = *reinterpret_cast<const volatile uint32_t*>(p.seq);
      for (int q = 0; q < products; q++) arrive_publish(p.flags, p.nranks, p.rank, first + static_cast<uint32_t>(q), arrive_share());
      // the last CTA to get here counts the products (the next kernel of the stream reads the count after this one has ended)
      if (atomicAdd(p.done, 1) == static_cast<int>(gridDim.x) - 1) {
        atomicExch(p.done, 0);
        *reinterpret_cast<volatile uint32_t*>(p.seq) = first + static_cast<uint32_t>(products);
      }
    }
  }
}

// ------------------------------------------------------------------ host side

template <int DT>
int launch_plain(cudaStream_t stream, const void* a, int64_t a_sm, const int8_t* b, const void* scales, void* c, int m, int n,
                 int k) {
  dim3 grid(static_cast<unsigned>(ceil_div(n, 8)), static_cast<unsigned>(std::min<int64_t>(ceil_div(m, kPlainRows), 64)));
  qmm8_plain_kernel<DT><<<grid, 256, 0, stream>>>(a, a_sm, b, scales, c, m, n, k);
  return launched("qmm8_plain", grid, dim3(256), 0, stream);
}

// Destinations of a sharded product (tvb_qmm8_gather): every rank's output buffer and flag array.
// What tvb_qmm8_linear adds to the product in the decode kernel's epilogue (either may be NULL).
struct SkinnyAdds {
  const void* bias;
  const void* residual;
};

struct GatherTargets {
  void* c[kMaxRanks];
  uint32_t* flags[kMaxRanks];
  int world, rank;
  uint32_t* seq;
  uint32_t independent;
  int64_t n_total;
};

template <int DT, int NT, int RW, int NWARPS, bool ADDS = false>
int launch_skinny_cfg(int device, cudaStream_t stream, const void* a, int64_t a_sm, const int8_t* b, const void* scales, void* c,
                      int m, int n, int k, int m0, const GatherTargets* gather = nullptr, const SkinnyAdds* adds = nullptr) {
  using Cfg = SkinnyCfg<NT, RW, NWARPS>;
  auto kernel = qmm8_skinny_kernel<DT, NT, RW, NWARPS, ADDS>;
  {
    static std::mutex mutex;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> lock(mutex);
    if (!configured[device & 63]) {
      TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      configured[device & 63] = true;
    }
  }
  CUtensorMap map_w, map_a;
  if (make_tensor_map_2d(&map_w, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, k, n, k, kChunkK, Cfg::kRowsPerTile,
                         CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  if (make_tensor_map_2d(&map_a, a, DT == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, m,
                         a_sm * 2, 64, Cfg::kTokens, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  SkinnyParams p{};
  p.tiles = static_cast<int>(ceil_div(n, Cfg::kRowsPerTile));
  p.chunks = k / kChunkK;
  long long units = static_cast<long long>(p.tiles) * p.chunks;
  int grid = static_cast<int>(std::min<long long>(sm_count(device), units));
  if (gather != nullptr && grid > static_cast<int>(kArriveWeight)) return fail("tvb_qmm8_gather: more than 1024 SMs");
  size_t partial_bytes = static_cast<size_t>(grid) * 2 * Cfg::kPartialFloats * sizeof(float);
  // Fixed layout, whatever the shape: 64 KB of tile counters (and, last, the finished-CTA counter), then the partial
  // sums. The counters must stay zero between launches, so no launch may ever use their bytes for anything else.
  constexpr size_t counter_bytes = kCounterBytes;
  if (p.tiles > kMaxTiles) return fail("tvb_qmm8: more than 4 million output columns for the decode kernel");
  void* ws = nullptr;
  if (workspace(device, 0, counter_bytes + partial_bytes, &ws) != 0) return -1;
  p.counters = static_cast<int*>(ws);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + counter_bytes);
  if (status_word(device, &p.status) != 0) return -1;
  p.scales = scales;
  p.c[0] = c;
  p.nranks = 1;
  p.c_ld = n;
  p.c_col0 = 0;
  p.m = m;
  p.n = n;
  p.k = k;
  p.m0 = m0;
  if (adds != nullptr) {
    p.bias = adds->bias;
    p.residual = adds->residual;
  }
  if (gather != nullptr) {
    for (int r = 0; r < gather->world; r++) {
      p.c[r] = gather->c[r];
      p.flags[r] = gather->flags[r];
    }
    p.nranks = gather->world;
    p.rank = gather->rank;
    p.seq = gather->seq;
    p.independent = gather->independent;
    p.wait_limit = g_wait_limit_cycles.load();
    p.c_ld = static_cast<int>(gather->n_total);
    p.c_col0 = gather->rank * n;
    p.done = reinterpret_cast<int*>(static_cast<uint8_t*>(ws) + counter_bytes - sizeof(int));
  }
  p.ndest = p.nranks;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TVB_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_w, map_a, p, NoGroup{}));
  return launched("qmm8_skinny", dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

template <int DT, int NT>
int launch_skinny(int device, cudaStream_t stream, const void* a, int64_t a_sm, const int8_t* b, const void* scales, void* c,
                  int m, int n, int k, int m0, const GatherTargets* gather = nullptr, const SkinnyAdds* adds = nullptr) {
  // Small weight matrices (a decoder's qkv, o and down projections) are cut into 128-row tiles: twice as many tiles, so half
  // as many CTAs share each and the completion of shared tiles, which dominates such short launches, is shorter. Large ones
  // keep 256-row tiles (fewer token fragments read per weight). Measured on a 32-layer stack: 4-6 % per decoding step.
  if constexpr (NT > 2) {
    // 32 or 64 rows of A in one pass (the weights streamed once): 128-row tiles whatever the matrix's size, which is what
    // the token fragments leave room for in registers and shared memory. (Bias and residual keep to passes of 16 rows.)
    if (adds != nullptr) return fail("tvb_qmm8: internal: wide passes carry no adds");
    return launch_skinny_cfg<DT, NT, 1, 8>(device, stream, a, a_sm, b, scales, c, m, n, k, m0, gather);
  } else {
    const bool small = static_cast<int64_t>(n) * k < (int64_t(64) << 20);
    if (adds != nullptr && gather == nullptr)
      return small ? launch_skinny_cfg<DT, NT, 1, 8, true>(device, stream, a, a_sm, b, scales, c, m, n, k, m0, nullptr, adds)
                   : launch_skinny_cfg<DT, NT, 2, 8, true>(device, stream, a, a_sm, b, scales, c, m, n, k, m0, nullptr, adds);
    if (small) return launch_skinny_cfg<DT, NT, 1, 8>(device, stream, a, a_sm, b, scales, c, m, n, k, m0, gather);
    return launch_skinny_cfg<DT, NT, 2, 8>(device, stream, a, a_sm, b, scales, c, m, n, k, m0, gather);
  }
}

// One product of a grouped launch as the host hands it over.
struct GroupItem {
  const void* a;
  int64_t a_sm;
  const int8_t* b;
  const void* scales;
  void* c[kMaxRanks];
  void* c_host;   // or NULL: one more destination, in page-locked host memory, laid out like the others
  int m;
};

// Several products of one shape (n, k) in one launch of the decode kernel, at most 16 rows of A each. `gather` as in
// launch_skinny_cfg (its c[] is not used: every item brings its own outputs); its products take consecutive numbers on
// the channel.
template <int DT, int NT, int RW>
int launch_skinny_group(int device, cudaStream_t stream, const GroupItem* items, int count, int n, int k, const GatherTargets* gather) {
  constexpr int NWARPS = 8;
  using Cfg = SkinnyCfg<NT, RW, NWARPS>;
  auto kernel = qmm8_skinny_kernel<DT, NT, RW, NWARPS, false, true>;
  {
    static std::mutex mutex;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> lock(mutex);
    if (!configured[device & 63]) {
      TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      configured[device & 63] = true;
    }
  }
  SkinnyGroup group{};
  group.count = count;
  const int nranks = gather != nullptr ? gather->world : 1;
  for (int g = 0; g < count; g++) {
    if (make_tensor_map_2d(&group.map_w[g], items[g].b, CU_TENSOR_MAP_DATA_TYPE_UINT8, k, n, k, kChunkK, Cfg::kRowsPerTile,
                           CU_TENSOR_MAP_SWIZZLE_128B) != 0)
      return -1;
    if (make_tensor_map_2d(&group.map_a[g], items[g].a, DT == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                           k, items[g].m, items[g].a_sm * 2, 64, Cfg::kTokens, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
      return -1;
    group.scales[g] = items[g].scales;
    group.m[g] = items[g].m;
    for (int r = 0; r < nranks; r++) group.c[g][r] = items[g].c[r];
    group.c[g][nranks] = items[g].c_host;
  }
  bool to_host = items[0].c_host != nullptr;
  for (int g = 0; g < count; g++)
    if ((items[g].c_host != nullptr) != to_host) return fail("tvb_qmm8_group: either every product has a host destination or none");
  SkinnyParams p{};
  p.tiles = static_cast<int>(ceil_div(n, Cfg::kRowsPerTile));
  p.chunks = k / kChunkK;
  const long long units = static_cast<long long>(p.tiles) * count * p.chunks;
  const int grid = static_cast<int>(std::min<long long>(sm_count(device), units));
  if (gather != nullptr && grid > static_cast<int>(kArriveWeight)) return fail("tvb_qmm8_group_gather: more than 1024 SMs");
  if (static_cast<long long>(p.tiles) * count > kMaxTiles) return fail("tvb_qmm8_group: more than 4 million output columns in all");
  const size_t partial_bytes = static_cast<size_t>(grid) * 2 * Cfg::kPartialFloats * sizeof(float);
  void* ws = nullptr;
  if (workspace(device, 0, kCounterBytes + partial_bytes, &ws) != 0) return -1;
  p.counters = static_cast<int*>(ws);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kCounterBytes);
  if (status_word(device, &p.status) != 0) return -1;
  p.nranks = 1;
  p.c_ld = n;
  p.c_col0 = 0;
  p.n = n;
  p.k = k;
  p.m0 = 0;
  if (gather != nullptr) {
    for (int r = 0; r < gather->world; r++) p.flags[r] = gather->flags[r];
    p.nranks = gather->world;
    p.rank = gather->rank;
    p.seq = gather->seq;
    p.independent = gather->independent;
    p.wait_limit = g_wait_limit_cycles.load();
    p.c_ld = static_cast<int>(gather->n_total);
    p.c_col0 = gather->rank * n;
    p.done = reinterpret_cast<int*>(static_cast<uint8_t*>(ws) + kCounterBytes - sizeof(int));
  }
  p.ndest = p.nranks + (to_host ? 1 : 0);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUtensorMap unused{};
  TVB_CUDA(cudaLaunchKernelEx(&cfg, kernel, unused, unused, p, group));
  return launched("qmm8_skinny(group)", dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

template <int DT>
int launch_group(int device, cudaStream_t stream, const GroupItem* items, int count, int n, int k, const GatherTargets* gather) {
  int rows = 0;
  for (int g = 0; g < count; g++) rows = std::max(rows, items[g].m);
  // tile height as for single products: by the size of one product's weights
  const bool small = static_cast<int64_t>(n) * k < (int64_t(64) << 20);
  if (rows <= 8)
    return small ? launch_skinny_group<DT, 1, 1>(device, stream, items, count, n, k, gather)
                 : launch_skinny_group<DT, 1, 2>(device, stream, items, count, n, k, gather);
  return small ? launch_skinny_group<DT, 2, 1>(device, stream, items, count, n, k, gather)
               : launch_skinny_group<DT, 2, 2>(device, stream, items, count, n, k, gather);
}

bool skinny_ok(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k) {
  return (dtype == TVB_BF16 || dtype == TVB_F16) && m <= 64 && k % kChunkK == 0 && k >= kChunkK &&
         (a_sm % 8 == 0 || m == 1) && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(b) & 15u) == 0 &&
         n >= 1;
}

// ------------------------------------------------------------------ sharded product: waiting for the peers' columns

// One warp waits (bounded, one arrival counter per lane) until every sharded product this rank has queued on the channel so
// far has arrived from every rank; a wait that runs out sets the status word and returns. The counters are added to by the
// peers' product kernels (and this rank's own) with system-scope reductions after a system-scope fence. Reads the product
// count, changes nothing: waiting twice is harmless.
__global__ void qmm8_wait_flags_kernel(const uint32_t* flags, int world, const uint32_t* seq_counter, int* status, long long limit) {
  // Launched with programmatic stream serialization. The next kernel of the stream may start its prologue at once (a
  // product kernel streams weights there); everything it does after its own griddepcontrol.wait comes after this kernel
  // has ended. This kernel in turn reads the product count only after the stream's earlier kernels have ended: every
  // kernel of such a chain waits, so "the previous kernel has ended" implies all earlier ones have.
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  const long long upto = static_cast<long long>(*reinterpret_cast<const volatile uint32_t*>(seq_counter)) - 1;
  const long long start = clock64();
  for (int spins = 0; !arrivals_complete_warp(flags, world, upto); spins++) {
    if ((spins & 63) == 63) {
      bool stop = *reinterpret_cast<volatile int*>(status) != 0;
      if (!stop && clock64() - start > limit) {
        atomicExch(status, 5);
        stop = true;
      }
      if (__any_sync(0xffffffffu, stop)) break;
    }
  }
}

// ------------------------------------------------------------------ the same kernel without any allocation
//
// Scratch for tvb_qmm8_static_scratch: the tile counters, then the per-CTA partial sums, then a status word, in one
// array that is part of the library's image (so every GPU that loads the library carries it until the process exits).
constexpr int kStaticMaxCtas = 160;    // CTAs of one launch = SMs of the device
constexpr int kStaticMaxTiles = 4096;  // 256-row tiles: n up to 1 048 576
constexpr size_t kStaticCounterBytes = static_cast<size_t>(kStaticMaxTiles) * sizeof(int);
constexpr size_t kStaticPartialBytes = static_cast<size_t>(kStaticMaxCtas) * 2 * SkinnyCfg<2, 2, 8>::kPartialFloats * sizeof(float);
constexpr size_t kStaticScratchBytes = kStaticCounterBytes + kStaticPartialBytes + 256;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mutex;
void* g_static_scratch_ptr[64] = {};   // per device: the array's device address (the symbol itself is not one)
bool g_static_configured[64][4] = {};

// The device address of g_static_scratch on `device` (which must be current). Looked up once per device.
int static_scratch_address(int device, unsigned char** out) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return fail_cuda("cudaGetSymbolAddress(g_static_scratch)", err);
    g_static_scratch_ptr[device] = ptr;
  }
  *out = static_cast<unsigned char*>(g_static_scratch_ptr[device]);
  return 0;
}

template <int DT, int NT>
int launch_skinny_static(int device, int sms, cudaStream_t stream, unsigned char* scratch, const void* a, int64_t a_sm,
                         const int8_t* b, const void* scales, void* c, int m, int n, int k, int m0) {
  constexpr int RW = 2, NWARPS = 8;
  using Cfg = SkinnyCfg<NT, RW, NWARPS>;
  auto kernel = qmm8_skinny_kernel<DT, NT, RW, NWARPS>;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    bool& done = g_static_configured[device][(DT == TVB_BF16 ? 0 : 2) + (NT - 1)];
    if (!done) {
      TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      done = true;
    }
  }
  CUtensorMap map_w, map_a;
  if (make_tensor_map_2d(&map_w, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, k, n, k, kChunkK, Cfg::kRowsPerTile,
                         CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  if (make_tensor_map_2d(&map_a, a, DT == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, m,
                         a_sm * 2, 64, Cfg::kTokens, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  SkinnyParams p{};
  p.tiles = static_cast<int>(ceil_div(n, Cfg::kRowsPerTile));
  p.chunks = k / kChunkK;
  const long long units = static_cast<long long>(p.tiles) * p.chunks;
  const int grid = static_cast<int>(std::min<long long>(sms, units));
  p.counters = reinterpret_cast<int*>(scratch);
  p.partials = reinterpret_cast<float*>(scratch + kStaticCounterBytes);
  p.status = reinterpret_cast<int*>(scratch + kStaticCounterBytes + kStaticPartialBytes);
  p.scales = scales;
  p.c[0] = c;
  p.nranks = 1;
  p.ndest = 1;
  p.c_ld = n;
  p.c_col0 = 0;
  p.m = m;
  p.n = n;
  p.k = k;
  p.m0 = m0;
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_w, map_a, p, NoGroup{});
  return launched("qmm8_skinny(static scratch)", dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" int tvb_qmm8_static_scratch(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                                       void* c, int64_t m, int64_t n, int64_t k, void* stream_handle) {
  TVB_REQUIRE(device >= 0 && device < 64, "tvb_qmm8_static_scratch: device index out of range");
  TVB_REQUIRE(dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8_static_scratch: A must be float16 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0 && k >= 0, "tvb_qmm8_static_scratch: negative size");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(a != nullptr && b != nullptr && scales != nullptr && c != nullptr, "tvb_qmm8_static_scratch: NULL pointer");
  TVB_REQUIRE(m <= 64, "tvb_qmm8_static_scratch: at most 64 rows of A (the decode kernel); use tvb_qmm8 beyond");
  TVB_REQUIRE(skinny_ok(a, dtype, a_sm, b, m, n, k),
              "tvb_qmm8_static_scratch: needs k a multiple of 128 and 16-byte aligned A rows and B; use tvb_qmm8 otherwise");
  TVB_REQUIRE(n <= static_cast<int64_t>(kStaticMaxTiles) * 256 && k < (int64_t(1) << 31),
              "tvb_qmm8_static_scratch: n exceeds the built-in scratch (1 048 576 output columns at most); use tvb_qmm8");
  TVB_CUDA(cudaSetDevice(device));
  int sms = 0;
  TVB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  TVB_REQUIRE(sms >= 1 && sms <= kStaticMaxCtas,
              "tvb_qmm8_static_scratch: this GPU has more SMs than the built-in scratch was sized for (160); use tvb_qmm8");
  unsigned char* scratch = nullptr;
  if (static_scratch_address(device, &scratch) != 0) return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  // The array keeps whatever the previous call left: the counters and the status word must start at zero.
  const int64_t tiles = ceil_div(n, 256);
  TVB_CUDA(cudaMemsetAsync(scratch, 0, static_cast<size_t>(tiles) * sizeof(int), stream));
  TVB_CUDA(cudaMemsetAsync(scratch + kStaticCounterBytes + kStaticPartialBytes, 0, sizeof(int), stream));
  const int mi = static_cast<int>(m), ni = static_cast<int>(n), ki = static_cast<int>(k);
  const int64_t stride = m == 1 ? k : a_sm;
  for (int m0 = 0; m0 < mi; m0 += 16) {
    const int rows = mi - m0;
    int rc;
    if (dtype == TVB_BF16)
      rc = rows <= 8 ? launch_skinny_static<TVB_BF16, 1>(device, sms, stream, scratch, a, stride, b, scales, c, mi, ni, ki, m0)
                     : launch_skinny_static<TVB_BF16, 2>(device, sms, stream, scratch, a, stride, b, scales, c, mi, ni, ki, m0);
    else
      rc = rows <= 8 ? launch_skinny_static<TVB_F16, 1>(device, sms, stream, scratch, a, stride, b, scales, c, mi, ni, ki, m0)
                     : launch_skinny_static<TVB_F16, 2>(device, sms, stream, scratch, a, stride, b, scales, c, mi, ni, ki, m0);
    if (rc != 0) return rc;
  }
  return 0;
}

extern "C" int tvb_qmm8_static_scratch_status(int device, void* stream_handle, int* host_out) {
  TVB_REQUIRE(device >= 0 && device < 64, "tvb_qmm8_static_scratch_status: device index out of range");
  TVB_REQUIRE(host_out != nullptr, "tvb_qmm8_static_scratch_status: NULL pointer");
  TVB_CUDA(cudaSetDevice(device));
  unsigned char* scratch = nullptr;
  if (static_scratch_address(device, &scratch) != 0) return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  int word = 0;
  TVB_CUDA(cudaMemcpyAsync(&word, scratch + kStaticCounterBytes + kStaticPartialBytes, sizeof(int), cudaMemcpyDeviceToHost, stream));
  TVB_CUDA(cudaStreamSynchronize(stream));
  *host_out = word;
  return 0;
}

extern "C" int tvb_set_wait_limit_ms(int ms) {
  TVB_REQUIRE(ms >= 1 && ms <= 60000, "tvb_set_wait_limit_ms: 1 to 60000 milliseconds");
  g_wait_limit_cycles.store(static_cast<long long>(ms) * 2000000ll);  // (at most ~2 GHz of SM clock)
  return 0;
}

// One pass of the decode kernel over `rows` rows of A from row m0 on (rows <= 8, 16, 32, 64 pick the token count).
template <int DT>
static int skinny_pass(int device, cudaStream_t stream, const void* a, int64_t stride, const int8_t* b, const void* scales, void* c,
                       int mi, int ni, int ki, int m0, int rows, const GatherTargets* gather, const SkinnyAdds* adds) {
  if (rows <= 8) return launch_skinny<DT, 1>(device, stream, a, stride, b, scales, c, mi, ni, ki, m0, gather, adds);
  if (rows <= 16) return launch_skinny<DT, 2>(device, stream, a, stride, b, scales, c, mi, ni, ki, m0, gather, adds);
  if (rows <= 32) return launch_skinny<DT, 4>(device, stream, a, stride, b, scales, c, mi, ni, ki, m0, gather, adds);
  return launch_skinny<DT, 8>(device, stream, a, stride, b, scales, c, mi, ni, ki, m0, gather, adds);
}

// Rows of A per pass: 16 with bias or residual in the epilogue, else up to 64 (one pass streams the weights once).
static int pass_rows(int m, const SkinnyAdds* adds) { return adds != nullptr || m <= 16 ? 16 : 64; }

extern "C" int tvb_qmm8_gather(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                               void* const* c_ranks, uint32_t* const* flag_ranks, int world, int rank, uint32_t* seq_counter,
                               int independent, int64_t m, int64_t n_local, int64_t k) {
  TVB_REQUIRE(independent >= 0 && independent <= 3, "tvb_qmm8_gather: independent must be between 0 and 3");
  TVB_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "tvb_qmm8_gather: 1 to 8 ranks");
  TVB_REQUIRE(dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8_gather: A must be float16 or bfloat16");
  TVB_REQUIRE(m >= 1 && m <= 64 && n_local >= 1 && k >= 1, "tvb_qmm8_gather: 1 <= m <= 64 (the decode kernel)");
  TVB_REQUIRE(a != nullptr && b != nullptr && scales != nullptr && c_ranks != nullptr && flag_ranks != nullptr &&
                  seq_counter != nullptr,
              "tvb_qmm8_gather: NULL pointer");
  TVB_REQUIRE(skinny_ok(a, dtype, a_sm, b, m, n_local, k), "tvb_qmm8_gather: needs k a multiple of 128 and 16-byte aligned A rows and B");
  TVB_REQUIRE(n_local * world < (int64_t(1) << 31), "tvb_qmm8_gather: sizes beyond 32 bits");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  GatherTargets g{};
  for (int r = 0; r < world; r++) {
    TVB_REQUIRE(c_ranks[r] != nullptr && flag_ranks[r] != nullptr, "tvb_qmm8_gather: NULL buffer of a rank");
    g.c[r] = c_ranks[r];
    g.flags[r] = flag_ranks[r];
  }
  g.world = world;
  g.rank = rank;
  g.seq = seq_counter;
  g.n_total = n_local * world;
  const int mi = static_cast<int>(m), ni = static_cast<int>(n_local), ki = static_cast<int>(k);
  const int64_t stride = m == 1 ? k : a_sm;
  // up to 64 rows of A per pass; every pass is a product of its own on the channel (it counts and is waited for like one)
  const int step = pass_rows(mi, nullptr);
  const int passes = static_cast<int>(ceil_div(mi, step));
  for (int m0 = 0, pass = 0; m0 < mi; m0 += step, pass++) {
    const int rows = std::min(step, mi - m0);
    // (the passes of one product do not depend on each other: pass i need not wait for the i passes before it either)
    g.independent = static_cast<uint32_t>(std::min(independent * passes + pass, kArriveSlots - 1));
    const int rc = dtype == TVB_BF16 ? skinny_pass<TVB_BF16>(device, stream, a, stride, b, scales, g.c[rank], mi, ni, ki, m0, rows, &g, nullptr)
                                     : skinny_pass<TVB_F16>(device, stream, a, stride, b, scales, g.c[rank], mi, ni, ki, m0, rows, &g, nullptr);
    if (rc != 0) return rc;
  }
  return 0;
}

// ------------------------------------------------------------------ several products of one shape in one launch

static int group_products(const char* who, int device, int dtype, const TvbGroupItem* items, int count, uint32_t* const* flag_ranks,
                          int world, int rank, uint32_t* seq_counter, int independent, int64_t n, int64_t k, bool sharded) {
  TVB_REQUIRE(items != nullptr && count >= 1 && count <= kMaxGroup, std::string(who) + ": 1 to 4 products");
  TVB_REQUIRE(dtype == TVB_F16 || dtype == TVB_BF16, std::string(who) + ": A must be float16 or bfloat16");
  TVB_REQUIRE(n >= 1 && k >= 1 && n * world < (int64_t(1) << 31), std::string(who) + ": bad sizes");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  GroupItem host[kMaxGroup] = {};
  for (int g = 0; g < count; g++) {
    const TvbGroupItem& it = items[g];
    TVB_REQUIRE(it.m >= 1 && it.m <= 16, std::string(who) + ": 1 <= m <= 16 for every product");
    TVB_REQUIRE(it.a != nullptr && it.b != nullptr && it.scales != nullptr && it.c_ranks != nullptr, std::string(who) + ": NULL pointer");
    TVB_REQUIRE(skinny_ok(it.a, dtype, it.a_sm, it.b, it.m, n, k), std::string(who) + ": needs k a multiple of 128 and 16-byte aligned A rows and B");
    host[g].a = it.a;
    host[g].a_sm = it.m == 1 ? k : it.a_sm;
    host[g].b = it.b;
    host[g].scales = it.scales;
    host[g].m = static_cast<int>(it.m);
    host[g].c_host = it.c_host;
    for (int r = 0; r < world; r++) {
      TVB_REQUIRE(it.c_ranks[r] != nullptr, std::string(who) + ": NULL output buffer");
      host[g].c[r] = it.c_ranks[r];
    }
  }
  GatherTargets gt{};
  if (sharded) {
    // the launch's products and the `independent` products before them report in different slots of the channel
    TVB_REQUIRE(independent >= 0 && independent + count <= kArriveSlots, std::string(who) + ": independent + count must not exceed 4");
    for (int r = 0; r < world; r++) {
      TVB_REQUIRE(flag_ranks[r] != nullptr, std::string(who) + ": NULL counters of a rank");
      gt.flags[r] = flag_ranks[r];
    }
    gt.world = world;
    gt.rank = rank;
    gt.seq = seq_counter;
    gt.independent = static_cast<uint32_t>(independent);
    gt.n_total = n * world;
  }
  const int ni = static_cast<int>(n), ki = static_cast<int>(k);
  return dtype == TVB_BF16 ? launch_group<TVB_BF16>(device, stream, host, count, ni, ki, sharded ? &gt : nullptr)
                           : launch_group<TVB_F16>(device, stream, host, count, ni, ki, sharded ? &gt : nullptr);
}

extern "C" int tvb_qmm8_group(int device, int dtype, const TvbGroupItem* items, int count, int64_t n, int64_t k) {
  return group_products("tvb_qmm8_group", device, dtype, items, count, nullptr, 1, 0, nullptr, 0, n, k, false);
}

extern "C" int tvb_qmm8_group_gather(int device, int dtype, const TvbGroupItem* items, int count, uint32_t* const* flag_ranks, int world,
                                     int rank, uint32_t* seq_counter, int independent, int64_t n_local, int64_t k) {
  TVB_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "tvb_qmm8_group_gather: 1 to 8 ranks");
  TVB_REQUIRE(flag_ranks != nullptr && seq_counter != nullptr, "tvb_qmm8_group_gather: NULL pointer");
  return group_products("tvb_qmm8_group_gather", device, dtype, items, count, flag_ranks, world, rank, seq_counter, independent, n_local,
                        k, true);
}

extern "C" int tvb_wait_flags(int device, const uint32_t* flags, int world, const uint32_t* seq_counter) {
  TVB_REQUIRE(flags != nullptr && seq_counter != nullptr && world >= 1 && world <= kMaxRanks, "tvb_wait_flags: bad arguments");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  int* status = nullptr;
  if (status_word(device, &status) != 0) return -1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TVB_CUDA(cudaLaunchKernelEx(&cfg, qmm8_wait_flags_kernel, flags, world, seq_counter, status, g_wait_limit_cycles.load()));
  return launched("qmm8_wait_flags", dim3(1), dim3(32), 0, stream);
}

// The decode kernel over all rows of A.
static int skinny_passes(int device, cudaStream_t stream, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                         void* c, int mi, int ni, int ki, const SkinnyAdds* adds) {
  const int64_t stride = mi == 1 ? ki : a_sm;  // (one row: any stride will do for the map)
  const int step = pass_rows(mi, adds);
  for (int m0 = 0; m0 < mi; m0 += step) {
    const int rows = std::min(step, mi - m0);
    const int rc = dtype == TVB_BF16 ? skinny_pass<TVB_BF16>(device, stream, a, stride, b, scales, c, mi, ni, ki, m0, rows, nullptr, adds)
                                     : skinny_pass<TVB_F16>(device, stream, a, stride, b, scales, c, mi, ni, ki, m0, rows, nullptr, adds);
    if (rc != 0) return rc;
  }
  return 0;
}

extern "C" int tvb_qmm8(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales, void* c,
                        int64_t m, int64_t n, int64_t k, int variant) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8: A must be float32, float16 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0 && k >= 0, "tvb_qmm8: negative size");
  TVB_REQUIRE(m < (int64_t(1) << 31) && n < (int64_t(1) << 31) && k < (int64_t(1) << 31) && n * k < (int64_t(1) << 40),
              "tvb_qmm8: sizes beyond 32 bits");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(c != nullptr && scales != nullptr && (k == 0 || (a != nullptr && b != nullptr)), "tvb_qmm8: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  int mi = static_cast<int>(m), ni = static_cast<int>(n), ki = static_cast<int>(k);
  bool can_skinny = skinny_ok(a, dtype, a_sm, b, m, n, k);
  TVB_REQUIRE(variant != 2 || can_skinny,
              "tvb_qmm8: the skinny kernel needs 16-bit A, m <= 64, k a multiple of 128, 16-byte aligned rows");
  TVB_REQUIRE(variant >= 0 && variant <= 5, "tvb_qmm8: unknown kernel variant");
  const bool can_f32_tc = qmm8_f32_tc_usable(a, dtype, a_sm, b, m, n, k);
  TVB_REQUIRE(variant != 5 || can_f32_tc,
              "tvb_qmm8: the float32 tensor-core kernel needs float32 A, at most 256 rows, k a multiple of 64, 16-byte aligned B");
  if (variant == 5 || (variant == 0 && can_f32_tc))
    return qmm8_f32_tc(device, stream, static_cast<const float*>(a), a_sm, b, static_cast<const float*>(scales), static_cast<float*>(c), m, n, k);
  const bool can_tc = qmm8_tc_usable(a, dtype, a_sm, b, m, n, k);
  TVB_REQUIRE(variant != 3 || can_tc, "tvb_qmm8: the tcgen05 kernel needs 16-bit A, k a multiple of 16, 16-byte aligned rows");
  const bool can_widen = qmm8_widen_gemm_usable(a, dtype, a_sm, b, m, n, k);
  TVB_REQUIRE(variant != 4 || can_widen, "tvb_qmm8: the widened GEMM needs 16-bit A, k a multiple of 16, 16-byte aligned rows");
  // the extra pass over the weights pays for itself from about 730 rows on (874 against 1237 TFLOP/s, 3 bytes per weight)
  if (variant == 4 || (variant == 0 && can_widen && m >= 1024))
    return qmm8_widen_gemm(device, stream, a, dtype, a_sm, b, scales, c, m, n, k);
  // up to 64 rows: one pass of the decode kernel (32 or 64 token columns per MMA row block) streams the weights once and
  // beats a 128-row tensor-core tile, which is mostly padding at these sizes
  const bool decode_pass = can_skinny && m <= 64;
  if (variant == 3 || (variant == 0 && can_tc && m > 16 && !decode_pass))
    return qmm8_tc(device, stream, a, dtype, m == 1 ? k : a_sm, b, scales, c, m, n, k);
  if (variant == 2 || (variant == 0 && can_skinny)) return skinny_passes(device, stream, a, dtype, a_sm, b, scales, c, mi, ni, ki, nullptr);
  if (dtype == TVB_F32 && variant == 0 && k % 16 == 0 && (a_sm % 4 == 0 || m == 1) && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
      (reinterpret_cast<uintptr_t>(b) & 15u) == 0) {
    // float32 A with aligned rows; row passes side by side in the grid (the weights of a typical layer stay in L2 between them)
    dim3 grid(static_cast<unsigned>(ceil_div(n, 8 * kF32Cols)), static_cast<unsigned>(std::min<int64_t>(ceil_div(m, kF32Rows), 64)));
    qmm8_f32_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(a), m == 1 ? k : a_sm, b, static_cast<const float*>(scales),
                                              static_cast<float*>(c), mi, ni, ki);
    return launched("qmm8_f32", grid, dim3(256), 0, stream);
  }
  switch (dtype) {
    case TVB_F32: return launch_plain<TVB_F32>(stream, a, a_sm, b, scales, c, mi, ni, ki);
    case TVB_F16: return launch_plain<TVB_F16>(stream, a, a_sm, b, scales, c, mi, ni, ki);
    default: return launch_plain<TVB_BF16>(stream, a, a_sm, b, scales, c, mi, ni, ki);
  }
}

extern "C" int tvb_qmm8_linear(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                               const void* bias, const void* residual, void* c, int64_t m, int64_t n, int64_t k) {
  if (bias == nullptr && residual == nullptr) return tvb_qmm8(device, a, dtype, a_sm, b, scales, c, m, n, k, 0);
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8_linear: A must be float32, float16 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0 && k >= 0 && m < (int64_t(1) << 31) && n < (int64_t(1) << 31) && k < (int64_t(1) << 31),
              "tvb_qmm8_linear: bad size");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(c != nullptr && scales != nullptr && (k == 0 || (a != nullptr && b != nullptr)), "tvb_qmm8_linear: NULL pointer");
  // at most 32 rows in a shape the decode kernel takes: the adds happen where the product is finished
  if (skinny_ok(a, dtype, a_sm, b, m, n, k) && m <= 32) {
    cudaStream_t stream;
    if (enter(device, &stream) != 0) return -1;
    const SkinnyAdds adds{bias, residual};
    return skinny_passes(device, stream, a, dtype, a_sm, b, scales, c, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
                         &adds);
  }
  // any other shape: the product, then one pass per operand (the same roundings)
  TVB_REQUIRE(residual != c, "tvb_qmm8_linear: the output may take the residual's place only where the decode kernel runs");
  int rc = tvb_qmm8(device, a, dtype, a_sm, b, scales, c, m, n, k, 0);
  if (rc == 0 && bias != nullptr) rc = tvb_add_rowvec(device, c, dtype, n, bias, dtype, m, n);
  if (rc == 0 && residual != nullptr) rc = tvb_add_rowvec(device, c, dtype, m * n, residual, dtype, 1, m * n);
  return rc;
}

// The tcgen05 GEMM main loop shared by the large-m kernels of this library:
// D[m, n] = A[m, k] . B[n, k]^T with both operands K-major in global memory.
//
// One persistent CTA per SM walks BM x BN output tiles, BM = 128 or 256. Warp roles (E = BM / 32 epilogue warps):
//   warp E, one lane: TMA producer. Fills a ring of shared-memory stages, each holding a
//            BM-row slice of A and a BN-row slice of B, 128 bytes of k wide, written by
//            cp.async.bulk.tensor with the 128-byte swizzle (each CTA loads for itself only).
//   warp E+1, one lane: issues tcgen05.mma (per stage four steps of 32 bytes of k, each step one MMA per 128 rows
//            of the tile) into TMEM accumulators (BN columns of float32 / int32 per 128 rows), and
//            tcgen05.commit's each stage back to the producer and each finished tile to the
//            epilogue. The warp also owns the TMEM allocation.
//   warps 0..E-1: epilogue. Each warp reads its 32 TMEM lanes (one output row per thread)
//            32 columns at a time with tcgen05.ld and hands them to the Epilogue policy.
// BM = 128: two accumulator buffers, so the MMA warp already works on the next tile while a tile is read back.
// BM = 256: both 128-row halves share every B stage, which cuts the operand bytes per MMA by a third: the ring then
//            covers the latency of the copies (with 128 rows it does not, and the tensor pipe idles ~40 % of the time);
//            the accumulators fill the whole tensor memory, so a tile's read-back is not overlapped.
// All mbarrier waits are bounded (ptx::mbar_wait); a wait that runs out makes every role
// leave its loop, the TMEM allocation is released, and the status word tells the host.
#pragma once

#include <cuda.h>

#include "ptx.cuh"

namespace tvb {

struct GemmTcShape {
  int m, n;
  int kblocks;       // ceil(k bytes / kGemmStageK)
  int k_elems_per_block;  // kGemmStageK for 8-bit operands, half of it for 16-bit
  int tiles_m, tiles_n;
  int band;           // tile rows per band of the tile order (gemm_tile_coords)
};

// Bytes of k per shared-memory stage: 128 (128-byte swizzle, four MMAs per stage). 64 (64-byte swizzle, twice as many
// stages in the same shared memory) is supported by the code below and was measured 15 % slower on 8192^3 float8.
constexpr int kGemmStageK = 128;

template <int BN, int EPI_SMEM, int BM = 128>
struct GemmTcCfg {
  static_assert(BM == 128 || BM == 256, "tiles are 128 or 256 rows");
  static constexpr int kBM = BM;
  static constexpr int kHalves = BM / 128;        // MMAs per k step (one per 128 rows)
  static constexpr int kEpiWarps = BM / 32;
  static constexpr int kStageA = kBM * kGemmStageK, kStageB = BN * kGemmStageK, kStage = kStageA + kStageB;
  // (an epilogue's shared memory beyond 8 KB comes on top of the budget: the 128-row configuration has room to spare)
  static constexpr int kBudget = (BM == 128 ? 200 : 224) * 1024 - (EPI_SMEM < 8192 ? EPI_SMEM : 8192);
  static constexpr int kStages = kBudget / kStage < 8 ? kBudget / kStage : 8;
  static constexpr int kThreads = (kEpiWarps + 2) * 32;
  static constexpr int kAccCols = kHalves * BN;   // TMEM columns of one tile's accumulators
  static constexpr int kAccBufs = 2 * kAccCols <= 512 ? 2 : 1;
  static constexpr int kWant = kAccBufs * kAccCols;
  static constexpr int kTmemCols = kWant <= 32 ? 32 : (kWant <= 64 ? 64 : (kWant <= 128 ? 128 : (kWant <= 256 ? 256 : 512)));
  static_assert(kWant <= 512, "the accumulators do not fit the tensor memory");
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStage + 1024 + kBarBytes + EPI_SMEM;
  static_assert(kSmemBytes <= 227 * 1024, "more shared memory than a CTA may have");
};

// Tile order: bands of `band` tile rows, walked column by column, so that the ~148 tiles in flight at any time cover a
// near-square patch of the output and share operand panels in L2 (band * BM rows of A against 148 / band * BN rows of B;
// the two are about equal for band = 16 with 128 x 256 tiles and 12 with 256 x 256 tiles).
__device__ __forceinline__ void gemm_tile_coords(int tile, int tiles_m, int tiles_n, int band, int& tm, int& tn) {
  const int per_band = band * tiles_n;
  const int b = tile / per_band;
  const int first = b * band;
  const int rows = tiles_m - first < band ? tiles_m - first : band;
  const int r = tile - b * per_band;
  tm = first + r % rows;
  tn = r / rows;
}

// Epilogue policy interface:
//   struct Params;                       kernel parameters of the epilogue
//   static constexpr int kSmemBytes;     per-CTA shared memory of the epilogue
//   __device__ static void begin_tile(const Params&, uint8_t* smem, int row0, int col0, int m, int n, int tid);
//       called by all 128 epilogue threads before a tile's loads (they synchronise inside as needed)
//   __device__ static void store(const Params&, const uint8_t* smem, int row, int col_tile0, int col_off,
//                                const uint32_t (&acc)[32], int m, int n);
//       thread `row`'s 32 accumulators for columns col_tile0 + col_off ... + 31
//   __device__ static void kernel_begin(const Params&, int tid);  __device__ static void kernel_end(const Params&, int tid, bool ok);
//       called by all epilogue threads before the first tile and after the last (what a sharded product does around its
//       stores: wait for the channel's earlier products, report this CTA's columns as delivered)
template <int KIND, int BN, class Epi, int BM = 128>
__global__ void __launch_bounds__((BM / 32 + 2) * 32, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmTcShape sh,
                   const uint32_t idesc, const typename Epi::Params ep, int* status) {
  using Cfg = GemmTcCfg<BN, Epi::kSmemBytes, BM>;
  constexpr int kProducerWarp = Cfg::kEpiWarps, kMmaWarp = Cfg::kEpiWarps + 1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + Cfg::kStages * Cfg::kStage);
  const uint32_t full0 = ptx::smem_u32(bars), empty0 = full0 + 8 * Cfg::kStages;
  const uint32_t tfull0 = empty0 + 8 * Cfg::kStages, tempty0 = tfull0 + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_smem = base_ptr + Cfg::kStages * Cfg::kStage + Cfg::kBarBytes;
  static_assert((2 * 8 + 4) * 8 + 8 <= Cfg::kBarBytes, "barrier area too small");
  static_assert(Cfg::kStages >= 2 && Cfg::kStages <= 8, "stage count out of range");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(tfull0 + 8 * a, 1);
      ptx::mbar_init(tempty0 + 8 * a, Cfg::kEpiWarps * 32);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) ptx::tmem_alloc(ptx::smem_u32(tmem_slot), Cfg::kTmemCols);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = sh.tiles_m * sh.tiles_n;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_a);
      ptx::prefetch_tensormap(&map_b);
      long long it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int tm, tn;
        gemm_tile_coords(tile, sh.tiles_m, sh.tiles_n, sh.band, tm, tn);
        for (int kb = 0; kb < sh.kblocks; kb++, it++) {
          const int s = static_cast<int>(it % Cfg::kStages);
          const uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
          ok = ptx::mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t dst = base + s * Cfg::kStage;
          ptx::mbar_expect_tx(full0 + 8 * s, Cfg::kStage);
          ptx::tma_load_2d(dst, &map_a, kb * sh.k_elems_per_block, tm * Cfg::kBM, full0 + 8 * s);
          ptx::tma_load_2d(dst + Cfg::kStageA, &map_b, kb * sh.k_elems_per_block, tn * BN, full0 + 8 * s);
        }
      }
      // no copy may still be in flight when the CTA's shared memory is released
      const long long first = it > Cfg::kStages ? it - Cfg::kStages : 0;
      for (long long j = first; j < it; j++) {
        volatile int never = 0;
        ptx::mbar_wait(full0 + 8 * static_cast<int>(j % Cfg::kStages), static_cast<uint32_t>((j / Cfg::kStages) & 1), &never);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      long long it = 0;
      int titer = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, titer++) {
        const int acc = titer % Cfg::kAccBufs;
        const uint32_t aph = static_cast<uint32_t>((titer / Cfg::kAccBufs) & 1);
        ok = ptx::mbar_wait(tempty0 + 8 * acc, aph ^ 1u, abort_flag);  // the epilogue has drained this buffer
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccCols);
        for (int kb = 0; kb < sh.kblocks; kb++, it++) {
          const int s = static_cast<int>(it % Cfg::kStages);
          const uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
          ok = ptx::mbar_wait(full0 + 8 * s, ph, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint64_t a_desc = kGemmStageK == 64 ? ptx::tc_smem_desc_sw64(base + s * Cfg::kStage) : ptx::tc_smem_desc_sw128(base + s * Cfg::kStage);
          const uint64_t b_desc = kGemmStageK == 64 ? ptx::tc_smem_desc_sw64(base + s * Cfg::kStage + Cfg::kStageA)
                                                    : ptx::tc_smem_desc_sw128(base + s * Cfg::kStage + Cfg::kStageA);
#pragma unroll
          for (int j = 0; j < kGemmStageK / 32; j++)  // 32 bytes of k per instruction: +2 in the descriptor's 16-byte units
#pragma unroll
            for (int h = 0; h < Cfg::kHalves; h++)  // rows 128 h ... of the tile: 128 * 128 bytes further into the A stage
              ptx::tc_mma<KIND>(d_tmem + h * BN, a_desc + (h * 128 * kGemmStageK >> 4) + 2 * j, b_desc + 2 * j, idesc,
                                (kb | j) != 0 ? 1u : 0u);
          ptx::tc_commit(empty0 + 8 * s);
        }
        if (ok) ptx::tc_commit(tfull0 + 8 * acc);
      }
    }
    __syncwarp();
  } else {
    int titer = 0;
    bool ok = true;
    Epi::kernel_begin(ep, threadIdx.x);
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, titer++) {
      int tm, tn;
      gemm_tile_coords(tile, sh.tiles_m, sh.tiles_n, sh.band, tm, tn);
      const int acc = titer % Cfg::kAccBufs;
      const uint32_t aph = static_cast<uint32_t>((titer / Cfg::kAccBufs) & 1);
      Epi::begin_tile(ep, epi_smem, tm * Cfg::kBM, tn * BN, sh.m, sh.n, threadIdx.x);
      ok = ptx::mbar_wait(tfull0 + 8 * acc, aph, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      // warp w reads TMEM lanes 32 (w % 4) ...; warps 4-7 (256-row tiles) the second half's accumulators, BN columns on
      const int half = warp >> 2;
      const int row = tm * Cfg::kBM + warp * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                             static_cast<uint32_t>(acc * Cfg::kAccCols + half * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        Epi::store(ep, epi_smem, row, tn * BN, c * 32, r, sh.m, sh.n);
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(tempty0 + 8 * acc);
    }
    Epi::kernel_end(ep, threadIdx.x, ok);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(status, 2);
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace tvb

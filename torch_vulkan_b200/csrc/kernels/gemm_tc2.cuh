// The tcgen05 GEMM main loop for a pair of CTAs on one 256 x 256 output tile (tcgen05.mma cta_group::2):
// D[m, n] = A[m, k] . B[n, k]^T with both operands K-major in global memory.
//
// A cluster of two CTAs (two SMs of one TPC) walks 256 x 256 tiles. CTA r of the pair loads rows 128 r ... of the
// tile's A slice and rows 128 r ... of its B slice (each CTA for itself: plain cp.async.bulk.tensor, no multicast), 128
// bytes of k per stage. One lane of the leader (CTA 0) issues the MMAs for both: an instruction multiplies the 256 rows of
// A that the two CTAs hold by the 256 rows of B that the two CTAs hold, and each CTA's tensor memory receives the
// accumulators of its own 128 rows of the tile, 256 columns wide. Compared with one CTA on a 256 x 256 tile, every SM
// stages half of B (32 KB per stage instead of 64 KB: six stages instead of three) and its accumulators take half of the
// tensor memory, so the read-back of a tile runs under the next tile's MMAs.
//
// Barriers (all in shared memory, the same offsets in both CTAs):
//   full[s]   (leader's only) one arrival by the leader's producer with the byte count of both CTAs' boxes; the peer's
//             copies report to the leader's barrier (cp.async.bulk.tensor with .cta_group::2).
//   empty[s]  each CTA's own, signalled in both CTAs by the leader's tcgen05.commit.
//   tfull[b]  each CTA's own, signalled in both CTAs by the leader's commit after a tile's last MMA.
//   tempty[b] (leader's only) one arrival per epilogue warp of either CTA (the peer's arrive remotely).
// All mbarrier waits are bounded; the CTAs of a pair leave through a cluster barrier, after which both free their tensor
// memory, so neither is gone while the other may still signal it or read its shared memory.
#pragma once

#include <cuda.h>

#include "gemm_tc.cuh"
#include "ptx_pair.cuh"

namespace tvb {

template <int EPI_SMEM>
struct GemmTc2Cfg {
  static constexpr int kRows = 128;    // rows of A, and of B, that one CTA stages
  static constexpr int kTile = 256;    // the pair's tile is kTile x kTile
  static constexpr int kEpiWarps = 4;
  static constexpr int kStageA = kRows * kGemmStageK, kStageB = kRows * kGemmStageK, kStage = kStageA + kStageB;
  static constexpr int kBudget = 208 * 1024 - (EPI_SMEM < 8192 ? EPI_SMEM : 8192);
  static constexpr int kStages = kBudget / kStage < 8 ? kBudget / kStage : 8;
  static constexpr int kThreads = (kEpiWarps + 2) * 32;
  static constexpr int kAccCols = kTile;  // float32 columns of one tile's accumulators in each CTA
  static constexpr int kAccBufs = 2;
  static constexpr int kTmemCols = 512;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStage + 1024 + kBarBytes + EPI_SMEM;
  static_assert(kSmemBytes <= 227 * 1024, "more shared memory than a CTA may have");
};

template <int KIND, class Epi>
__global__ void __launch_bounds__(192, 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmTcShape sh,
                    const uint32_t idesc, const typename Epi::Params ep, int* status) {
  using Cfg = GemmTc2Cfg<Epi::kSmemBytes>;
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
  const uint32_t rank = ptx::cluster_ctarank();  // 0: the leader, which issues the MMAs
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(tfull0 + 8 * a, 1);
      ptx::mbar_init(tempty0 + 8 * a, 2 * Cfg::kEpiWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), Cfg::kTmemCols);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // both CTAs' barriers exist before either signals the other's
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = sh.tiles_m * sh.tiles_n;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_a);
      ptx::prefetch_tensormap(&map_b);
      long long it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        int tm, tn;
        gemm_tile_coords(tile, sh.tiles_m, sh.tiles_n, sh.band, tm, tn);
        const int row_a = tm * Cfg::kTile + static_cast<int>(rank) * Cfg::kRows;
        const int row_b = tn * Cfg::kTile + static_cast<int>(rank) * Cfg::kRows;
        for (int kb = 0; kb < sh.kblocks; kb++, it++) {
          const int s = static_cast<int>(it % Cfg::kStages);
          const uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
          ok = ptx::mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t dst = base + s * Cfg::kStage;
          if (rank == 0) ptx::mbar_expect_tx(full0 + 8 * s, 2 * Cfg::kStage);  // both CTAs' boxes of this stage
          const uint32_t bar = ptx::mapa(full0 + 8 * s, 0);                    // the leader's barrier, from either CTA
          ptx::tma_load_2d_pair(dst, &map_a, kb * sh.k_elems_per_block, row_a, bar);
          ptx::tma_load_2d_pair(dst + Cfg::kStageA, &map_b, kb * sh.k_elems_per_block, row_b, bar);
        }
      }
      if (rank == 0) {
        // no copy of either CTA may still be in flight when the pair's shared memory is released (the leader's barriers
        // count both CTAs' bytes; the peer stays until the cluster barrier below)
        const long long first = it > Cfg::kStages ? it - Cfg::kStages : 0;
        for (long long j = first; j < it; j++) {
          volatile int never = 0;
          ptx::mbar_wait(full0 + 8 * static_cast<int>(j % Cfg::kStages), static_cast<uint32_t>((j / Cfg::kStages) & 1), &never);
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    if (lane == 0 && rank == 0) {
      long long it = 0;
      int titer = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, titer++) {
        const int acc = titer & 1;
        const uint32_t aph = static_cast<uint32_t>((titer >> 1) & 1);
        ok = ptx::mbar_wait(tempty0 + 8 * acc, aph ^ 1u, abort_flag);  // both CTAs' epilogues have drained this buffer
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccCols);
        for (int kb = 0; kb < sh.kblocks; kb++, it++) {
          const int s = static_cast<int>(it % Cfg::kStages);
          const uint32_t ph = static_cast<uint32_t>((it / Cfg::kStages) & 1);
          ok = ptx::mbar_wait(full0 + 8 * s, ph, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint64_t a_desc = ptx::tc_smem_desc_sw128(base + s * Cfg::kStage);
          const uint64_t b_desc = ptx::tc_smem_desc_sw128(base + s * Cfg::kStage + Cfg::kStageA);
#pragma unroll
          for (int j = 0; j < kGemmStageK / 32; j++)  // 32 bytes of k per instruction: +2 in the descriptor's 16-byte units
            ptx::tc_mma_pair<KIND>(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, (kb | j) != 0 ? 1u : 0u);
          ptx::tc_commit_pair(empty0 + 8 * s);  // frees the stage in both CTAs
        }
        if (ok) ptx::tc_commit_pair(tfull0 + 8 * acc);
      }
    }
    __syncwarp();
  } else {
    int titer = 0;
    bool ok = true;
    Epi::kernel_begin(ep, threadIdx.x);
    for (int tile = pair; tile < tiles && ok; tile += pairs, titer++) {
      int tm, tn;
      gemm_tile_coords(tile, sh.tiles_m, sh.tiles_n, sh.band, tm, tn);
      const int acc = titer & 1;
      const uint32_t aph = static_cast<uint32_t>((titer >> 1) & 1);
      const int row0 = tm * Cfg::kTile + static_cast<int>(rank) * Cfg::kRows;
      Epi::begin_tile(ep, epi_smem, row0, tn * Cfg::kTile, sh.m, sh.n, threadIdx.x);
      ok = ptx::mbar_wait(tfull0 + 8 * acc, aph, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      const int row = row0 + warp * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc * Cfg::kAccCols);
#pragma unroll 1
      for (int c = 0; c < Cfg::kTile / 32; c++) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        Epi::store(ep, epi_smem, row, tn * Cfg::kTile, c * 32, r, sh.m, sh.n);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(tempty0 + 8 * acc, 0));
    }
    Epi::kernel_end(ep, threadIdx.x, ok);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(status, 2);
  ptx::cluster_sync();  // neither CTA signals the other, or is read by the other's MMAs, from here on
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace tvb

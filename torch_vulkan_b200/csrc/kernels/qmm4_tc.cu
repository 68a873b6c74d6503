// aten::_dyn_quant_matmul_4bit for large m on the fifth-generation tensor cores, still bit for bit.
//
// The reference's PHASE 1 (crates/vkcore/shaders/qmm4.slang:183-247) scales every block of bs values of k by
// its own float32 scale and adds the blocks up in order, so the int32 block sums cannot be merged: each one has
// to leave the tensor core, be converted, multiplied and added with the reference's roundings. This kernel lets
// tcgen05.mma kind::i8 produce the block sums and makes that drain as cheap as it can be:
//
//   * Operands: the int4 weights unpacked once to int8 [n, k] (tvb_qmm4_prepare; the ATen layer caches it per
//     packed tensor), the activations quantised to int8 [m, k] by PHASE 0 with 64 extra columns per row holding
//     o1 + o2 = -zero_point. (q - zp) does not fit int8, but q and -zp do, except -zp = 128 (a row without negative
//     values), which is stored as 64 + 64. A block sum is W.q + W.o1 into the same accumulator, plus W.o2 only for a
//     tile of tokens in which some row needs it (exact integers, same value as the shader's loop).
//   * Orientation: weight rows ride the MMA's 128 rows (TMEM lanes), tokens its 128 columns, so each draining
//     thread owns one output column n and keeps that column's block scale in a register.
//   * Drain: tcgen05.ld brings 32 int32 sums per thread; float(iacc) * scale costs one integer add and one FMA:
//     bits(0x4B400000 + iacc) is the float 12582912 + iacc exactly, and fma(that, s, -12582912 s) rounds the exact
//     product iacc * s once, which is fl(float(iacc) * s). (Needs 3 s exact in float32, true for scales that came
//     from bfloat16; otherwise, or for blocks over 1024 values, a convert and a multiply are used.) One more add
//     accumulates, as the reference does; the first block assigns. (Starting the accumulators at 0x4B400000, stored
//     back by the draining warp with tcgen05.st so that the integer add disappears, was measured 2.5 times slower.)
//   * Four TMEM accumulator buffers (4 x 128 columns) let the MMAs of the next blocks run under the drain.
//
// The float16 form of the same kernel (tvb_qmm4_tc16) exists for the one case in which the drain can be a single
// instruction per output and block. The integers (q - zp) in [-255, 255] and the weights in [-8, 7] are exact in float16
// and their block sums (below 2^24) exact in the float32 accumulators of kind::f16, so the tensor core hands over
// float(iacc) itself: no offset operands, no conversion. And when the block holds 32 values (|iacc| <= 65280 < 2^16)
// and the scale came from bfloat16 (8 significant bits), iacc * s has at most 24 significant bits: fl(float(iacc) * s)
// IS iacc * s, so the reference's fl(acc + fl(float(iacc) * s)) equals fma(float(iacc), s, acc), one rounding either way.
// Scales that are not such (a device flag set when the weights are prepared) take multiply and add. The price is two
// bytes per operand element (weights unpacked to float16 [n, k]) and the kind::f16 rate, half of kind::i8, which the
// drain, the limit of both forms, does not feel.
//
// Warp roles: 0-15 drain and epilogue (four warps per TMEM lane quarter, one per 32 tokens: four warps per scheduler
// hide each other's tcgen05.ld and barrier waits, which two could not), 16 TMA producer, 17 and 18 MMA issuers (17 owns the
// tensor memory allocation).
// Every wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "numerics.cuh"
#include "ptx.cuh"
#include "qmm4_phase0.cuh"

namespace tvb {
namespace {

constexpr int kTileN = 128;   // weight rows (output columns) per tile = MMA rows
constexpr int kTileM = 128;   // tokens per tile = MMA columns
constexpr int kStageK = 128;  // bytes of k per shared-memory stage (four 32-k MMA steps)
constexpr int kStages = 6;
constexpr int kStageBytes = (kTileN + kTileM) * kStageK;  // 32 KB
constexpr int kOTileBytes = kTileM * kStageK;             // 16 KB: the tokens' o1 / o2 columns
constexpr int kAccBuffers = 4;
constexpr int kDrainWarps = 16;
constexpr int kIssuers = 2;   // warps that issue MMAs (one lane each): blocks in turn
constexpr int kThreads = (kDrainWarps + 1 + kIssuers) * 32;
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kOTileBytes + 1024 + 256;
constexpr int kExtraCols = 64;  // per activation row: 32 x o1, 32 x o2

struct TcParams {
  const float* scales;   // [n, ndrains] (inside the packed vector)
  const float* bias;     // [n] or NULL
  const float* recip;    // [m]
  const int32_t* neg_zp; // [m]
  const int* wide_scales;  // device flag: some scale has more than 22 significant bits
  void* out;             // [m, n] float32 or bfloat16
  int* status;
  int m, n, k;
  int steps_per_drain;   // bs / 32
  int ndrains;           // k / bs
  int tiles_m, tiles_n;
  int out_bf16;
};

// PHASE 0 with the tensor-core layout: q rows of k + 64 bytes, the tail holding o1 (32 bytes) and o2 (32 bytes).
// F16: rows of k float16 values q - zero_point (in [-255, 255], exact) instead, with no tail.
template <int DT, bool F16 = false>
__global__ void __launch_bounds__(256) qmm4_quantize_tc_kernel(const void* __restrict__ inp, int k, int groupwise,
                                                               int8_t* __restrict__ q, float* __restrict__ recip_out,
                                                               int32_t* __restrict__ neg_zp_out) {
  __shared__ float red_min[8], red_max[8];
  __shared__ float row_scale;
  __shared__ int row_zp;
  ptx::grid_launch_dependents();  // (a kernel launched with programmatic serialization may start its own prologue now)
  ptx::grid_dependency_wait();    // (and this one, launched that way itself, touches memory only after its predecessors)
  const int64_t base = static_cast<int64_t>(blockIdx.x) * k;
  const int64_t qbase = static_cast<int64_t>(blockIdx.x) * (k + kExtraCols);
  const int t = threadIdx.x;
  float mn = 3.40282347e38f, mx = -3.40282347e38f;
  for (int kk = t; kk < k; kk += 256) {
    float v = load_float<DT>(inp, base + kk);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((t & 31) == 0) {
    red_min[t >> 5] = mn;
    red_max[t >> 5] = mx;
  }
  __syncthreads();
  if (t == 0) {
    for (int i = 1; i < 8; i++) {
      mn = fminf(mn, red_min[i]);
      mx = fmaxf(mx, red_max[i]);
    }
    const Phase0Row row = phase0_row(mn, mx, groupwise);
    row_scale = row.scale;
    row_zp = row.zero_point;
    recip_out[blockIdx.x] = row.recip;
    neg_zp_out[blockIdx.x] = -row.zero_point;
  }
  __syncthreads();
  const float scale = row_scale;
  const int zp = row_zp;
  if constexpr (F16) {
    __half* v = reinterpret_cast<__half*>(q) + base;
    for (int kk = t; kk < k; kk += 256) v[kk] = __int2half_rn(phase0_code(load_float<DT>(inp, base + kk), scale, zp) - zp);
    return;
  }
  for (int kk = t; kk < k; kk += 256) {
    q[qbase + kk] = static_cast<int8_t>(phase0_code(load_float<DT>(inp, base + kk), scale, zp));
  }
  if (t < kExtraCols) {
    const int off = -zp;                 // in [-127, 128]
    const int o1 = off > 127 ? 64 : off;  // (128 does not fit int8: the one value that takes both halves)
    q[qbase + k + t] = static_cast<int8_t>(t < 32 ? o1 : off - o1);
  }
}

// The same weights as float16 [n, k] (the operands of the float16 form).
__global__ void qmm4_unpack16_kernel(const float* __restrict__ packed, int64_t nbytes, __half2* __restrict__ w) {
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
    const int byte = static_cast<int>(packed[i]);
    w[i] = __halves2half2(__int2half_rn((byte & 15) - 8), __int2half_rn((byte >> 4) - 8));
  }
}

// The packed vector's float-encoded weight bytes -> int8 weights [n, k] (low nibble first, value nibble - 8).
__global__ void qmm4_unpack_kernel(const float* __restrict__ packed, int64_t nbytes, int8_t* __restrict__ w) {
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
    uint32_t byte = static_cast<uint32_t>(packed[i]);
    uint32_t lo = ((byte & 15u) - 8u) & 0xffu, hi = ((byte >> 4) - 8u) & 0xffu;
    reinterpret_cast<uint16_t*>(w)[i] = static_cast<uint16_t>(lo | (hi << 8));
  }
}

// Sets bit 0 of *flag when a scale's low two mantissa bits are not zero (3 * s would then not be exact in float32), or it
// is subnormal, or so large that a product could overflow; bit 1 when a scale has more than bfloat16's 8 significant bits
// (its low 16 bits are not zero) or bit 0's exceptions apply.
__global__ void qmm4_scan_scales_kernel(const float* __restrict__ scales, int64_t count, int* __restrict__ flag) {
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int wide = 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    uint32_t bits = __float_as_uint(scales[i]);
    uint32_t exp = (bits >> 23) & 0xffu;
    const bool odd = (exp == 0u && (bits & 0x7fffffu) != 0u) || exp >= 0xf0u;
    if ((bits & 3u) != 0u || odd) wide |= 1;
    if ((bits & 0xffffu) != 0u || odd || exp >= 0xe0u) wide |= 2;  // (from 2^97 on a block's product could overflow)
  }
  for (int o = 16; o > 0; o >>= 1) wide |= __shfl_xor_sync(0xffffffffu, wide, o);
  if (wide != 0 && (threadIdx.x & 31) == 0) atomicOr(flag, wide);
}

// One block's 32 integer sums folded into 32 running outputs: x = fl(float(iacc) * s); acc = FIRST ? x : fl(acc + x).
// Not WIDE: bits(iacc + 0x4B400000) is the float 12582912 + iacc exactly, and fma(that, s, -12582912 s) rounds the
// exact product iacc * s once. WIDE: convert and multiply.
// MODE 0: int32 sums, scales of at most 22 significant bits. 1: int32 sums, any scale (WIDE). 2: float32 sums (the float16
// form), blocks of 32 values and scales that came from bfloat16: float(iacc) * s is exact, so one fma is the reference's
// multiply and add. 3: float32 sums, any scale or block: multiply, add.
template <int MODE, bool FIRST>
__device__ __forceinline__ void fold_block(float (&acc)[32], const uint32_t (&r)[32], const float s, const float t) {
#pragma unroll
  for (int i = 0; i < 32; i++) {
    if (MODE == 2 && !FIRST) {
      acc[i] = __fmaf_rn(__uint_as_float(r[i]), s, acc[i]);
    } else {
      const float x = MODE >= 2 ? __fmul_rn(__uint_as_float(r[i]), s)
                                : (MODE == 1 ? __fmul_rn(static_cast<float>(static_cast<int>(r[i])), s)
                                             : __fmaf_rn(__uint_as_float(r[i] + 0x4B400000u), s, t));
      acc[i] = FIRST ? x : __fadd_rn(acc[i], x);  // (the first block assigns: keeps -0)
    }
  }
}

// The drain and epilogue of warps 0-15. MODE as in fold_block.
template <int MODE>
__device__ __forceinline__ void drain_tiles(const TcParams& p, const uint32_t tmem_base, const uint32_t tfull0,
                                            const uint32_t tempty0, volatile int* abort_flag, const int warp, const int lane) {
  const int tiles = p.tiles_m * p.tiles_n;
  const int quarter = warp & 3, group = warp >> 2;  // TMEM lanes 32 quarter ..., tokens 32 group ... of the tile
  const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(group * 32);
  uint32_t buf = 0, buf_phase = 0;
  bool ok = true;
  for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
    const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
    const int col = tn * kTileN + quarter * 32 + lane;   // output column = weight row
    const int col_ld = min(col, p.n - 1);
    const int tok0 = tm * kTileM + group * 32;
    const float* srow = p.scales + static_cast<int64_t>(col_ld) * p.ndrains;
    float acc0[32];   // tokens tok0 .. tok0+31
    float s_next = __ldg(srow);
    for (int d = 0; d < p.ndrains && ok; d++) {
      const float s = s_next;
      if (d + 1 < p.ndrains) s_next = __ldg(srow + d + 1);
      const float t = __fmul_rn(-12582912.0f, s);  // exact when s has at most 22 significant bits
      ok = ptx::mbar_wait(tfull0 + 8 * buf, buf_phase, abort_flag);  // the block's MMAs have completed
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t r0[32];
      ptx::tmem_ld_32x32(lane_base + buf * kTileM, r0);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty0 + 8 * buf);  // the sums are in registers: the buffer is free again
      if (++buf == kAccBuffers) {
        buf = 0;
        buf_phase ^= 1u;
      }
      if (d == 0) fold_block<MODE, true>(acc0, r0, s, t);
      else fold_block<MODE, false>(acc0, r0, s, t);
    }
    if (!ok) break;
    if (col < p.n) {
      const float bias = p.bias != nullptr ? __ldg(p.bias + col) : 0.0f;
      const float hi = p.out_bf16 ? 3.38953139e38f : 3.40282347e38f;
#pragma unroll
      for (int i = 0; i < 32; i++) {
        const int tok = tok0 + i;
        if (tok < p.m) {
          float v = __fmul_rn(acc0[i], __ldg(p.recip + tok));
          if (p.bias != nullptr) v = __fadd_rn(v, bias);
          v = v < -hi ? -hi : v;  // (std::max / std::min: NaN passes)
          v = hi < v ? hi : v;
          const int64_t o = static_cast<int64_t>(tok) * p.n + col;
          if (p.out_bf16) static_cast<uint16_t*>(p.out)[o] = static_cast<uint16_t>(__float_as_uint(v) >> 16);
          else static_cast<float*>(p.out)[o] = v;
        }
      }
    }
  }
}

template <bool F16>
__global__ void __launch_bounds__(kThreads, 1)
    qmm4_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q, const TcParams p) {
  constexpr int kStepElems = F16 ? 16 : 32;         // values of k per MMA instruction (32 bytes)
  constexpr int kStageElems = kStageK / (F16 ? 2 : 1);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t otile0 = base + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kStages * kStageBytes + 2 * kOTileBytes);
  const uint32_t full0 = ptx::smem_u32(bars), empty0 = full0 + 8 * kStages;
  const uint32_t ofull0 = empty0 + 8 * kStages, oempty0 = ofull0 + 16;
  const uint32_t tfull0 = oempty0 + 16, tempty0 = tfull0 + 8 * kAccBuffers;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + 2 * kAccBuffers);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* needs_o2 = abort_flag + 1;  // per slot of the o tile: some token of the tile has -zero_point = 128
  static_assert((2 * kStages + 4 + 2 * kAccBuffers) * 8 + 16 <= 256, "barrier area too small");
  static_assert((kAccBuffers & (kAccBuffers - 1)) == 0, "the buffer ring is indexed with a mask");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The usual case, blocks of 32 values and k a multiple of a stage: every stage holds whole blocks, and the issuers take
  // whole stages in turn (the straight-line loop below). Otherwise every issuer walks every stage.
  constexpr int kStepsPerBlock32 = F16 ? 2 : 1, kBlocksPerStage = 4 / kStepsPerBlock32;
  const bool by_stage = p.steps_per_drain == kStepsPerBlock32 && ((p.k / (F16 ? 16 : 32)) & 3) == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, by_stage && F16 ? 1 : kIssuers);  // (float16 form by stage: only one issuer has MMAs on a stage)
    }
    for (int i = 0; i < 2; i++) {
      ptx::mbar_init(ofull0 + 8 * i, 1);
      ptx::mbar_init(oempty0 + 8 * i, kIssuers);
    }
    for (int b = 0; b < kAccBuffers; b++) {
      ptx::mbar_init(tfull0 + 8 * b, 1);
      ptx::mbar_init(tempty0 + 8 * b, kDrainWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kDrainWarps + 1) ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.tiles_m * p.tiles_n;
  const int nstages = (p.k + kStageElems - 1) / kStageElems;
  const int nsteps = p.k / kStepElems;

  if (warp == kDrainWarps) {
    // ---------------- producer: lane 0 issues every TMA copy; the warp together looks at the tile's zero points
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_w);
      ptx::prefetch_tensormap(&map_q);
    }
    long long it = 0;
    int ti = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ti++) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int slot = ti & 1;
      // does a token of this tile carry -zero_point = 128 (then the MMA lane adds the W.o2 term)? four tokens per lane
      bool wide_row = false;
      if constexpr (!F16) {
        for (int i = lane; i < kTileM; i += 32) {
          const int tok = tm * kTileM + i;
          wide_row = wide_row || (tok < p.m && __ldg(p.neg_zp + tok) == 128);
        }
        wide_row = __any_sync(0xffffffffu, wide_row);
      }
      if (lane == 0) {
        if constexpr (!F16) {
          ok = ptx::mbar_wait(oempty0 + 8 * slot, static_cast<uint32_t>(((ti >> 1) & 1) ^ 1), abort_flag);
          if (ok) {
            needs_o2[slot] = wide_row ? 1 : 0;  // (ordered before the MMA lane's read by the barrier it waits on)
            ptx::mbar_expect_tx(ofull0 + 8 * slot, kOTileBytes);
            ptx::tma_load_2d(otile0 + slot * kOTileBytes, &map_q, p.k, tm * kTileM, ofull0 + 8 * slot);
          }
        }
        if (ok) {
          for (int kb = 0; kb < nstages; kb++, it++) {
            const int s = static_cast<int>(it % kStages);
            ok = ptx::mbar_wait(empty0 + 8 * s, static_cast<uint32_t>(((it / kStages) & 1) ^ 1), abort_flag);
            if (!ok) break;
            const uint32_t dst = base + s * kStageBytes;
            ptx::mbar_expect_tx(full0 + 8 * s, kStageBytes);
            ptx::tma_load_2d(dst, &map_w, kb * kStageElems, tn * kTileN, full0 + 8 * s);
            ptx::tma_load_2d(dst + kTileN * kStageK, &map_q, kb * kStageElems, tm * kTileM, full0 + 8 * s);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    if (lane == 0) {
      // no copy may still be in flight when the CTA's shared memory is released
      const long long first = it > kStages ? it - kStages : 0;
      for (long long j = first; j < it; j++) {
        volatile int never = 0;
        ptx::mbar_wait(full0 + 8 * static_cast<int>(j % kStages), static_cast<uint32_t>((j / kStages) & 1), &never);
      }
      if (!F16 && ti > 0 && ok) {
        volatile int never = 0;
        ptx::mbar_wait(ofull0 + 8 * ((ti - 1) & 1), static_cast<uint32_t>(((ti - 1) >> 1) & 1), &never);
      }
    }
    __syncwarp();
  } else if (warp > kDrainWarps) {
    // ---------------- MMA issuers. An MMA of this size occupies the tensor pipe for about 64 clocks, but one thread's
    // instruction stream around it (barrier waits, descriptors, commits, loop) takes several hundred per block: measured
    // with one issuer, that stream set the pace of the whole kernel, whatever the drain did. So the blocks (one
    // accumulator buffer each) are dealt to kIssuers lanes in turn; every issuer walks all stages, waits for each, issues
    // the steps of its own blocks and commits each stage (a stage is free when every issuer's MMAs on it are done).
    const int issuer = warp - kDrainWarps - 1;
    if (lane == 0) {
      // int32 accumulators and signed 8-bit operands, or float32 accumulators and float16 operands; both K-major, 128 x 128
      const uint32_t idesc = F16 ? ptx::tc_instr_desc(1, 0, 0, kTileN, kTileM) : ptx::tc_instr_desc(2, 1, 1, kTileN, kTileM);
      // This one thread's instruction stream paces the tensor core (an MMA of this size lasts ~64 clocks), so the
      // bookkeeping is kept to counters that are bumped, never divided.
      if (by_stage) {
        // One thread's instruction stream around an MMA of this size (about 64 clocks of tensor pipe) costs far more than
        // the MMA: every branch of a lone thread is tens of clocks. So this loop has no bookkeeping beyond two counters:
        // stage gs of the CTA's stream holds blocks gs * kBlocksPerStage ..., and block b goes to accumulator buffer b % 4.
        // An issuer keeps to its own two buffers (a barrier's parity tells "this phase or the one before" only to a thread
        // that has seen every phase): with two blocks per stage (float16) that is every other stage, with four (int8) half
        // of every stage.
        static_assert(kIssuers == 2 && kAccBuffers == 4, "the split of the buffers between the issuers");
        uint32_t gs = 0;
        int ti = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ti++) {
          const int slot = ti & 1;
          uint64_t o_desc = 0;
          bool with_o2 = false;
          if constexpr (!F16) {
            ok = ptx::mbar_wait(ofull0 + 8 * slot, static_cast<uint32_t>((ti >> 1) & 1), abort_flag);
            if (!ok) break;
            o_desc = ptx::tc_smem_desc_sw128(otile0 + slot * kOTileBytes);
            with_o2 = needs_o2[slot] != 0;
          }
          for (int kb = 0; kb < nstages && ok; kb++, gs++) {
            if (F16 && gs % kIssuers != static_cast<uint32_t>(issuer)) continue;
            const uint32_t stage = gs % kStages, stage_phase = (gs / kStages) & 1u;
            ok = ptx::mbar_wait(full0 + 8 * stage, stage_phase, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint64_t w_desc = ptx::tc_smem_desc_sw128(base + stage * kStageBytes);
            const uint64_t q_desc = ptx::tc_smem_desc_sw128(base + stage * kStageBytes + kTileN * kStageK);
#pragma unroll
            for (int bb = 0; bb < 2; bb++) {
              const int b = F16 ? bb : 2 * issuer + bb;
              const uint32_t blk = gs * kBlocksPerStage + b, buf = blk & (kAccBuffers - 1), buf_phase = (blk / kAccBuffers) & 1u;
              ok = ptx::mbar_wait(tempty0 + 8 * buf, buf_phase ^ 1u, abort_flag);  // the drain warps have read it
              if (!ok) break;
              ptx::tc_fence_after();
              const uint32_t d_tmem = tmem_base + buf * kTileM;
              if constexpr (F16) {  // W . (q - zp): two steps of 16 values of k (32 bytes each: +2 in the descriptor's units)
                ptx::tc_mma<2>(d_tmem, w_desc + 4 * b, q_desc + 4 * b, idesc, 0u);
                ptx::tc_mma<2>(d_tmem, w_desc + 4 * b + 2, q_desc + 4 * b + 2, idesc, 1u);
              } else {
                ptx::tc_mma<1>(d_tmem, w_desc + 2 * b, q_desc + 2 * b, idesc, 0u);
                ptx::tc_mma<1>(d_tmem, w_desc + 2 * b, o_desc, idesc, 1u);                   // + W . o1
                if (with_o2) ptx::tc_mma<1>(d_tmem, w_desc + 2 * b, o_desc + 2, idesc, 1u);  // + W . o2
              }
              ptx::tc_commit(tfull0 + 8 * buf);
            }
            if (ok) ptx::tc_commit(empty0 + 8 * stage);
          }
          if (!F16 && ok) ptx::tc_commit(oempty0 + 8 * slot);
        }
      } else {
      uint32_t stage = 0, stage_phase = 0;      // shared-memory ring position
      uint32_t buf = 0, buf_phase = 0;          // TMEM accumulator ring position (of the block under way, whoever issues it)
      int turn = 0;                             // whose block it is
      int in_drain = 0;
      const int spd = p.steps_per_drain;
      int ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ti++) {
        const int slot = ti & 1;
        uint64_t o_desc = 0;
        bool with_o2 = false;
        if constexpr (!F16) {
          ok = ptx::mbar_wait(ofull0 + 8 * slot, static_cast<uint32_t>((ti >> 1) & 1), abort_flag);
          if (!ok) break;
          o_desc = ptx::tc_smem_desc_sw128(otile0 + slot * kOTileBytes);
          with_o2 = needs_o2[slot] != 0;
        }
        int steps_left = nsteps;
        for (int kb = 0; kb < nstages && ok; kb++) {
          ok = ptx::mbar_wait(full0 + 8 * stage, stage_phase, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          uint64_t w_desc = ptx::tc_smem_desc_sw128(base + stage * kStageBytes);
          uint64_t q_desc = ptx::tc_smem_desc_sw128(base + stage * kStageBytes + kTileN * kStageK);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            if (steps_left <= 0) break;
            steps_left--;
            const bool mine = turn == issuer;
            if (mine && in_drain == 0) {
              ok = ptx::mbar_wait(tempty0 + 8 * buf, buf_phase ^ 1u, abort_flag);  // the drain warps have read it
              if (!ok) break;
              ptx::tc_fence_after();
            }
            const uint32_t d_tmem = tmem_base + buf * kTileM;
            if (mine) {
              if constexpr (F16) {
                ptx::tc_mma<2>(d_tmem, w_desc, q_desc, idesc, in_drain != 0 ? 1u : 0u);  // W . (q - zp), 16 values of k
              } else {
                ptx::tc_mma<1>(d_tmem, w_desc, q_desc, idesc, in_drain != 0 ? 1u : 0u);
                ptx::tc_mma<1>(d_tmem, w_desc, o_desc, idesc, 1u);                   // + W . o1
                if (with_o2) ptx::tc_mma<1>(d_tmem, w_desc, o_desc + 2, idesc, 1u);  // + W . o2 (a row with -zero_point = 128)
              }
            }
            w_desc += 2;  // the next 32 bytes of k, in the descriptor's 16-byte units
            q_desc += 2;
            if (++in_drain == spd) {
              if (mine) ptx::tc_commit(tfull0 + 8 * buf);
              if (++turn == kIssuers) turn = 0;
              in_drain = 0;
              if (++buf == kAccBuffers) {
                buf = 0;
                buf_phase ^= 1u;
              }
            }
          }
          ptx::tc_commit(empty0 + 8 * stage);
          if (++stage == kStages) {
            stage = 0;
            stage_phase ^= 1u;
          }
        }
        if (!F16 && ok) ptx::tc_commit(oempty0 + 8 * slot);
      }
      }
    }
    __syncwarp();
  } else {
    // ---------------- drain: thread = one weight row (output column), 32 tokens
    const int flag = *p.wide_scales;  // bit 0: a scale with more than 22 significant bits; bit 1: one that did not come from bfloat16
    if constexpr (F16) {
      if (flag == 0 && p.steps_per_drain == 2) drain_tiles<2>(p, tmem_base, tfull0, tempty0, abort_flag, warp, lane);
      else drain_tiles<3>(p, tmem_base, tfull0, tempty0, abort_flag, warp, lane);
    } else {
      if ((flag & 1) != 0 || p.steps_per_drain > 32) drain_tiles<1>(p, tmem_base, tfull0, tempty0, abort_flag, warp, lane);
      else drain_tiles<0>(p, tmem_base, tfull0, tempty0, abort_flag, warp, lane);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 3);
  if (warp == kDrainWarps + 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

uint64_t align256(uint64_t x) { return (x + 255) & ~uint64_t(255); }

}  // namespace
}  // namespace tvb

namespace tvb {

// PHASE 0 in the tensor-core layout, for the other kernels that read it (qmm4_decode.cu).
int qmm4_quantize_rows(cudaStream_t stream, const void* inp, int dtype, int64_t m, int64_t k, int groupwise, int8_t* q, float* recip,
                       int32_t* neg_zp) {
  dim3 qgrid(static_cast<unsigned>(m));
  // Launched with programmatic stream serialization: in a stream of decoding products its launch latency hides behind the
  // previous product (whose completion it still waits for before it reads or writes anything).
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = qgrid;
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int ki = static_cast<int>(k);
  if (dtype == TVB_F32) {
    TVB_CUDA(cudaLaunchKernelEx(&cfg, qmm4_quantize_tc_kernel<TVB_F32>, inp, ki, groupwise, q, recip, neg_zp));
  } else {
    TVB_CUDA(cudaLaunchKernelEx(&cfg, qmm4_quantize_tc_kernel<TVB_BF16>, inp, ki, groupwise, q, recip, neg_zp));
  }
  return launched("qmm4_quantize_tc", qgrid, dim3(256), 0, stream);
}

}  // namespace tvb

using namespace tvb;

extern "C" uint64_t tvb_qmm4_prepared_bytes(int64_t n, int64_t k) {
  return 256 + align256(static_cast<uint64_t>(n) * static_cast<uint64_t>(k));
}

extern "C" int tvb_qmm4_prepare(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                                uint64_t prepared_bytes) {
  TVB_REQUIRE(n > 0 && k > 0 && bs > 0 && k % 2 == 0 && k % bs == 0, "tvb_qmm4_prepare: bad shape");
  TVB_REQUIRE(packed != nullptr && prepared != nullptr && prepared_bytes >= tvb_qmm4_prepared_bytes(n, k),
              "tvb_qmm4_prepare: prepared buffer too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  int* flag = static_cast<int*>(prepared);
  int8_t* w = static_cast<int8_t*>(prepared) + 256;
  TVB_CUDA(cudaMemsetAsync(flag, 0, 256, stream));
  const int64_t nbytes = n * k / 2, nscales = n * (k / bs);
  const int cap = sm_count(device) * 16;
  int grid = static_cast<int>(std::min<int64_t>(ceil_div(nbytes, 256), cap));
  qmm4_unpack_kernel<<<grid, 256, 0, stream>>>(packed, nbytes, w);
  if (launched("qmm4_unpack", dim3(grid), dim3(256), 0, stream) != 0) return -1;
  grid = static_cast<int>(std::min<int64_t>(ceil_div(nscales, 256), cap));
  qmm4_scan_scales_kernel<<<grid, 256, 0, stream>>>(packed + nbytes, nscales, flag);
  return launched("qmm4_scan_scales", dim3(grid), dim3(256), 0, stream);
}

extern "C" uint64_t tvb_qmm4_prepared16_bytes(int64_t n, int64_t k) {
  return 256 + align256(2 * static_cast<uint64_t>(n) * static_cast<uint64_t>(k));
}

extern "C" int tvb_qmm4_prepare16(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                                  uint64_t prepared_bytes) {
  TVB_REQUIRE(n > 0 && k > 0 && bs > 0 && k % 2 == 0 && k % bs == 0, "tvb_qmm4_prepare16: bad shape");
  TVB_REQUIRE(packed != nullptr && prepared != nullptr && prepared_bytes >= tvb_qmm4_prepared16_bytes(n, k),
              "tvb_qmm4_prepare16: prepared buffer too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  int* flag = static_cast<int*>(prepared);
  __half2* w = reinterpret_cast<__half2*>(static_cast<uint8_t*>(prepared) + 256);
  TVB_CUDA(cudaMemsetAsync(flag, 0, 256, stream));
  const int64_t nbytes = n * k / 2, nscales = n * (k / bs);
  const int cap = sm_count(device) * 16;
  int grid = static_cast<int>(std::min<int64_t>(ceil_div(nbytes, 256), cap));
  qmm4_unpack16_kernel<<<grid, 256, 0, stream>>>(packed, nbytes, w);
  if (launched("qmm4_unpack16", dim3(grid), dim3(256), 0, stream) != 0) return -1;
  grid = static_cast<int>(std::min<int64_t>(ceil_div(nscales, 256), cap));
  qmm4_scan_scales_kernel<<<grid, 256, 0, stream>>>(packed + nbytes, nscales, flag);
  return launched("qmm4_scan_scales", dim3(grid), dim3(256), 0, stream);
}

extern "C" uint64_t tvb_qmm4_tc16_workspace_bytes(int64_t m, int64_t k) {
  return align256(2 * static_cast<uint64_t>(m) * static_cast<uint64_t>(k)) + 2 * align256(static_cast<uint64_t>(m) * 4);
}

extern "C" int tvb_qmm4_tc16(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                             void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_BF16, "tvb_qmm4_tc16: input must be float32 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0 && k > 0 && bs > 0, "tvb_qmm4_tc16: bad size");
  TVB_REQUIRE(k % 32 == 0 && bs % 32 == 0 && k % bs == 0, "tvb_qmm4_tc16: k and the block size must be multiples of 32");
  // (a block's sum must stay below 2^24 to be exact in the float32 accumulator: bs * 255 * 8)
  TVB_REQUIRE(bs <= 8192, "tvb_qmm4_tc16: blocks of at most 8192 values");
  TVB_REQUIRE(m * k < (int64_t(1) << 31) && n * k < (int64_t(1) << 32) && m * n < (int64_t(1) << 40), "tvb_qmm4_tc16: sizes beyond 32 bits");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(inp != nullptr && packed != nullptr && prepared != nullptr && out != nullptr, "tvb_qmm4_tc16: NULL pointer");
  TVB_REQUIRE(workspace != nullptr && workspace_bytes >= tvb_qmm4_tc16_workspace_bytes(m, k), "tvb_qmm4_tc16: workspace too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  const uint64_t qbytes = align256(2 * static_cast<uint64_t>(m) * static_cast<uint64_t>(k));
  const uint64_t rbytes = align256(static_cast<uint64_t>(m) * 4);
  int8_t* q = static_cast<int8_t*>(workspace);
  float* recip = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + qbytes);
  int32_t* neg_zp = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + qbytes + rbytes);
  const int groupwise = bs != k ? 1 : 0;
  dim3 qgrid(static_cast<unsigned>(m));
  if (dtype == TVB_F32)
    qmm4_quantize_tc_kernel<TVB_F32, true><<<qgrid, 256, 0, stream>>>(inp, static_cast<int>(k), groupwise, q, recip, neg_zp);
  else
    qmm4_quantize_tc_kernel<TVB_BF16, true><<<qgrid, 256, 0, stream>>>(inp, static_cast<int>(k), groupwise, q, recip, neg_zp);
  if (launched("qmm4_quantize_tc16", qgrid, dim3(256), 0, stream) != 0) return -1;

  static std::mutex mutex;
  static bool configured[64] = {};
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (!configured[device & 63]) {
      TVB_CUDA(cudaFuncSetAttribute(qmm4_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      configured[device & 63] = true;
    }
  }
  const uint8_t* w = static_cast<const uint8_t*>(prepared) + 256;
  CUtensorMap map_w, map_q;
  if (make_tensor_map_2d(&map_w, w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, n, 2 * k, kStageK / 2, kTileN, CU_TENSOR_MAP_SWIZZLE_128B) != 0) return -1;
  if (make_tensor_map_2d(&map_q, q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, m, 2 * k, kStageK / 2, kTileM, CU_TENSOR_MAP_SWIZZLE_128B) != 0) return -1;
  TcParams p{};
  const int64_t wcount = n * k / 2;
  p.ndrains = static_cast<int>(k / bs);
  p.steps_per_drain = static_cast<int>(bs / 16);
  p.scales = packed + wcount;
  p.bias = has_bias ? packed + wcount + n * p.ndrains : nullptr;
  p.recip = recip;
  p.neg_zp = neg_zp;
  p.wide_scales = static_cast<const int*>(prepared);
  p.out = out;
  if (status_word(device, &p.status) != 0) return -1;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.tiles_m = static_cast<int>(ceil_div(m, kTileM));
  p.tiles_n = static_cast<int>(ceil_div(n, kTileN));
  p.out_bf16 = dtype == TVB_BF16;
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(device), static_cast<int64_t>(p.tiles_m) * p.tiles_n));
  qmm4_tc_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(map_w, map_q, p);
  return launched("qmm4_tc16", dim3(grid), dim3(kThreads), kSmemBytes, stream);
}

extern "C" uint64_t tvb_qmm4_tc_workspace_bytes(int64_t m, int64_t k) {
  return align256(static_cast<uint64_t>(m) * static_cast<uint64_t>(k + kExtraCols)) + 2 * align256(static_cast<uint64_t>(m) * 4);
}

extern "C" int tvb_qmm4_tc(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                           void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_BF16, "tvb_qmm4_tc: input must be float32 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0 && k > 0 && bs > 0, "tvb_qmm4_tc: bad size");
  TVB_REQUIRE(k % 32 == 0 && bs % 32 == 0 && k % bs == 0, "tvb_qmm4_tc: k and the block size must be multiples of 32");
  TVB_REQUIRE(m * (k + kExtraCols) < (int64_t(1) << 31) && n * k < (int64_t(1) << 32) && m * n < (int64_t(1) << 40),
              "tvb_qmm4_tc: sizes beyond 32 bits");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(inp != nullptr && packed != nullptr && prepared != nullptr && out != nullptr, "tvb_qmm4_tc: NULL pointer");
  TVB_REQUIRE(workspace != nullptr && workspace_bytes >= tvb_qmm4_tc_workspace_bytes(m, k), "tvb_qmm4_tc: workspace too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  const uint64_t qbytes = align256(static_cast<uint64_t>(m) * static_cast<uint64_t>(k + kExtraCols));
  const uint64_t rbytes = align256(static_cast<uint64_t>(m) * 4);
  int8_t* q = static_cast<int8_t*>(workspace);
  float* recip = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + qbytes);
  int32_t* neg_zp = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + qbytes + rbytes);
  const int groupwise = bs != k ? 1 : 0;
  dim3 qgrid(static_cast<unsigned>(m));
  if (dtype == TVB_F32)
    qmm4_quantize_tc_kernel<TVB_F32><<<qgrid, 256, 0, stream>>>(inp, static_cast<int>(k), groupwise, q, recip, neg_zp);
  else
    qmm4_quantize_tc_kernel<TVB_BF16><<<qgrid, 256, 0, stream>>>(inp, static_cast<int>(k), groupwise, q, recip, neg_zp);
  if (launched("qmm4_quantize_tc", qgrid, dim3(256), 0, stream) != 0) return -1;

  static bool configured[64] = {};
  if (!configured[device & 63]) {
    TVB_CUDA(cudaFuncSetAttribute(qmm4_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[device & 63] = true;
  }
  const int8_t* w = static_cast<const int8_t*>(prepared) + 256;
  CUtensorMap map_w, map_q;
  if (make_tensor_map_2d(&map_w, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, k, n, k, kStageK, kTileN, CU_TENSOR_MAP_SWIZZLE_128B) != 0) return -1;
  if (make_tensor_map_2d(&map_q, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, k + kExtraCols, m, k + kExtraCols, kStageK, kTileM,
                         CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  TcParams p{};
  const int64_t wcount = n * k / 2;
  p.ndrains = static_cast<int>(k / bs);
  p.steps_per_drain = static_cast<int>(bs / 32);
  p.scales = packed + wcount;
  p.bias = has_bias ? packed + wcount + n * p.ndrains : nullptr;
  p.recip = recip;
  p.neg_zp = neg_zp;
  p.wide_scales = static_cast<const int*>(prepared);
  p.out = out;
  if (status_word(device, &p.status) != 0) return -1;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.tiles_m = static_cast<int>(ceil_div(m, kTileM));
  p.tiles_n = static_cast<int>(ceil_div(n, kTileN));
  p.out_bf16 = dtype == TVB_BF16;
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(device), static_cast<int64_t>(p.tiles_m) * p.tiles_n));
  qmm4_tc_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(map_w, map_q, p);
  return launched("qmm4_tc", dim3(grid), dim3(kThreads), kSmemBytes, stream);
}

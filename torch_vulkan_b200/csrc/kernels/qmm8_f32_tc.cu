// aten::_weight_int8pack_mm with float32 activations on the fifth-generation tensor cores, for a moderate number of rows.
//
// C[m, n] = A[m, k] @ (int8 B[n, k] * scales[n]).T in float32 (the reference's tiled path for more than 8 rows,
// crates/vkcore/shaders/qmm8.slang:113-173, launched from crates/pyvk/csrc/quant.cpp:102-117). A float32 value does not
// fit a 16-bit tensor-core operand, but it is exactly the sum of three bfloat16 values (hi = bf16(a), mid = bf16(a - hi),
// lo = bf16(a - hi - mid): 3 x 8 significant bits), an int8 weight is exact in bfloat16, and a bfloat16 x bfloat16
// product is exact in float32. So the product is three bfloat16 products whose float32 sums are added at the end:
//
//   qmm8_f32_tc_kernel, one CTA per (32 rows of A, 128 weight rows, slice of k): the weight rows ride the MMA's 128 rows
//   (TMEM lanes), the 96 term rows its columns, so every term has its own float32 accumulator column and small terms are
//   not lost in a large running sum. A producer warp streams raw boxes by TMA (lane 0 the int8 weights, lane 1 the float32
//   rows of A); eight converter warps widen the weights to bfloat16 (exactly) and split the rows of A into their three
//   terms, both into the 128-byte-swizzled operand ring; one lane issues tcgen05.mma kind::f16 (one 128 x 96 x 16 MMA per
//   16 values of k); four epilogue warps read the accumulators back, add (lo + mid) + hi and either finish (scale, store)
//   or, when k is split over several CTAs so that a small matrix still fills the GPU, store the partial sums; the last CTA
//   of a tile to arrive adds the slices in ascending order (a fixed order: the result does not depend on who came last).
//   Launched with programmatic stream serialization: the weights of the next product stream while this one finishes.
// The scale multiplies the finished sum, (sum a b) s, so an intermediate sum beyond float32's range overflows where the
// reference's sum of a (b s) might not; otherwise both are within the float32 rounding the reference's tests allow.
// The kernel is bound by streaming B from HBM once. All waits are bounded.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "numerics.cuh"
#include "ptx.cuh"

namespace tvb {
namespace {

constexpr int kRows = 128;                 // weight rows (output columns) per tile = MMA rows
constexpr int kTokens = 32;                // rows of A per tile
constexpr int kTermRows = 3 * kTokens;     // MMA columns: hi, mid, lo of every row
constexpr int kBK = 64;                    // values of k per stage
constexpr int kRawStages = 6, kOpStages = 4;
constexpr int kRawBytes = kRows * kBK;            // 8 KB of int8
constexpr int kARawBytes = kTokens * kBK * 4;     // 8 KB of float32
constexpr int kWBytes = kRows * kBK * 2;          // 16 KB of bfloat16
constexpr int kTBytes = kTermRows * kBK * 2;      // 12 KB
constexpr int kOpBytes = kWBytes + kTBytes;
constexpr int kConvWarps = 8;                     // warps 4 .. 11
constexpr int kProducerWarp = 4 + kConvWarps, kMmaWarp = kProducerWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr int kSmemBytes = kOpStages * kOpBytes + kRawStages * (kRawBytes + kARawBytes) + 1024 + 512;

struct F32TcParams {
  const float* scales;
  float* c;          // [m, n]
  float* partials;   // [tiles_m * tiles_n][ksplit][kRows][kTokens], used when ksplit > 1
  int* counters;     // [tiles_m * tiles_n], zero between launches
  int* status;
  int m, n, k;
  int tiles_n, ksplit, kblocks_per_split, kblocks;
};

// int8 x 4 -> two packed pairs of bfloat16, exactly (see widen_int8x4 in qmm8_skinny.cuh).
__device__ __forceinline__ void widen4_bf16(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t l = w & 0x7f7f7f7fu, s = w & 0x80808080u;
  lo = ptx::sub_bf16x2(ptx::prmt(l, 0x43434343u, 0x4140u), ptx::prmt(s, 0x43434343u, 0x4140u));
  hi = ptx::sub_bf16x2(ptx::prmt(l, 0x43434343u, 0x4342u), ptx::prmt(s, 0x43434343u, 0x4342u));
}

// (lo, hi) -> two bfloat16 values in one word, lo in the low half, both rounded to nearest even.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
    qmm8_f32_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_t, const F32TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t raw0 = base + kOpStages * kOpBytes, araw0 = raw0 + kRawStages * kRawBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kOpStages * kOpBytes + kRawStages * (kRawBytes + kARawBytes));
  const uint32_t raw_full0 = ptx::smem_u32(bars), raw_empty0 = raw_full0 + 8 * kRawStages;
  const uint32_t araw_full0 = raw_empty0 + 8 * kRawStages, araw_empty0 = araw_full0 + 8 * kRawStages;
  const uint32_t op_full0 = araw_empty0 + 8 * kRawStages, op_empty0 = op_full0 + 8 * kOpStages;
  const uint32_t tfull = op_empty0 + 8 * kOpStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kRawStages + 2 * kOpStages + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  static_assert((4 * kRawStages + 2 * kOpStages + 1) * 8 + 12 <= 512, "barrier area too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; s++) {
      ptx::mbar_init(raw_full0 + 8 * s, 1);
      ptx::mbar_init(raw_empty0 + 8 * s, kConvWarps);
      ptx::mbar_init(araw_full0 + 8 * s, 1);
      ptx::mbar_init(araw_empty0 + 8 * s, kConvWarps);
    }
    for (int s = 0; s < kOpStages; s++) {
      ptx::mbar_init(op_full0 + 8 * s, kConvWarps);
      ptx::mbar_init(op_empty0 + 8 * s, 1);
    }
    ptx::mbar_init(tfull, 1);
    *abort_flag = 0;
    *last_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 128);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  ptx::grid_launch_dependents();  // the next kernel of the stream may take SMs as this one's CTAs retire

  // this CTA's unit: (tile of A rows, tile of weight rows, slice of k)
  const int split = blockIdx.x % p.ksplit;
  const int tile = blockIdx.x / p.ksplit;
  const int tn = tile % p.tiles_n, tm = tile / p.tiles_n;
  const int kb0 = split * p.kblocks_per_split;
  const int kb1 = min(p.kblocks, kb0 + p.kblocks_per_split);
  const int nkb = kb1 - kb0;  // (at least one: the host sizes the split that way)

  if (warp == kProducerWarp) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_w);
      const uint64_t stream_policy = ptx::policy_evict_first();  // weights are read once
      bool ok = true;
      for (int i = 0; i < nkb && ok; i++) {
        const int r = i % kRawStages;
        ok = ptx::mbar_wait_spin(raw_empty0 + 8 * r, static_cast<uint32_t>(((i / kRawStages) & 1) ^ 1), abort_flag);
        if (!ok) break;
        ptx::mbar_expect_tx(raw_full0 + 8 * r, kRawBytes);
        ptx::tma_load_2d_hint(raw0 + r * kRawBytes, &map_w, (kb0 + i) * kBK, tn * kRows, raw_full0 + 8 * r, stream_policy);
      }
      // nothing may still be landing when the CTA's shared memory is released
      for (int j = nkb > kRawStages ? nkb - kRawStages : 0; j < nkb && ok; j++) {
        volatile int never = 0;
        ptx::mbar_wait(raw_full0 + 8 * (j % kRawStages), static_cast<uint32_t>((j / kRawStages) & 1), &never);
      }
    } else if (lane == 1) {
      ptx::prefetch_tensormap(&map_t);
      ptx::grid_dependency_wait();  // (A may be the previous kernel's output; the weights above are nobody's output)
      bool ok = true;
      for (int i = 0; i < nkb && ok; i++) {
        const int r = i % kRawStages;
        ok = ptx::mbar_wait_spin(araw_empty0 + 8 * r, static_cast<uint32_t>(((i / kRawStages) & 1) ^ 1), abort_flag);
        if (!ok) break;
        ptx::mbar_expect_tx(araw_full0 + 8 * r, kARawBytes);
        ptx::tma_load_2d(araw0 + r * kARawBytes, &map_t, (kb0 + i) * kBK, tm * kTokens, araw_full0 + 8 * r);
      }
      for (int j = nkb > kRawStages ? nkb - kRawStages : 0; j < nkb && ok; j++) {
        volatile int never = 0;
        ptx::mbar_wait(araw_full0 + 8 * (j % kRawStages), static_cast<uint32_t>((j / kRawStages) & 1), &never);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = ptx::tc_instr_desc(1, 1, 1, kRows, kTermRows);  // float32 accumulators, bfloat16 operands
      bool ok = true;
      for (int i = 0; i < nkb && ok; i++) {
        const int s = i % kOpStages;
        const uint32_t ph = static_cast<uint32_t>((i / kOpStages) & 1);
        ok = ptx::mbar_wait_spin(op_full0 + 8 * s, ph, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
        uint64_t w_desc = ptx::tc_smem_desc_sw128(base + s * kOpBytes);
        uint64_t t_desc = ptx::tc_smem_desc_sw128(base + s * kOpBytes + kWBytes);
#pragma unroll
        for (int j = 0; j < kBK / 16; j++) {
          ptx::tc_mma<2>(tmem_base, w_desc, t_desc, idesc, (i | j) != 0 ? 1u : 0u);
          w_desc += 2;  // the next 16 values of k (32 bytes), in the descriptor's 16-byte units
          t_desc += 2;
        }
        ptx::tc_commit(op_empty0 + 8 * s);
      }
      if (ok) ptx::tc_commit(tfull);
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------- converters: raw int8 [128][64] -> bfloat16 [128][128 bytes], raw float32 [32][64] -> three bfloat16
    // tiles [32][128 bytes], all in the 128-byte-swizzled K-major layout the MMA's shared-memory descriptors expect
    const int ct = threadIdx.x - 128;  // 0 .. 255
    bool ok = true;
    for (int i = 0; i < nkb && ok; i++) {
      const int r = i % kRawStages, s = i % kOpStages;
      const uint32_t rph = static_cast<uint32_t>((i / kRawStages) & 1);
      ok = ptx::mbar_wait_spin(raw_full0 + 8 * r, rph, abort_flag) && ptx::mbar_wait_spin(araw_full0 + 8 * r, rph, abort_flag) &&
           ptx::mbar_wait_spin(op_empty0 + 8 * s, static_cast<uint32_t>(((i / kOpStages) & 1) ^ 1), abort_flag);
      if (!ok) break;
      const uint32_t src = raw0 + r * kRawBytes, dst = base + s * kOpBytes;
#pragma unroll
      for (int u = 0; u < kRawBytes / 16 / (32 * kConvWarps); u++) {
        const int q = ct + 32 * kConvWarps * u;  // 16-byte chunk of the raw tile: row q / 4, k 16 * (q % 4) ...
        const int row = q >> 2, c = q & 3;
        const uint4 v = ptx::lds128(src + q * 16);
        uint32_t o[8];
        widen4_bf16(v.x, o[0], o[1]);
        widen4_bf16(v.y, o[2], o[3]);
        widen4_bf16(v.z, o[4], o[5]);
        widen4_bf16(v.w, o[6], o[7]);
        const uint32_t rowaddr = dst + row * 128;
        sts128(rowaddr + (((2 * c) ^ (row & 7)) << 4), o[0], o[1], o[2], o[3]);
        sts128(rowaddr + (((2 * c + 1) ^ (row & 7)) << 4), o[4], o[5], o[6], o[7]);
      }
      {
        // this thread's eight values of A: row ct / 8, k 8 * (ct % 8) ...; each becomes hi + mid + lo exactly
        const int row = ct >> 3, c = ct & 7;
        const uint32_t asrc = araw0 + r * kARawBytes + row * (kBK * 4) + c * 32;
        const uint4 x0 = ptx::lds128(asrc), x1 = ptx::lds128(asrc + 16);
        const uint32_t bits[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        uint32_t t[3][4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          // two values at a time through the hardware's packed float32 -> bfloat16 conversion (round to nearest even)
          const float v0 = __uint_as_float(bits[2 * j]), v1 = __uint_as_float(bits[2 * j + 1]);
          const uint32_t h = pack_bf16x2(v0, v1);
          const float h0 = __uint_as_float(h << 16), h1 = __uint_as_float(h & 0xffff0000u);
          // (an infinity or NaN stays in the first term alone: its remainders would be NaN)
          const float r0 = (h & 0x7f80u) == 0x7f80u ? 0.0f : __fsub_rn(v0, h0);
          const float r1 = (h & 0x7f800000u) == 0x7f800000u ? 0.0f : __fsub_rn(v1, h1);
          const uint32_t md = pack_bf16x2(r0, r1);
          const float q0 = __fsub_rn(r0, __uint_as_float(md << 16)), q1 = __fsub_rn(r1, __uint_as_float(md & 0xffff0000u));
          t[0][j] = h;
          t[1][j] = md;
          t[2][j] = pack_bf16x2(q0, q1);
        }
#pragma unroll
        for (int term = 0; term < 3; term++) {
          const int trow = term * kTokens + row;
          sts128(dst + kWBytes + trow * 128 + ((c ^ (trow & 7)) << 4), t[term][0], t[term][1], t[term][2], t[term][3]);
        }
      }
      ptx::fence_proxy_async();  // the MMA reads these generic-proxy stores through the async proxy
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(op_full0 + 8 * s);
        ptx::mbar_arrive(raw_empty0 + 8 * r);
        ptx::mbar_arrive(araw_empty0 + 8 * r);
      }
    }
  } else {
    // ---------------- epilogue: thread = one weight row (output column), 32 rows of A
    bool ok = ptx::mbar_wait(tfull, 0, abort_flag);
    if (ok) {
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      float v[32];
      {
        uint32_t mid[32], lo[32];
        ptx::tmem_ld_32x32(taddr + kTokens, mid);
        ptx::tmem_ld_32x32(taddr + 2 * kTokens, lo);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __uint_as_float(lo[i]) + __uint_as_float(mid[i]);  // the small terms first
      }
      {
        uint32_t hi[32];
        ptx::tmem_ld_32x32(taddr, hi);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] += __uint_as_float(hi[i]);
      }
      const int rowl = warp * 32 + lane;  // weight row within the tile
      const int col = tn * kRows + rowl;
      bool finish = true;
      ptx::grid_dependency_wait();  // (scratch, counters and C may still be in use by the stream's previous kernel)
      if (p.ksplit > 1) {
        // this slice's sums go to scratch; the last of the tile's CTAs to arrive adds all slices, in ascending order
        float* mine = p.partials + ((static_cast<size_t>(tile) * p.ksplit + split) * kRows + rowl) * kTokens;
#pragma unroll
        for (int i = 0; i < 32; i += 4) __stcg(reinterpret_cast<float4*>(mine + i), make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]));
        ptx::named_bar_sync(1, 128);
        if (threadIdx.x == 0) {
          __threadfence();
          const int last = atomicAdd(&p.counters[tile], 1) == p.ksplit - 1;
          if (last) atomicExch(&p.counters[tile], 0);  // zero again for the next launch
          *last_flag = last;
        }
        ptx::named_bar_sync(1, 128);
        finish = *last_flag != 0;
        if (finish) {
          __threadfence();
#pragma unroll
          for (int i = 0; i < 32; i++) v[i] = 0.0f;
          for (int sp = 0; sp < p.ksplit; sp++) {
            const float* theirs = p.partials + ((static_cast<size_t>(tile) * p.ksplit + sp) * kRows + rowl) * kTokens;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 x = __ldcg(reinterpret_cast<const float4*>(theirs + i));
              v[i] += x.x; v[i + 1] += x.y; v[i + 2] += x.z; v[i + 3] += x.w;
            }
          }
        }
      }
      if (finish && col < p.n) {
        const float scale = p.scales[col];
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const int row = tm * kTokens + i;
          if (row < p.m) p.c[static_cast<int64_t>(row) * p.n + col] = v[i] * scale;  // (a warp: 32 consecutive columns of a row)
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 6);
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 128);
  }
}

uint64_t align256(uint64_t x) { return (x + 255) & ~uint64_t(255); }

}  // namespace

// float32 A with at most 256 rows, k a multiple of 64, A's rows and B 16-byte aligned.
bool qmm8_f32_tc_usable(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k) {
  return dtype == TVB_F32 && m >= 1 && m <= 256 && n >= 1 && k >= kBK && k % kBK == 0 && k < (int64_t(1) << 24) &&
         (reinterpret_cast<uintptr_t>(b) & 15u) == 0 && a != nullptr && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
         (m == 1 || (a_sm >= k && a_sm % 4 == 0));
}

int qmm8_f32_tc(int device, cudaStream_t stream, const float* a, int64_t a_sm, const int8_t* b, const float* scales, float* c, int64_t m,
                int64_t n, int64_t k) {
  {
    static std::mutex mutex;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> lock(mutex);
    if (!configured[device & 63]) {
      TVB_CUDA(cudaFuncSetAttribute(qmm8_f32_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      configured[device & 63] = true;
    }
  }
  const int tiles_m = static_cast<int>(ceil_div(m, kTokens)), tiles_n = static_cast<int>(ceil_div(n, kRows));
  const int kblocks = static_cast<int>(k / kBK);
  // k is split so that a small matrix still occupies the SMs; a slice keeps at least 256 values of k
  const int sms = sm_count(device);
  int ksplit = std::max(1, sms / (tiles_m * tiles_n));
  ksplit = std::min(ksplit, std::max(1, kblocks / 4));
  if (const char* forced = std::getenv("TVB200_F32_KSPLIT")) ksplit = std::max(1, std::min(std::atoi(forced), kblocks));
  const int per_split = static_cast<int>(ceil_div(kblocks, ksplit));
  ksplit = static_cast<int>(ceil_div(kblocks, per_split));
  // scratch: the tiles' counters (zero between launches), then the slices' partial sums
  const uint64_t counter_bytes = align256(static_cast<uint64_t>(tiles_m) * tiles_n * sizeof(int));
  TVB_REQUIRE(counter_bytes <= 65536, "tvb_qmm8: too many tiles for the float32 tensor-core kernel");
  const uint64_t partial_bytes = ksplit > 1 ? static_cast<uint64_t>(tiles_m) * tiles_n * ksplit * kRows * kTokens * sizeof(float) : 0;
  void* ws = nullptr;
  if (workspace(device, 2, 65536 + partial_bytes, &ws) != 0) return -1;
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  CUtensorMap map_w, map_t;
  if (make_tensor_map_2d(&map_w, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, k, n, k, kBK, kRows, CU_TENSOR_MAP_SWIZZLE_NONE) != 0) return -1;
  if (make_tensor_map_2d(&map_t, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, k, m, (m == 1 ? k : a_sm) * 4, kBK, kTokens,
                         CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
    return -1;
  F32TcParams p{};
  p.scales = scales;
  p.c = c;
  p.partials = reinterpret_cast<float*>(wsb + 65536);
  p.counters = reinterpret_cast<int*>(wsb);
  if (status_word(device, &p.status) != 0) return -1;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.tiles_n = tiles_n;
  p.ksplit = ksplit;
  p.kblocks_per_split = per_split;
  p.kblocks = kblocks;
  const int grid = tiles_m * tiles_n * ksplit;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TVB_CUDA(cudaLaunchKernelEx(&cfg, qmm8_f32_tc_kernel, map_w, map_t, p));
  return launched("qmm8_f32_tc", dim3(grid), dim3(kThreads), kSmemBytes, stream);
}

}  // namespace tvb

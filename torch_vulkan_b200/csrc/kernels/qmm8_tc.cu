// aten::_weight_int8pack_mm for m > 16 on the fifth-generation tensor cores.
//
// C[m, n] = A[m, k] @ (int8 B[n, k] * scales[n]).T with bfloat16 / float16 A (the reference's tiled path,
// crates/vkcore/shaders/qmm8.slang:113-173, dequantises the weights as it stages them in shared memory; so does this
// kernel, onto tcgen05). int8 values are exact in bf16 / f16 and the products are exact in float32, so the sum
// differs from the reference's only by float32 accumulation order; the scale multiplies the finished sum.
//
// Persistent CTAs over 128 x 256 output tiles; per 64 values of k:
//   warp 12 (two lanes) TMA: a 256-row x 64-byte box of int8 weights into a raw ring (no swizzle) and a 128-row x
//                      128-byte box of A into the operand ring (128-byte swizzle); every CTA fetches its own copy
//   warps 4-11         widen the raw weights to 16-bit floats in registers (byte permutes and one packed subtract per
//                      pair, exact) and store them into the operand ring in the 128-byte-swizzled K-major layout
//                      that the MMA's shared-memory descriptor expects
//   warp 13 (one lane) four tcgen05.mma kind::f16 (k = 16 each) per stage into one of two 256-column TMEM buffers
//   warps 0-3          epilogue: tcgen05.ld, times scales[n], one rounding to A's dtype, 16-byte stores
// All waits are bounded; a wait that runs out releases TMEM and sets the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "numerics.cuh"
#include "ptx.cuh"
#include "scaled_mm.h"

namespace tvb {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64;     // tile and k per stage
constexpr int kRawStages = 4, kOpStages = 3;
constexpr int kRawBytes = kBN * kBK;              // 16 KB of int8
constexpr int kABytes = kBM * kBK * 2;            // 16 KB
constexpr int kWBytes = kBN * kBK * 2;            // 32 KB
constexpr int kOpBytes = kABytes + kWBytes;
constexpr int kEpiBytes = 4 * kBN * 4;            // per epilogue warp: the tile's column scales
constexpr int kConvWarps = 8;                    // warps 4 .. 4 + kConvWarps - 1
constexpr int kProducerWarp = 4 + kConvWarps, kMmaWarp = kProducerWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr int kSmemBytes = kOpStages * kOpBytes + kRawStages * kRawBytes + kEpiBytes + 1024 + 256;

struct Q8TcParams {
  const void* scales;
  void* c;
  int* status;
  int m, n, k;
  int tiles_m, tiles_n, kblocks;
  int vector_ok;
};

template <int DT>
__device__ __forceinline__ void widen4(uint32_t w, uint32_t& lo, uint32_t& hi) {
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

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1)
    qmm8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Q8TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t raw0 = base + kOpStages * kOpBytes;
  float* epi = reinterpret_cast<float*>(base_ptr + kOpStages * kOpBytes + kRawStages * kRawBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kOpStages * kOpBytes + kRawStages * kRawBytes + kEpiBytes);
  const uint32_t raw_full0 = ptx::smem_u32(bars), raw_empty0 = raw_full0 + 8 * kRawStages;
  const uint32_t a_full0 = raw_empty0 + 8 * kRawStages, w_full0 = a_full0 + 8 * kOpStages, op_empty0 = w_full0 + 8 * kOpStages;
  const uint32_t tfull0 = op_empty0 + 8 * kOpStages, tempty0 = tfull0 + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kRawStages + 3 * kOpStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * kRawStages + 3 * kOpStages + 4) * 8 + 8 <= 256, "barrier area too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; s++) {
      ptx::mbar_init(raw_full0 + 8 * s, 1);
      ptx::mbar_init(raw_empty0 + 8 * s, kConvWarps);
    }
    for (int s = 0; s < kOpStages; s++) {
      ptx::mbar_init(a_full0 + 8 * s, 1);
      ptx::mbar_init(w_full0 + 8 * s, kConvWarps);
      ptx::mbar_init(op_empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(tfull0 + 8 * a, 1);
      ptx::mbar_init(tempty0 + 8 * a, 128);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.tiles_m * p.tiles_n;

  if (warp == kProducerWarp) {
    // Two independent loaders, so that the weight stream (whose latency is HBM's) runs as far ahead as the raw ring
    // allows and never waits for an operand slot: lane 0 streams the weights, lane 1 the tiles of A.
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_w);
      const uint64_t stream_policy = ptx::policy_evict_first();
      long long it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int tn = tile / p.tiles_m;
        for (int kb = 0; kb < p.kblocks; kb++, it++) {
          const int r = static_cast<int>(it % kRawStages);
          ok = ptx::mbar_wait(raw_empty0 + 8 * r, static_cast<uint32_t>(((it / kRawStages) & 1) ^ 1), abort_flag);
          if (!ok) break;
          ptx::mbar_expect_tx(raw_full0 + 8 * r, kRawBytes);
          ptx::tma_load_2d_hint(raw0 + r * kRawBytes, &map_w, kb * kBK, tn * kBN, raw_full0 + 8 * r, stream_policy);
        }
      }
      // nothing may still be landing when the CTA's shared memory is released
      for (long long j = it > kRawStages ? it - kRawStages : 0; j < it; j++) {
        volatile int never = 0;
        ptx::mbar_wait(raw_full0 + 8 * static_cast<int>(j % kRawStages), static_cast<uint32_t>((j / kRawStages) & 1), &never);
      }
    } else if (lane == 1) {
      ptx::prefetch_tensormap(&map_a);
      long long it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int tm = tile % p.tiles_m;
        for (int kb = 0; kb < p.kblocks; kb++, it++) {
          const int s = static_cast<int>(it % kOpStages);
          ok = ptx::mbar_wait(op_empty0 + 8 * s, static_cast<uint32_t>(((it / kOpStages) & 1) ^ 1), abort_flag);
          if (!ok) break;
          ptx::mbar_expect_tx(a_full0 + 8 * s, kABytes);
          ptx::tma_load_2d(base + s * kOpBytes, &map_a, kb * kBK, tm * kBM, a_full0 + 8 * s);
        }
      }
      for (long long j = it > kOpStages ? it - kOpStages : 0; j < it; j++) {
        volatile int never = 0;
        ptx::mbar_wait(a_full0 + 8 * static_cast<int>(j % kOpStages), static_cast<uint32_t>((j / kOpStages) & 1), &never);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t fmt = DT == TVB_BF16 ? 1u : 0u;  // kind::f16 operand formats: 0 float16, 1 bfloat16
      const uint32_t idesc = ptx::tc_instr_desc(1, fmt, fmt, kBM, kBN);
      uint32_t s = 0, s_phase = 0;
      int titer = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, titer++) {
        const int acc = titer & 1;
        ok = ptx::mbar_wait(tempty0 + 8 * acc, static_cast<uint32_t>(((titer >> 1) & 1) ^ 1), abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBN);
        for (int kb = 0; kb < p.kblocks; kb++) {
          ok = ptx::mbar_wait(a_full0 + 8 * s, s_phase, abort_flag) && ptx::mbar_wait(w_full0 + 8 * s, s_phase, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          uint64_t a_desc = ptx::tc_smem_desc_sw128(base + s * kOpBytes);
          uint64_t w_desc = ptx::tc_smem_desc_sw128(base + s * kOpBytes + kABytes);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            ptx::tc_mma<2>(d_tmem, a_desc, w_desc, idesc, (kb | j) != 0 ? 1u : 0u);
            a_desc += 2;
            w_desc += 2;
          }
          ptx::tc_commit(op_empty0 + 8 * s);
          if (++s == kOpStages) {
            s = 0;
            s_phase ^= 1u;
          }
        }
        if (ok) ptx::tc_commit(tfull0 + 8 * acc);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------- converters: raw int8 [256][64] -> 16-bit floats [256][128 bytes], swizzled
    const int ct = threadIdx.x - 128;  // 0 .. 32 * kConvWarps - 1
    long long it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < p.kblocks; kb++, it++) {
        const int r = static_cast<int>(it % kRawStages), s = static_cast<int>(it % kOpStages);
        ok = ptx::mbar_wait(raw_full0 + 8 * r, static_cast<uint32_t>((it / kRawStages) & 1), abort_flag) &&
             ptx::mbar_wait(op_empty0 + 8 * s, static_cast<uint32_t>(((it / kOpStages) & 1) ^ 1), abort_flag);
        if (!ok) break;
        const uint32_t src = raw0 + r * kRawBytes, dst = base + s * kOpBytes + kABytes;
#pragma unroll
        for (int i = 0; i < kRawBytes / 16 / (32 * kConvWarps); i++) {
          const int q = ct + 32 * kConvWarps * i;  // 16-byte chunk of the raw tile: row q / 4, k 16 * (q % 4) ...
          const int row = q >> 2, c = q & 3;
          const uint4 v = ptx::lds128(src + q * 16);
          uint32_t o[8];
          widen4<DT>(v.x, o[0], o[1]);
          widen4<DT>(v.y, o[2], o[3]);
          widen4<DT>(v.z, o[4], o[5]);
          widen4<DT>(v.w, o[6], o[7]);
          const uint32_t rowaddr = dst + row * 128;
          sts128(rowaddr + (((2 * c) ^ (row & 7)) << 4), o[0], o[1], o[2], o[3]);
          sts128(rowaddr + (((2 * c + 1) ^ (row & 7)) << 4), o[4], o[5], o[6], o[7]);
        }
        ptx::fence_proxy_async();  // the MMA reads these generic-proxy stores through the async proxy
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(w_full0 + 8 * s);
          ptx::mbar_arrive(raw_empty0 + 8 * r);
        }
      }
    }
  } else {
    // ---------------- epilogue
    float* cs = epi + warp * kBN;
    int titer = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, titer++) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int acc = titer & 1;
      __syncwarp();
      for (int i = lane; i < kBN; i += 32) {
        const int col = tn * kBN + i;
        cs[i] = col < p.n ? load_float<DT>(p.scales, col) : 0.0f;
      }
      __syncwarp();
      ok = ptx::mbar_wait(tfull0 + 8 * acc, static_cast<uint32_t>((titer >> 1) & 1), abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      const int row = tm * kBM + warp * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc * kBN);
#pragma unroll 1
      for (int cb = 0; cb < kBN / 32; cb++) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + cb * 32, r);
        ptx::tmem_ld_wait();
        const int col = tn * kBN + cb * 32;
        if (row < p.m && col < p.n) {
          uint16_t* out = static_cast<uint16_t*>(p.c) + static_cast<int64_t>(row) * p.n + col;
          if (p.vector_ok && col + 32 <= p.n) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; j++) {
                const float v0 = __uint_as_float(r[q * 8 + 2 * j]) * cs[cb * 32 + q * 8 + 2 * j];
                const float v1 = __uint_as_float(r[q * 8 + 2 * j + 1]) * cs[cb * 32 + q * 8 + 2 * j + 1];
                if (DT == TVB_BF16) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                  w[j] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                  __half2 h = __floats2half2_rn(v0, v1);
                  w[j] = *reinterpret_cast<uint32_t*>(&h);
                }
              }
              reinterpret_cast<uint4*>(out)[q] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i++)
              if (col + i < p.n) store_float<DT>(p.c, static_cast<int64_t>(row) * p.n + col + i, __uint_as_float(r[i]) * cs[cb * 32 + i]);
          }
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(tempty0 + 8 * acc);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 4);
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <int DT>
int launch_qmm8_tc(int device, cudaStream_t stream, const void* a, int64_t a_sm, const int8_t* b, const void* scales, void* c,
                   int64_t m, int64_t n, int64_t k) {
  auto kernel = qmm8_tc_kernel<DT>;
  static bool configured[64] = {};
  if (!configured[device & 63]) {
    TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[device & 63] = true;
  }
  CUtensorMap map_a, map_w;
  if (make_tensor_map_2d(&map_a, a, DT == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, m,
                         a_sm * 2, kBK, kBM, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  if (make_tensor_map_2d(&map_w, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, k, n, k, kBK, kBN, CU_TENSOR_MAP_SWIZZLE_NONE) != 0) return -1;
  Q8TcParams p{};
  p.scales = scales;
  p.c = c;
  if (status_word(device, &p.status) != 0) return -1;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.tiles_m = static_cast<int>(ceil_div(m, kBM));
  p.tiles_n = static_cast<int>(ceil_div(n, kBN));
  p.kblocks = static_cast<int>(ceil_div(k, kBK));
  p.vector_ok = (reinterpret_cast<uintptr_t>(c) & 15u) == 0 && (n * 2) % 16 == 0;
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(device), static_cast<int64_t>(p.tiles_m) * p.tiles_n));
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_w, p);
  return launched("qmm8_tc", dim3(grid), dim3(kThreads), kSmemBytes, stream);
}

}  // namespace

bool qmm8_tc_usable(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k) {
  return (dtype == TVB_BF16 || dtype == TVB_F16) && m >= 1 && n >= 1 && k >= 16 && k % 16 == 0 && (a_sm % 8 == 0 || m == 1) &&
         a_sm >= k && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(b) & 15u) == 0;
}

int qmm8_tc(int device, cudaStream_t stream, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales, void* c,
            int64_t m, int64_t n, int64_t k) {
  if (dtype == TVB_BF16) return launch_qmm8_tc<TVB_BF16>(device, stream, a, a_sm, b, scales, c, m, n, k);
  return launch_qmm8_tc<TVB_F16>(device, stream, a, a_sm, b, scales, c, m, n, k);
}

// ------------------------------------------------------------------ very large m: widen once, then the 16-bit GEMM
//
// From about a thousand rows of A on, widening the weights once into a scratch copy in A's dtype (n * k 16-bit values, a
// pass over 3 bytes per weight) and running the plain 16-bit tcgen05 GEMM over it, with the scales in its epilogue, is
// faster than widening inside the main loop (which the converter warps' ALU work bounds). The arithmetic is the same:
// exact 16-bit weights, float32 accumulation, the finished sum times scales[n], one rounding.

namespace {

template <int DT>
__global__ void qmm8_widen_kernel(const int8_t* __restrict__ b, uint16_t* __restrict__ wide, int64_t count16,
                                  const void* __restrict__ scales, float* __restrict__ scales32, int n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t i = first; i < n; i += stride) scales32[i] = load_float<DT>(scales, i);
  const uint4* src = reinterpret_cast<const uint4*>(b);
  uint4* dst = reinterpret_cast<uint4*>(wide);
  for (int64_t i = first; i < count16; i += stride) {  // 16 weights per step
    const uint4 v = __ldcs(src + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const float lo = static_cast<float>(static_cast<int8_t>(w[j] >> (16 * h)));
        const float hi = static_cast<float>(static_cast<int8_t>(w[j] >> (16 * h + 8)));
        o[2 * j + h] = DT == TVB_BF16 ? (static_cast<uint32_t>(f32_to_bf16_bits(lo)) | (static_cast<uint32_t>(f32_to_bf16_bits(hi)) << 16))
                                      : (static_cast<uint32_t>(f32_to_f16_bits(lo)) | (static_cast<uint32_t>(f32_to_f16_bits(hi)) << 16));
      }
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace

bool qmm8_widen_gemm_usable(const void* a, int dtype, int64_t a_sm, const int8_t* b, int64_t m, int64_t n, int64_t k) {
  return qmm8_tc_usable(a, dtype, a_sm, b, m, n, k) && (n * k) % 16 == 0 && k % 8 == 0;
}

// [n * k 16-bit weights][256-byte aligned: n float32 scales]
uint64_t widened_scale_offset(int64_t n, int64_t k) { return (static_cast<uint64_t>(n) * k * 2 + 255) & ~uint64_t(255); }

int qmm8_widen_into(int device, cudaStream_t stream, const int8_t* b, const void* scales, int dtype, int64_t n, int64_t k, void* widened) {
  uint16_t* wide = static_cast<uint16_t*>(widened);
  float* scales32 = reinterpret_cast<float*>(static_cast<uint8_t*>(widened) + widened_scale_offset(n, k));
  const int64_t count16 = n * k / 16;
  const int grid = static_cast<int>(std::min<int64_t>(static_cast<int64_t>(sm_count(device)) * 16, ceil_div(count16, 256)));
  if (dtype == TVB_BF16) qmm8_widen_kernel<TVB_BF16><<<grid, 256, 0, stream>>>(b, wide, count16, scales, scales32, static_cast<int>(n));
  else qmm8_widen_kernel<TVB_F16><<<grid, 256, 0, stream>>>(b, wide, count16, scales, scales32, static_cast<int>(n));
  return launched("qmm8_widen", dim3(grid), dim3(256), 0, stream);
}

int qmm8_widened_gemm(int device, cudaStream_t stream, const void* a, int dtype, int64_t a_sm, const void* widened, void* c, int64_t m,
                      int64_t n, int64_t k) {
  ScaledMmParams p{};
  p.a = a;
  p.b = widened;
  p.scale_a = nullptr;      // (the epilogue multiplies by 1 for A ...)
  p.scale_b = reinterpret_cast<const float*>(static_cast<const uint8_t*>(widened) + widened_scale_offset(n, k));  // (... by scales[n] for the columns)
  p.rowwise = 1;
  p.out = c;
  p.m = m; p.n = n; p.k = k;
  p.a_s0 = a_sm; p.a_s1 = 1;
  p.b_s0 = 1; p.b_s1 = k;   // B[kk, j] = wide[j * k + kk]
  p.a_dtype = dtype; p.b_dtype = dtype; p.out_dtype = dtype; p.bias_dtype = TVB_F32;
  if (!scaled_mm_tc_usable(p)) return fail("tvb_qmm8: the widened GEMM needs 16-byte aligned rows");
  return scaled_mm_tc(device, stream, p);
}

int qmm8_widen_gemm(int device, cudaStream_t stream, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                    void* c, int64_t m, int64_t n, int64_t k) {
  void* ws = nullptr;
  if (workspace(device, 1, widened_scale_offset(n, k) + static_cast<uint64_t>(n) * 4, &ws) != 0) return -1;
  if (qmm8_widen_into(device, stream, b, scales, dtype, n, k, ws) != 0) return -1;
  return qmm8_widened_gemm(device, stream, a, dtype, a_sm, ws, c, m, n, k);
}

}  // namespace tvb

using namespace tvb;

extern "C" uint64_t tvb_qmm8_widened_bytes(int64_t n, int64_t k) {
  return widened_scale_offset(n, k) + static_cast<uint64_t>(n) * 4;
}

extern "C" int tvb_qmm8_widen(int device, const int8_t* b, const void* scales, int dtype, int64_t n, int64_t k, void* widened,
                              uint64_t widened_bytes) {
  TVB_REQUIRE(dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8_widen: float16 or bfloat16 only");
  TVB_REQUIRE(n >= 1 && k >= 16 && k % 16 == 0 && (n * k) % 16 == 0, "tvb_qmm8_widen: k must be a multiple of 16");
  TVB_REQUIRE(b != nullptr && scales != nullptr && widened != nullptr && widened_bytes >= tvb_qmm8_widened_bytes(n, k),
              "tvb_qmm8_widen: NULL pointer or buffer too small");
  TVB_REQUIRE((reinterpret_cast<uintptr_t>(b) & 15u) == 0 && (reinterpret_cast<uintptr_t>(widened) & 255u) == 0,
              "tvb_qmm8_widen: B must be 16-byte and the buffer 256-byte aligned");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  return qmm8_widen_into(device, stream, b, scales, dtype, n, k, widened);
}

extern "C" int tvb_qmm8_widened(int device, const void* a, int dtype, int64_t a_sm, const void* widened, void* c, int64_t m, int64_t n,
                                int64_t k) {
  TVB_REQUIRE(dtype == TVB_F16 || dtype == TVB_BF16, "tvb_qmm8_widened: float16 or bfloat16 only");
  TVB_REQUIRE(m >= 0 && n >= 0 && k >= 16 && k % 16 == 0, "tvb_qmm8_widened: bad size");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(a != nullptr && widened != nullptr && c != nullptr, "tvb_qmm8_widened: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  return qmm8_widened_gemm(device, stream, a, dtype, m == 1 ? k : a_sm, widened, c, m, n, k);
}

// aten::_dyn_quant_matmul_4bit, the opt-in fast route (TORCH_VK_QMM4=fast): one float16 GEMM on tcgen05.
//
// Not bit-exact: the reference (crates/vkcore/shaders/qmm4.slang:183-247) rounds once per block of bs values of k;
// here the whole sum over k is accumulated in float32 inside the tensor core. What stays exact is every operand and
// every product: (q - zero_point) in [-255, 255] and weight * block scale (at most 3 + 8 significant bits when the
// scales came from bfloat16) are exact in float16, their products exact in float32. The result differs from the
// reference by float32 accumulation order only (the benchmark's stated bound: rtol 1e-5 with a magnitude floor);
// the int32 block sums, which the bound wants bit-exact, are what the two exact kernels produce (qmm4.cu, qmm4_tc.cu).
// Scales that are not exact in float16 after multiplication (float32 scales with full mantissas, or out of float16's
// range) set a flag when the weights are prepared; the caller must then use the exact route.
#include <cuda.h>
#include <cuda_fp16.h>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "gemm_tc.cuh"
#include "numerics.cuh"

namespace tvb {
namespace {

constexpr int kBN = 256;

// Per weight row, a power of two that brings the row's largest |weight * scale| just under float16's range (so that
// small scales do not fall into float16's denormals), and its inverse for the epilogue. Both exact.
__global__ void qmm4_fast_row_scale_kernel(const float* __restrict__ scales, int64_t n, int64_t nblocks, float* __restrict__ up,
                                           float* __restrict__ down) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= n) return;
  float smax = 0.0f;
  for (int64_t b = 0; b < nblocks; b++) smax = fmaxf(smax, fabsf(scales[row * nblocks + b]));
  int e = 0;
  if (smax > 0.0f && smax < 3.0e38f) {
    int ex;
    frexpf(smax * 8.0f, &ex);  // smax * 8 = f * 2^ex, f in [0.5, 1)
    e = 15 - ex;               // largest product scaled to [2^14, 2^15)
    e = max(-100, min(100, e));
  }
  up[row] = ldexpf(1.0f, e);
  down[row] = ldexpf(1.0f, -e);
}

// packed vector -> float16 [n, k] of (nibble - 8) * scale[n][k / bs] * up[n]; *flag set if some product is not exact.
__global__ void qmm4_fast_prepare_kernel(const float* __restrict__ packed, int64_t n, int64_t k, int64_t bs, const float* __restrict__ up,
                                         uint16_t* __restrict__ w, int* __restrict__ flag) {
  const int64_t nbytes = n * k / 2, nblocks = k / bs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int inexact = 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
    const int64_t row = i / (k / 2), kk = (i % (k / 2)) * 2;
    const float s = packed[nbytes + row * nblocks + kk / bs] * up[row];
    const int byte = static_cast<int>(packed[i]);
    const float v0 = static_cast<float>((byte & 15) - 8) * s, v1 = static_cast<float>((byte >> 4) - 8) * s;
    const __half h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
    if (__half2float(h0) != v0 || __half2float(h1) != v1) inexact = 1;
    reinterpret_cast<uint32_t*>(w)[i] = static_cast<uint32_t>(__half_as_ushort(h0)) | (static_cast<uint32_t>(__half_as_ushort(h1)) << 16);
  }
  if (__any_sync(0xffffffffu, inexact) && (threadIdx.x & 31) == 0) atomicOr(flag, 1);
}

// PHASE 0 (bit-exact, as qmm4.cu) writing q - zp as float16.
template <int DT>
__global__ void __launch_bounds__(256) qmm4_fast_quantize_kernel(const void* __restrict__ inp, int k, int groupwise,
                                                                 uint16_t* __restrict__ q, float* __restrict__ recip_out) {
  __shared__ float red_min[8], red_max[8];
  __shared__ float row_scale;
  __shared__ int row_zp;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * k;
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
    const float qmin = -128.0f, qmax = 127.0f;
    float rmin = fminf(0.0f, mn), rmax = fmaxf(0.0f, mx);
    float scale = rmin == rmax ? 1.0f : __fdiv_rn(qmax - qmin, __fsub_rn(rmax, rmin));
    float recip = scale != 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
    float dmin = __fmul_rn(rmin, scale), dmax = __fmul_rn(rmax, scale);
    float err = groupwise ? __fadd_rn(__fadd_rn(__fadd_rn(qmin, dmin), qmax), dmax)
                          : __fadd_rn(__fadd_rn(qmin, dmin), __fadd_rn(qmax, dmax));
    float zp = err > 0.0f ? __fsub_rn(qmin, dmin) : __fsub_rn(qmax, dmax);
    zp = fminf(fmaxf(zp, qmin), qmax);
    row_scale = scale;
    row_zp = __float2int_rn(zp);
    recip_out[blockIdx.x] = recip;
  }
  __syncthreads();
  const float scale = row_scale;
  const int zp = row_zp;
  for (int kk = t; kk < k; kk += 256) {
    float scaled = __fmul_rn(load_float<DT>(inp, base + kk), scale);
    int v = max(-128, min(127, static_cast<int>(roundf(scaled)) + zp)) - zp;
    q[base + kk] = __half_as_ushort(__int2half_rn(v));
  }
}

struct FastEpilogue {
  struct Params {
    const float* recip;  // [m]
    const float* down;   // [n]: the inverse of the power of two folded into each weight row
    const float* bias;   // [n] or NULL
    void* out;
    int out_bf16, vector_ok;
  };
  static constexpr int kSmemBytes = 4 * kBN * 2 * 4;  // per epilogue warp: the tile's biases and column factors
  __device__ static void kernel_begin(const Params&, int) {}
  __device__ static void kernel_end(const Params&, int, bool) {}

  __device__ static void begin_tile(const Params& p, uint8_t* smem, int row0, int col0, int m, int n, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    float* cb = reinterpret_cast<float*>(smem) + warp * 2 * kBN;
    float* cd = cb + kBN;
    __syncwarp();
    for (int i = lane; i < kBN; i += 32) {
      cb[i] = (p.bias != nullptr && col0 + i < n) ? p.bias[col0 + i] : 0.0f;
      cd[i] = col0 + i < n ? p.down[col0 + i] : 0.0f;
    }
    __syncwarp();
  }

  __device__ static void store(const Params& p, const uint8_t* smem, int row, int col_tile0, int col_off, const uint32_t (&acc)[32],
                               int m, int n) {
    if (row >= m) return;
    const int warp = (threadIdx.x >> 5) & 3;
    const float* cb = reinterpret_cast<const float*>(smem) + warp * 2 * kBN + col_off;
    const float* cd = cb + kBN;
    const float recip = p.recip[row];
    const float hi = p.out_bf16 ? 3.38953139e38f : 3.40282347e38f;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) {
      float x = (__uint_as_float(acc[i]) * cd[i]) * recip;  // (the power of two first: exact)
      if (p.bias != nullptr) x += cb[i];
      x = x < -hi ? -hi : x;
      v[i] = hi < x ? hi : x;
    }
    const int col = col_tile0 + col_off;
    const int64_t o = static_cast<int64_t>(row) * n + col;
    if (!p.out_bf16 && p.vector_ok && col + 32 <= n) {
      float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + o);
#pragma unroll
      for (int q = 0; q < 8; q++) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      return;
    }
#pragma unroll
    for (int i = 0; i < 32; i++)
      if (col + i < n) {
        if (p.out_bf16) static_cast<uint16_t*>(p.out)[o + i] = static_cast<uint16_t>(__float_as_uint(v[i]) >> 16);  // truncation
        else static_cast<float*>(p.out)[o + i] = v[i];
      }
  }
};

uint64_t align256(uint64_t x) { return (x + 255) & ~uint64_t(255); }

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" uint64_t tvb_qmm4_fast_prepared_bytes(int64_t n, int64_t k) {
  // flag | per-row power of two | its inverse | float16 weights
  return 256 + 2 * align256(static_cast<uint64_t>(n) * 4) + align256(static_cast<uint64_t>(n) * static_cast<uint64_t>(k) * 2);
}

extern "C" int tvb_qmm4_fast_prepare(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                                     uint64_t prepared_bytes, int* inexact_host) {
  TVB_REQUIRE(n > 0 && k > 0 && bs > 0 && k % 2 == 0 && k % bs == 0 && bs % 2 == 0, "tvb_qmm4_fast_prepare: bad shape");
  TVB_REQUIRE(packed != nullptr && prepared != nullptr && prepared_bytes >= tvb_qmm4_fast_prepared_bytes(n, k),
              "tvb_qmm4_fast_prepare: prepared buffer too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  TVB_CUDA(cudaMemsetAsync(prepared, 0, 256, stream));
  const int64_t nbytes = n * k / 2;
  uint8_t* basep = static_cast<uint8_t*>(prepared);
  float* up = reinterpret_cast<float*>(basep + 256);
  float* down = reinterpret_cast<float*>(basep + 256 + align256(static_cast<uint64_t>(n) * 4));
  uint16_t* wout = reinterpret_cast<uint16_t*>(basep + 256 + 2 * align256(static_cast<uint64_t>(n) * 4));
  const int rgrid = static_cast<int>(ceil_div(n, 256));
  qmm4_fast_row_scale_kernel<<<rgrid, 256, 0, stream>>>(packed + nbytes, n, k / bs, up, down);
  if (launched("qmm4_fast_row_scale", dim3(rgrid), dim3(256), 0, stream) != 0) return -1;
  const int grid = static_cast<int>(std::min<int64_t>(ceil_div(nbytes, 256), static_cast<int64_t>(sm_count(device)) * 16));
  qmm4_fast_prepare_kernel<<<grid, 256, 0, stream>>>(packed, n, k, bs, up, wout, static_cast<int*>(prepared));
  if (launched("qmm4_fast_prepare", dim3(grid), dim3(256), 0, stream) != 0) return -1;
  if (inexact_host != nullptr) {  // once per weight tensor: the caller decides the route from it
    TVB_CUDA(cudaMemcpyAsync(inexact_host, prepared, sizeof(int), cudaMemcpyDeviceToHost, stream));
    TVB_CUDA(cudaStreamSynchronize(stream));
  }
  return 0;
}

extern "C" uint64_t tvb_qmm4_fast_workspace_bytes(int64_t m, int64_t k) {
  return align256(static_cast<uint64_t>(m) * static_cast<uint64_t>(k) * 2) + align256(static_cast<uint64_t>(m) * 4);
}

extern "C" int tvb_qmm4_fast(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                             void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_BF16, "tvb_qmm4_fast: input must be float32 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0 && k > 0 && bs > 0 && k % 8 == 0 && k % bs == 0, "tvb_qmm4_fast: k must be a multiple of 8 and of bs");
  TVB_REQUIRE(m * k < (int64_t(1) << 31) && n * k < (int64_t(1) << 32), "tvb_qmm4_fast: sizes beyond 32 bits");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(inp != nullptr && packed != nullptr && prepared != nullptr && out != nullptr, "tvb_qmm4_fast: NULL pointer");
  TVB_REQUIRE(workspace != nullptr && workspace_bytes >= tvb_qmm4_fast_workspace_bytes(m, k), "tvb_qmm4_fast: workspace too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  uint16_t* q = static_cast<uint16_t*>(workspace);
  float* recip = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + align256(static_cast<uint64_t>(m) * k * 2));
  dim3 qgrid(static_cast<unsigned>(m));
  if (dtype == TVB_F32)
    qmm4_fast_quantize_kernel<TVB_F32><<<qgrid, 256, 0, stream>>>(inp, static_cast<int>(k), bs != k ? 1 : 0, q, recip);
  else
    qmm4_fast_quantize_kernel<TVB_BF16><<<qgrid, 256, 0, stream>>>(inp, static_cast<int>(k), bs != k ? 1 : 0, q, recip);
  if (launched("qmm4_fast_quantize", qgrid, dim3(256), 0, stream) != 0) return -1;

  using Cfg = GemmTcCfg<kBN, FastEpilogue::kSmemBytes>;
  auto kernel = gemm_tc_kernel<2, kBN, FastEpilogue>;
  static bool configured[64] = {};
  if (!configured[device & 63]) {
    TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[device & 63] = true;
  }
  const uint8_t* basep = static_cast<const uint8_t*>(prepared);
  const float* down = reinterpret_cast<const float*>(basep + 256 + align256(static_cast<uint64_t>(n) * 4));
  const void* w = basep + 256 + 2 * align256(static_cast<uint64_t>(n) * 4);
  CUtensorMap map_a, map_b;
  if (make_tensor_map_2d(&map_a, q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, m, k * 2, kGemmStageK / 2, Cfg::kBM, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  if (make_tensor_map_2d(&map_b, w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, n, k * 2, kGemmStageK / 2, kBN, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;
  GemmTcShape sh{};
  sh.m = static_cast<int>(m);
  sh.n = static_cast<int>(n);
  sh.kblocks = static_cast<int>(ceil_div(k * 2, kGemmStageK));
  sh.k_elems_per_block = kGemmStageK / 2;
  sh.tiles_m = static_cast<int>(ceil_div(m, Cfg::kBM));
  sh.tiles_n = static_cast<int>(ceil_div(n, kBN));
  sh.band = Cfg::kBM == 128 ? 16 : 12;
  FastEpilogue::Params ep{};
  const int64_t wcount = n * k / 2, nblocks = k / bs;
  ep.recip = recip;
  ep.down = down;
  ep.bias = has_bias ? packed + wcount + n * nblocks : nullptr;
  ep.out = out;
  ep.out_bf16 = dtype == TVB_BF16;
  ep.vector_ok = (reinterpret_cast<uintptr_t>(out) & 15u) == 0 && (n * 4) % 16 == 0;
  const uint32_t idesc = ptx::tc_instr_desc(1, 0, 0, Cfg::kBM, kBN);  // float32 accumulators, float16 operands
  int* status = nullptr;
  if (status_word(device, &status) != 0) return -1;
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(device), static_cast<int64_t>(sh.tiles_m) * sh.tiles_n));
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_a, map_b, sh, idesc, ep, status);
  return launched("qmm4_fast", dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

// aten::_scaled_mm (and, without scales, aten::mm / addmm of 16-bit floats: tvb_mm at the end of this file, kind::f16
// on the same main loop) on the fifth-generation tensor cores: float8 operands straight into
// tcgen05.mma kind::f8f6f4, float32 accumulation in tensor memory, and the scales, bias,
// 1 / scale_result and the cast to the output type applied as the accumulators are read back.
//
// The reference emulates the op (crates/pyvk/csrc/quant.cpp:283-299): two float8 -> float32
// casts, two multiplications by the scales, a float32 GEMM (linalg.cpp:285-321), a bias add and
// a cast, seven dispatches in all. Float8 products are exact in float32, so
// (sum a*b) * scale_a[i] * scale_b[j] differs from sum (a*scale_a)(b*scale_b) only by
// float32 roundings, inside the bound the reference's test uses (tests/python/test_quant.py:124-128).
#include <atomic>
#include <cstdlib>
#include <mutex>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../core/common.h"
#include "../core/tensormap.h"
#include "gemm_tc.cuh"
#include "gemm_tc2.cuh"
#include "numerics.cuh"
#include "qmm8_skinny.cuh"
#include "scaled_mm.h"

namespace tvb {

extern std::atomic<long long> g_wait_limit_cycles;  // (qmm8.cu; tvb_set_wait_limit_ms)

namespace {

constexpr int kBN = 256;

// RES: the instantiation that also adds a residual matrix (aten::addmm with a full `self`); the others carry no code for it.
// GATHER: the instantiation of a sharded product (tvb_scaled_mm_gather): the tile's rows go into every rank's [m, n_total]
// buffer at this rank's columns (plain 16-byte stores, to peer memory over NVLink), and around its stores the CTA waits for
// the channel's earlier products and reports its own columns, as the sharded decode kernel does (qmm8.cu).
template <int WARPS, bool RES, bool GATHER = false>
struct ScaledEpilogueT {
  struct Params {
    const float* scale_a;
    const float* scale_b;
    const void* bias;
    const float* scale_result;
    const void* residual;
    int64_t residual_ld;
    void* out;
    int bias_dtype, out_dtype, rowwise, vector_ok, residual_dtype, residual_vector_ok;
    // sharded output
    void* outs[kMaxRanks];
    uint32_t* flags[kMaxRanks];
    uint32_t* seq;
    int* done;
    int* status;
    long long wait_limit;
    int64_t out_ld, out_col0;
    int nranks, rank;
    uint32_t independent;
  };
  static constexpr int kScaleBytes = WARPS * kBN * 2 * 4;  // per epilogue warp: column scales and biases of the tile
  static constexpr int kStageBytes = GATHER ? WARPS * 32 * 128 : 0;  // sharded: per warp 32 rows x 64 columns of bfloat16 on their way out
  static constexpr int kSmemBytes = kScaleBytes + kStageBytes;

  __device__ static void kernel_begin(const Params& p, int tid) {
    if constexpr (GATHER) {
      // before a column is stored: every rank has delivered the channel's earlier products (and so has finished reading
      // what this product may be about to overwrite); one warp waits, bounded, one arrival counter per lane
      if (tid < 32) {
        const long long upto = static_cast<long long>(*reinterpret_cast<const volatile uint32_t*>(p.seq)) - 1 - static_cast<long long>(p.independent);
        const long long start = clock64();
        for (int spins = 0; !arrivals_complete_warp(p.flags[p.rank], p.nranks, upto); spins++) {
          if ((spins & 63) == 63) {
            bool stop = *reinterpret_cast<volatile int*>(p.status) != 0;
            if (!stop && clock64() - start > p.wait_limit) {
              atomicExch(p.status, 5);
              stop = true;
            }
            if (__any_sync(0xffffffffu, stop)) break;
          }
        }
      }
      ptx::named_bar_sync(1, WARPS * 32);
    }
  }

  __device__ static void kernel_end(const Params& p, int tid, bool ok) {
    if constexpr (GATHER) {
      ptx::named_bar_sync(1, WARPS * 32);  // (every epilogue thread's stores come before the report)
      if (tid == 0 && ok) {
        if (p.nranks == 1) __threadfence();
        else __threadfence_system();
        arrive_publish(p.flags, p.nranks, p.rank, *reinterpret_cast<const volatile uint32_t*>(p.seq), arrive_share());
        // the last CTA to get here counts the product (the next kernel of the stream reads the count after this one has ended)
        if (atomicAdd(p.done, 1) == static_cast<int>(gridDim.x) - 1) {
          atomicExch(p.done, 0);
          *reinterpret_cast<volatile uint32_t*>(p.seq) = *reinterpret_cast<const volatile uint32_t*>(p.seq) + 1u;
        }
      }
    }
  }

  __device__ static void begin_tile(const Params& p, uint8_t* smem, int row0, int col0, int m, int n, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    float* cs = reinterpret_cast<float*>(smem) + warp * 2 * kBN;
    float* cb = cs + kBN;
    __syncwarp();  // (the previous tile's reads are done)
    for (int i = lane; i < kBN; i += 32) {
      const int col = col0 + i;
      float s = 1.0f, b = 0.0f;
      if (col < n) {
        if (p.scale_b != nullptr) s = p.rowwise ? p.scale_b[col] : p.scale_b[0];
        if (p.bias != nullptr) b = load_float_rt(p.bias, col, p.bias_dtype);
      }
      cs[i] = s;
      cb[i] = b;
    }
    __syncwarp();
  }

  // v += the 32 values of the residual's row `row` from column `col` on (times `inv`, as the product was): 16-byte loads
  // where the row segment is aligned and whole, one value at a time at the matrix's ragged edge.
  __device__ static void add_residual(const Params& p, int row, int col, int n, float inv, float (&v)[32]) {
    const int64_t r = static_cast<int64_t>(row) * p.residual_ld + col;
    if (p.residual_vector_ok && col + 32 <= n) {
      if (p.residual_dtype == TVB_F32) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.residual) + r);
#pragma unroll
        for (int q = 0; q < 8; q++) {
          const float4 x = src[q];
          v[4 * q] += x.x * inv; v[4 * q + 1] += x.y * inv; v[4 * q + 2] += x.z * inv; v[4 * q + 3] += x.w * inv;
        }
        return;
      }
      if (p.residual_dtype == TVB_BF16 || p.residual_dtype == TVB_F16) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) + r);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const uint4 x = src[q];
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float2 f;
            if (p.residual_dtype == TVB_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            v[q * 8 + 2 * j] += f.x * inv;
            v[q * 8 + 2 * j + 1] += f.y * inv;
          }
        }
        return;
      }
    }
    for (int i = 0; i < 32; i++)
      if (col + i < n) v[i] += load_float_rt(p.residual, r + i, p.residual_dtype) * inv;
  }

  __device__ static void store(const Params& p, const uint8_t* smem, int row, int col_tile0, int col_off,
                               const uint32_t (&acc)[32], int m, int n) {
    if (!GATHER && row >= m) return;  // (a sharded product's warps stay together: they exchange rows through shared memory)
    const int warp = (threadIdx.x >> 5) % WARPS;
    const float* cs = reinterpret_cast<const float*>(smem) + warp * 2 * kBN + col_off;
    const float* cb = cs + kBN;
    const float sa = p.scale_a == nullptr ? 1.0f : (p.rowwise ? p.scale_a[row < m ? row : m - 1] : p.scale_a[0]);
    const bool f8_out = p.out_dtype == TVB_E4M3 || p.out_dtype == TVB_E5M2;
    const float inv = f8_out && p.scale_result != nullptr ? 1.0f / p.scale_result[0] : 1.0f;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) {
      float x = __uint_as_float(acc[i]) * sa * cs[i] + cb[i];
      v[i] = f8_out ? x * inv : x;
    }
    const int col = col_tile0 + col_off;
    if constexpr (GATHER) {
      // This rank's columns of every rank's [m, n_total] buffer. A thread holds 64 bytes of one row; stored as they are, a
      // warp's stores would be 32 scattered 16-byte pieces per instruction, which NVLink carries at a fraction of its
      // rate. So the warp collects 64 columns of its 32 rows in shared memory and writes them out as 128-byte row
      // segments: eight lanes per row, four rows per instruction.
      if (p.vector_ok && p.out_dtype == TVB_BF16) {
        const int lane = threadIdx.x & 31;
        const uint32_t stage = ptx::smem_u32(smem) + kScaleBytes + warp * (32 * 128);
        const int half = (col_off >> 5) & 1;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128 + (((half * 4 + q) ^ (lane & 7)) << 4)), "r"(w[0]),
                       "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
        if (half == 1) {
          __syncwarp();
          const int row0 = row - lane, c = lane & 7;
          const int colg = col_tile0 + col_off - 32 + c * 8;
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int r = it * 4 + (lane >> 3);
            if (row0 + r < m && colg + 8 <= n) {
              const uint4 val = ptx::lds128(stage + r * 128 + ((c ^ (r & 7)) << 4));
              const int64_t og = static_cast<int64_t>(row0 + r) * p.out_ld + p.out_col0 + colg;
              for (int rk = 0; rk < p.nranks; rk++) *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.outs[rk]) + og) = val;
            }
          }
          __syncwarp();  // (the staging rows are free again)
        }
        return;
      }
      if (row >= m) return;
      const int64_t og = static_cast<int64_t>(row) * p.out_ld + p.out_col0 + col;
      for (int r = 0; r < p.nranks; r++)
        for (int i = 0; i < 32; i++)
          if (col + i < n) store_float_rt(p.outs[r], og + i, p.out_dtype, v[i]);
      return;
    }
    const int64_t o = static_cast<int64_t>(row) * n + col;
    if constexpr (RES) add_residual(p, row, col, n, inv, v);
    if (p.vector_ok && col + 32 <= n) {
      if (p.out_dtype == TVB_BF16) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + o);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        return;
      }
      if (p.out_dtype == TVB_F32) {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + o);
#pragma unroll
        for (int q = 0; q < 8; q++) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        return;
      }
    }
    for (int i = 0; i < 32; i++)
      if (col + i < n) store_float_rt(p.out, o + i, p.out_dtype, v[i]);
  }
};

}  // namespace

bool scaled_mm_tc_usable(const ScaledMmParams& p) {
  auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  const int64_t es = dtype_size(p.a_dtype);  // 1 (float8) or 2 (float16 / bfloat16): rows must be 16-byte multiples
  if (es != 1 && es != 2) return false;
  return p.m >= 1 && p.n >= 1 && p.k * es >= 16 && p.a_s1 == 1 && p.b_s0 == 1 && (p.a_s0 * es) % 16 == 0 && (p.b_s1 * es) % 16 == 0 &&
         p.a_s0 >= p.k && p.b_s1 >= p.k && aligned(p.a) && aligned(p.b) && p.m < (int64_t(1) << 31) && p.n < (int64_t(1) << 31) &&
         p.k < (int64_t(1) << 30);
}

template <int KIND, int BM, bool RES, bool GATHER = false>
int scaled_mm_tc_tile(int device, cudaStream_t stream, const ScaledMmParams& p) {
  using ScaledEpilogue = ScaledEpilogueT<BM / 32, RES, GATHER>;
  using Cfg = GemmTcCfg<kBN, ScaledEpilogue::kSmemBytes, BM>;
  auto kernel = gemm_tc_kernel<KIND, kBN, ScaledEpilogue, BM>;
  static bool configured[64] = {};
  if (!configured[device & 63]) {
    TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[device & 63] = true;
  }
  const int es = static_cast<int>(dtype_size(p.a_dtype));
  const CUtensorMapDataType dt = es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                         : (p.a_dtype == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  const int k_per_stage = kGemmStageK / es;
  const CUtensorMapSwizzle swz = kGemmStageK == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap map_a, map_b;
  if (make_tensor_map_2d(&map_a, p.a, dt, p.k, p.m, p.a_s0 * es, k_per_stage, Cfg::kBM, swz) != 0) return -1;
  if (make_tensor_map_2d(&map_b, p.b, dt, p.k, p.n, p.b_s1 * es, k_per_stage, kBN, swz) != 0) return -1;
  GemmTcShape sh{};
  sh.m = static_cast<int>(p.m);
  sh.n = static_cast<int>(p.n);
  sh.kblocks = static_cast<int>(ceil_div(p.k, k_per_stage));
  sh.k_elems_per_block = k_per_stage;
  sh.tiles_m = static_cast<int>(ceil_div(p.m, Cfg::kBM));
  sh.tiles_n = static_cast<int>(ceil_div(p.n, kBN));
  sh.band = BM == 128 ? 16 : 12;
  typename ScaledEpilogue::Params ep{};
  ep.scale_a = p.scale_a;
  ep.scale_b = p.scale_b;
  ep.bias = p.bias;
  ep.scale_result = p.scale_result;
  ep.out = p.out;
  ep.bias_dtype = p.bias_dtype;
  ep.out_dtype = p.out_dtype;
  ep.rowwise = p.rowwise;
  ep.vector_ok = (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0 && (p.n * dtype_size(p.out_dtype)) % 16 == 0;
  int* status = nullptr;
  if (status_word(device, &status) != 0) return -1;
  if constexpr (GATHER) {
    const ScaledMmGather& g = *p.gather;
    const int64_t es_out = dtype_size(p.out_dtype);
    ep.vector_ok = (g.n_total * es_out) % 16 == 0 && (p.n * es_out) % 16 == 0;
    for (int r = 0; r < g.world; r++) {
      ep.outs[r] = g.out[r];
      ep.flags[r] = g.flags[r];
      ep.vector_ok = ep.vector_ok && (reinterpret_cast<uintptr_t>(g.out[r]) & 15u) == 0;
    }
    ep.nranks = g.world;
    ep.rank = g.rank;
    ep.seq = g.seq;
    ep.independent = g.independent;
    ep.out_ld = g.n_total;
    ep.out_col0 = static_cast<int64_t>(g.rank) * p.n;
    ep.status = status;
    ep.wait_limit = g_wait_limit_cycles.load();
    void* ws = nullptr;  // the counter of finished CTAs (zero between launches)
    if (workspace(device, 3, 256, &ws) != 0) return -1;
    ep.done = static_cast<int*>(ws);
  }
  ep.residual = p.residual;
  ep.residual_ld = p.residual_ld;
  ep.residual_dtype = p.residual_dtype;
  ep.residual_vector_ok = p.residual != nullptr && (reinterpret_cast<uintptr_t>(p.residual) & 15u) == 0 &&
                          (p.residual_ld * dtype_size(p.residual_dtype)) % 16 == 0;
  // operand formats: kind::f8f6f4 0 = e4m3, 1 = e5m2; kind::f16 0 = float16, 1 = bfloat16; float32 accumulators
  const uint32_t fa = KIND == 0 ? (p.a_dtype == TVB_E4M3 ? 0 : 1) : (p.a_dtype == TVB_F16 ? 0 : 1);
  const uint32_t fb = KIND == 0 ? (p.b_dtype == TVB_E4M3 ? 0 : 1) : (p.b_dtype == TVB_F16 ? 0 : 1);
  const uint32_t idesc = ptx::tc_instr_desc(1, fa, fb, 128, kBN);  // (every MMA covers 128 rows of the tile)
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(device), static_cast<int64_t>(sh.tiles_m) * sh.tiles_n));
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_a, map_b, sh, idesc, ep, status);
  return launched(KIND == 0 ? "scaled_mm_tc" : "mm_tc", dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

// The pair kernel (gemm_tc2.cuh): two CTAs per 256 x 256 tile. How many pairs the device holds at once is asked of the
// runtime once per device (a pair needs both SMs of a TPC).
template <int KIND, bool RES>
int scaled_mm_tc_pair(int device, cudaStream_t stream, const ScaledMmParams& p) {
  using ScaledEpilogue = ScaledEpilogueT<4, RES, false>;
  using Cfg = GemmTc2Cfg<ScaledEpilogue::kSmemBytes>;
  auto kernel = gemm_tc2_kernel<KIND, ScaledEpilogue>;
  static std::mutex mutex;
  static int max_pairs[64] = {};
  const int es = static_cast<int>(dtype_size(p.a_dtype));
  const CUtensorMapDataType dt = es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                         : (p.a_dtype == TVB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  const int k_per_stage = kGemmStageK / es;
  CUtensorMap map_a, map_b;
  if (make_tensor_map_2d(&map_a, p.a, dt, p.k, p.m, p.a_s0 * es, k_per_stage, Cfg::kRows, CU_TENSOR_MAP_SWIZZLE_128B) != 0) return -1;
  if (make_tensor_map_2d(&map_b, p.b, dt, p.k, p.n, p.b_s1 * es, k_per_stage, Cfg::kRows, CU_TENSOR_MAP_SWIZZLE_128B) != 0) return -1;
  GemmTcShape sh{};
  sh.m = static_cast<int>(p.m);
  sh.n = static_cast<int>(p.n);
  sh.kblocks = static_cast<int>(ceil_div(p.k, k_per_stage));
  sh.k_elems_per_block = k_per_stage;
  sh.tiles_m = static_cast<int>(ceil_div(p.m, Cfg::kTile));
  sh.tiles_n = static_cast<int>(ceil_div(p.n, Cfg::kTile));
  static const int band_forced = [] { const char* v = std::getenv("TVB200_GEMM_BAND"); return v != nullptr ? std::atoi(v) : 0; }();
  sh.band = band_forced > 0 ? band_forced : 16;
  typename ScaledEpilogue::Params ep{};
  ep.scale_a = p.scale_a;
  ep.scale_b = p.scale_b;
  ep.bias = p.bias;
  ep.scale_result = p.scale_result;
  ep.out = p.out;
  ep.bias_dtype = p.bias_dtype;
  ep.out_dtype = p.out_dtype;
  ep.rowwise = p.rowwise;
  ep.vector_ok = (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0 && (p.n * dtype_size(p.out_dtype)) % 16 == 0;
  ep.residual = p.residual;
  ep.residual_ld = p.residual_ld;
  ep.residual_dtype = p.residual_dtype;
  ep.residual_vector_ok = p.residual != nullptr && (reinterpret_cast<uintptr_t>(p.residual) & 15u) == 0 &&
                          (p.residual_ld * dtype_size(p.residual_dtype)) % 16 == 0;
  int* status = nullptr;
  if (status_word(device, &status) != 0) return -1;
  const uint32_t fa = KIND == 0 ? (p.a_dtype == TVB_E4M3 ? 0 : 1) : (p.a_dtype == TVB_F16 ? 0 : 1);
  const uint32_t fb = KIND == 0 ? (p.b_dtype == TVB_E4M3 ? 0 : 1) : (p.b_dtype == TVB_F16 ? 0 : 1);
  const uint32_t idesc = ptx::tc_instr_desc(1, fa, fb, Cfg::kTile, Cfg::kTile);  // (one instruction covers the pair's 256 rows)
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int pairs_max = 0;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (max_pairs[device & 63] == 0) {
      TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      cfg.gridDim = dim3(2 * static_cast<unsigned>(sm_count(device) / 2));
      int clusters = 0;
      TVB_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
      TVB_REQUIRE(clusters >= 1, "scaled_mm_tc: the device holds no pair of CTAs of the tile kernel");
      max_pairs[device & 63] = clusters;
    }
    pairs_max = max_pairs[device & 63];
  }
  const int pairs = static_cast<int>(std::min<int64_t>(pairs_max, static_cast<int64_t>(sh.tiles_m) * sh.tiles_n));
  cfg.gridDim = dim3(2 * pairs);
  TVB_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, sh, idesc, ep, status));
  return launched(KIND == 0 ? "scaled_mm_tc2" : "mm_tc2", dim3(2 * pairs), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream);
}

// 256-row tiles keep the tensor pipe fed, but their read-back is not overlapped and there are half as many of them.
// Measured against 128-row tiles (8192 x 8192 outputs): +14 % from 16 KB of k per row on, +6 % at 8 KB, -8 % at 2 KB. They
// are taken when k is long enough and the tiles still fill the SMs as evenly.
template <int KIND>
int scaled_mm_tc_kind(int device, cudaStream_t stream, const ScaledMmParams& p) {
  static const int forced = [] { const char* v = std::getenv("TVB200_GEMM_BM"); return v != nullptr ? std::atoi(v) : 0; }();
  const int64_t sms = sm_count(device);
  const int64_t k_bytes = p.k * static_cast<int64_t>(dtype_size(p.a_dtype));
  const double gain = k_bytes >= 16384 ? 1.14 : (k_bytes >= 8192 ? 1.05 : 0.9);
  auto waves_cost = [&](int64_t bm) {  // time in units of one wave of 128-row tiles
    const int64_t tiles = ceil_div(p.m, bm) * ceil_div(p.n, kBN);
    return static_cast<double>(ceil_div(tiles, sms)) * (bm == 256 ? 2.0 / gain : 1.0);
  };
  bool big = p.m > 128 && waves_cost(256) < waves_cost(128);
  if (forced == 128) big = false;
  if (forced == 256) big = true;
  // The pair kernel (two CTAs per 256 x 256 tile). Measured against the better of the single-CTA tilings, float8: +3 % at
  // 8192^3, +8 % at 4096^3 and at 2048 x 14336 x 4096, +7 % at 16384 x 8192 x 2048, level at 1024 x 8192 x 8192; bfloat16:
  // +3 to +10 % on the same shapes except those with 16 KB of k per row (8192^3, 1024 x 8192 x 8192: -5 %), which keep the
  // single-CTA 256-row tiles.
  static const int pair_forced = [] { const char* v = std::getenv("TVB200_GEMM_PAIR"); return v != nullptr ? std::atoi(v) : -1; }();
  const bool pair_suits = p.m > 256 && p.n >= 512 && (KIND == 0 || k_bytes < 16384);
  const bool pair = p.gather == nullptr && (p.pair != 0 || (pair_forced >= 0 ? pair_forced != 0 && p.m > 128 : pair_suits));
  if (pair) {
    if constexpr (KIND == 2) {
      if (p.residual != nullptr) return scaled_mm_tc_pair<KIND, true>(device, stream, p);
    }
    if (p.residual == nullptr) return scaled_mm_tc_pair<KIND, false>(device, stream, p);
  }
  if constexpr (KIND == 2) {  // (only aten::addmm passes a residual, and only 16-bit operands come with one)
    if (p.residual != nullptr)
      return big ? scaled_mm_tc_tile<KIND, 256, true>(device, stream, p) : scaled_mm_tc_tile<KIND, 128, true>(device, stream, p);
  }
  if (p.residual != nullptr) return fail("scaled_mm_tc: a residual goes with 16-bit operands only");
  if constexpr (KIND == 0) {
    // A sharded product takes 128-row tiles whatever the shape: with their two accumulator buffers the epilogue, whose
    // stores to the peers are paced by NVLink, runs under the next tile's MMAs (256-row tiles have one buffer).
    if (p.gather != nullptr)
      return scaled_mm_tc_tile<KIND, 128, false, true>(device, stream, p);
  }
  if (p.gather != nullptr) return fail("scaled_mm_tc: a sharded output goes with float8 operands only");
  return big ? scaled_mm_tc_tile<KIND, 256, false>(device, stream, p) : scaled_mm_tc_tile<KIND, 128, false>(device, stream, p);
}

int scaled_mm_tc(int device, cudaStream_t stream, const ScaledMmParams& p) {
  return dtype_size(p.a_dtype) == 1 ? scaled_mm_tc_kind<0>(device, stream, p) : scaled_mm_tc_kind<2>(device, stream, p);
}

}  // namespace tvb

using namespace tvb;

extern "C" int tvb_scaled_mm(int device, const void* a, int a_dtype, int64_t a_s0, int64_t a_s1, const void* b, int b_dtype,
                             int64_t b_s0, int64_t b_s1, const float* scale_a, const float* scale_b, int rowwise,
                             const void* bias, int bias_dtype, const float* scale_result, void* out, int out_dtype, int64_t m,
                             int64_t n, int64_t k, int variant) {
  auto is_f8 = [](int dt) { return dt == TVB_E4M3 || dt == TVB_E5M2 || dt == TVB_E4M3FNUZ || dt == TVB_E5M2FNUZ; };
  TVB_REQUIRE(is_f8(a_dtype) && is_f8(b_dtype), "tvb_scaled_mm: operands must be float8 (e4m3fn, e5m2, e4m3fnuz or e5m2fnuz)");
  TVB_REQUIRE(out_dtype == TVB_F32 || out_dtype == TVB_F16 || out_dtype == TVB_BF16 || is_f8(out_dtype),
              "tvb_scaled_mm: unsupported output dtype");
  // the tensor cores take e4m3fn and e5m2 operands; the fnuz formats (operands or output) are decoded / encoded by the plain kernel
  const bool hw_formats = (a_dtype == TVB_E4M3 || a_dtype == TVB_E5M2) && (b_dtype == TVB_E4M3 || b_dtype == TVB_E5M2) &&
                          out_dtype != TVB_E4M3FNUZ && out_dtype != TVB_E5M2FNUZ;
  TVB_REQUIRE(m >= 0 && n >= 0 && k >= 0, "tvb_scaled_mm: negative size");
  TVB_REQUIRE(variant >= 0 && variant <= 3, "tvb_scaled_mm: unknown kernel variant");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(out != nullptr && scale_a != nullptr && scale_b != nullptr && (k == 0 || (a != nullptr && b != nullptr)),
              "tvb_scaled_mm: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  ScaledMmParams p{};
  p.a = a; p.b = b; p.scale_a = scale_a; p.scale_b = scale_b; p.bias = bias; p.scale_result = scale_result; p.out = out;
  p.m = m; p.n = n; p.k = k;
  p.a_s0 = a_s0; p.a_s1 = a_s1; p.b_s0 = b_s0; p.b_s1 = b_s1;
  p.a_dtype = a_dtype; p.b_dtype = b_dtype; p.bias_dtype = bias_dtype; p.out_dtype = out_dtype; p.rowwise = rowwise;
  const bool usable = hw_formats && scaled_mm_tc_usable(p);
  TVB_REQUIRE(variant < 2 || usable, "tvb_scaled_mm: the tcgen05 kernels need e4m3fn / e5m2 K-major operands with 16-byte aligned rows");
  p.pair = variant == 3;
  // small problems do not fill one wave of 128 x 256 tiles: the plain kernel's 64 x 64 tiles spread them wider
  const bool big = m * n >= int64_t(128) * 256 * 8 && k >= 128;
  if (variant >= 2 || (variant == 0 && usable && big)) return scaled_mm_tc(device, stream, p);
  return scaled_mm_plain(stream, p);
}

extern "C" int tvb_scaled_mm_gather(int device, const void* a, int a_dtype, int64_t a_s0, int64_t a_s1, const void* b, int b_dtype,
                                    int64_t b_s0, int64_t b_s1, const float* scale_a, const float* scale_b, int rowwise,
                                    const void* bias, int bias_dtype, const float* scale_result, void* const* c_ranks, int out_dtype,
                                    uint32_t* const* flag_ranks, int world, int rank, uint32_t* seq_counter, int independent,
                                    int64_t m, int64_t n_local, int64_t k) {
  TVB_REQUIRE((a_dtype == TVB_E4M3 || a_dtype == TVB_E5M2) && (b_dtype == TVB_E4M3 || b_dtype == TVB_E5M2),
              "tvb_scaled_mm_gather: operands must be float8_e4m3fn or float8_e5m2");
  TVB_REQUIRE(out_dtype == TVB_F32 || out_dtype == TVB_F16 || out_dtype == TVB_BF16 || out_dtype == TVB_E4M3 || out_dtype == TVB_E5M2,
              "tvb_scaled_mm_gather: unsupported output dtype");
  TVB_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "tvb_scaled_mm_gather: 1 to 8 ranks");
  TVB_REQUIRE(independent >= 0 && independent <= kArriveSlots - 1, "tvb_scaled_mm_gather: independent must be between 0 and 3");
  TVB_REQUIRE(m >= 1 && n_local >= 1 && k >= 1, "tvb_scaled_mm_gather: empty product");
  TVB_REQUIRE(a != nullptr && b != nullptr && scale_a != nullptr && scale_b != nullptr && c_ranks != nullptr && flag_ranks != nullptr &&
                  seq_counter != nullptr,
              "tvb_scaled_mm_gather: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  ScaledMmGather g{};
  for (int r = 0; r < world; r++) {
    TVB_REQUIRE(c_ranks[r] != nullptr && flag_ranks[r] != nullptr, "tvb_scaled_mm_gather: NULL buffer of a rank");
    g.out[r] = c_ranks[r];
    g.flags[r] = flag_ranks[r];
  }
  g.world = world;
  g.rank = rank;
  g.seq = seq_counter;
  g.independent = static_cast<uint32_t>(independent);
  g.n_total = n_local * world;
  ScaledMmParams p{};
  p.a = a; p.b = b; p.scale_a = scale_a; p.scale_b = scale_b; p.bias = bias; p.scale_result = scale_result; p.out = c_ranks[rank];
  p.m = m; p.n = n_local; p.k = k;
  p.a_s0 = a_s0; p.a_s1 = a_s1; p.b_s0 = b_s0; p.b_s1 = b_s1;
  p.a_dtype = a_dtype; p.b_dtype = b_dtype; p.bias_dtype = bias_dtype; p.out_dtype = out_dtype; p.rowwise = rowwise;
  p.gather = &g;
  TVB_REQUIRE(scaled_mm_tc_usable(p), "tvb_scaled_mm_gather: needs K-major operands with 16-byte aligned rows (the tcgen05 kernel)");
  return scaled_mm_tc(device, stream, p);
}

extern "C" int tvb_addmm(int device, const void* a, int dtype, int64_t a_s0, int64_t a_s1, const void* b, int64_t b_s0,
                         int64_t b_s1, const void* bias, int bias_dtype, const void* residual, int residual_dtype,
                         int64_t residual_ld, void* out, int out_dtype, int64_t m, int64_t n, int64_t k, int variant) {
  auto is_float = [](int dt) { return dt == TVB_F32 || dt == TVB_F16 || dt == TVB_BF16; };
  TVB_REQUIRE(is_float(dtype) && is_float(out_dtype), "tvb_mm: float32, float16 or bfloat16 only");
  TVB_REQUIRE(bias == nullptr || is_float(bias_dtype), "tvb_mm: the bias must be float32, float16 or bfloat16");
  TVB_REQUIRE(residual == nullptr || (is_float(residual_dtype) && residual_ld >= n),
              "tvb_addmm: the residual must be float32, float16 or bfloat16 with rows at least n apart");
  TVB_REQUIRE(m >= 0 && n >= 0 && k >= 0, "tvb_mm: negative size");
  TVB_REQUIRE(variant >= 0 && variant <= 3, "tvb_mm: unknown kernel variant");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(out != nullptr && (k == 0 || (a != nullptr && b != nullptr)), "tvb_mm: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  ScaledMmParams p{};
  p.a = a; p.b = b; p.bias = bias; p.out = out;
  p.residual = residual; p.residual_dtype = residual_dtype; p.residual_ld = residual_ld;
  p.m = m; p.n = n; p.k = k;
  p.a_s0 = a_s0; p.a_s1 = a_s1; p.b_s0 = b_s0; p.b_s1 = b_s1;
  p.a_dtype = dtype; p.b_dtype = dtype; p.bias_dtype = bias_dtype; p.out_dtype = out_dtype;
  const bool usable = dtype != TVB_F32 && scaled_mm_tc_usable(p);
  TVB_REQUIRE(variant < 2 || usable, "tvb_mm: the tcgen05 kernels need 16-bit K-major operands with 16-byte aligned rows");
  p.pair = variant == 3;
  const bool big = m * n >= int64_t(128) * 256 * 8 && k >= 64;
  if (variant >= 2 || (variant == 0 && usable && big)) return scaled_mm_tc(device, stream, p);
  return scaled_mm_plain(stream, p);
}

extern "C" int tvb_mm(int device, const void* a, int dtype, int64_t a_s0, int64_t a_s1, const void* b, int64_t b_s0, int64_t b_s1,
                      const void* bias, int bias_dtype, void* out, int out_dtype, int64_t m, int64_t n, int64_t k, int variant) {
  return tvb_addmm(device, a, dtype, a_s0, a_s1, b, b_s0, b_s1, bias, bias_dtype, nullptr, TVB_F32, 0, out, out_dtype, m, n, k,
                   variant);
}

// aten::_dyn_quant_pack_4bit_weight and aten::_dyn_quant_matmul_4bit on sm_100a.
//
// The arithmetic is the reference's qmm4 shader (crates/vkcore/shaders/qmm4.slang),
// itself a copy of PyTorch's CPU reference kernels, and must come out bit for bit:
//   PHASE 0 (qmm4.slang:132-181): per input row, min / max with 0, scale
//     255 / (rmax - rmin) and its reciprocal by correctly rounded divisions, the zero
//     point from the error terms (association differs groupwise / channelwise), rounded
//     to nearest even; q = clamp(round_half_away(v * scale) + zp, -128, 127).
//   PHASE 1 (qmm4.slang:183-247): per block of bs values of k, the int32 sum of
//     (q - zp) * w, converted to float32 and multiplied by the block's scale, added up in
//     block order; then times 1 / scale, plus bias, clamped, stored (bfloat16: truncated).
// Every float32 step is an explicit round-to-nearest intrinsic (__fmul_rn, __fadd_rn,
// __fdiv_rn): the compiler must not contract them into FMAs, which round differently.
//
// Differences in how, not what: q is int8 (the shader keeps int32), the (q - zp) * w sum
// is computed as dot(q, w) - zp * sum(w) with 4-way byte dot products (an integer
// identity), and the packed vector's float-encoded weight bytes (quant.cpp:139-143)
// are decoded as they are staged.
#include "../core/common.h"
#include "numerics.cuh"
#include "ptx.cuh"

namespace tvb {
namespace {

// ------------------------------------------------------------------ pack

__global__ void qmm4_pack_kernel(const uint8_t* __restrict__ w, int64_t nw, const void* __restrict__ scales, int scales_dtype,
                                 int64_t ns, const void* __restrict__ bias, int bias_dtype, int64_t nbias,
                                 float* __restrict__ packed) {
  int64_t total = nw + ns + nbias;
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    float v;
    if (i < nw) v = static_cast<float>(w[i]);
    else if (i < nw + ns) v = load_float_rt(scales, i - nw, scales_dtype);
    else v = load_float_rt(bias, i - nw - ns, bias_dtype);
    packed[i] = v;
  }
}

// ------------------------------------------------------------------ PHASE 0

template <int DT>
__global__ void __launch_bounds__(256) qmm4_quantize_kernel(const void* __restrict__ inp, int k, int groupwise,
                                                            int8_t* __restrict__ q, float* __restrict__ recip_out,
                                                            int32_t* __restrict__ neg_zp_out) {
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
    int izp = __float2int_rn(zp);  // nearest even
    row_scale = scale;
    row_zp = izp;
    recip_out[blockIdx.x] = recip;
    neg_zp_out[blockIdx.x] = -izp;
  }
  __syncthreads();
  const float scale = row_scale;
  const int zp = row_zp;
  for (int kk = t; kk < k; kk += 256) {
    float scaled = __fmul_rn(load_float<DT>(inp, base + kk), scale);
    int v = static_cast<int>(roundf(scaled)) + zp;  // roundf: halfway cases away from zero
    q[base + kk] = static_cast<int8_t>(max(-128, min(127, v)));
  }
}

// ------------------------------------------------------------------ PHASE 1 (bit-exact kernel)

constexpr int kTM = 32, kTN = 64;  // tile of outputs per 256-thread CTA: 2 rows x 4 columns per thread
constexpr int kWordsPad = 9;       // 8 words (32 int8) per row and step, padded against bank conflicts

struct Q4Params {
  const int8_t* q;
  const float* recip;
  const int32_t* neg_zp;
  const float* packed;
  void* out;
  int32_t* iacc_out;
  int m, n, k, bs, has_bias, out_bf16;
};

__global__ void __launch_bounds__(256) qmm4_matmul_kernel(const Q4Params p) {
  __shared__ uint32_t qs[kTM][kWordsPad];
  __shared__ uint32_t ws[kTN][kWordsPad];
  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  const int64_t rstride = (p.k + 1) / 2;
  const int64_t wcount = static_cast<int64_t>(p.n) * p.k / 2;
  const int nblocks = (p.k + p.bs - 1) / p.bs;

  int off[2];
#pragma unroll
  for (int r = 0; r < 2; r++) off[r] = p.neg_zp[min(m0 + ty * 2 + r, p.m - 1)];
  float main_acc[2][4];
  int iacc[2][4];
#pragma unroll
  for (int r = 0; r < 2; r++)
#pragma unroll
    for (int c = 0; c < 4; c++) {
      main_acc[r][c] = 0.0f;
      iacc[r][c] = 0;
    }
  bool first = true;

  for (int k0 = 0; k0 < p.k; k0 += 32) {
    __syncthreads();  // (the previous step's tiles consumed)
    {  // q: 32 rows x 8 words, one word per thread
      int r = t >> 3, wd = t & 7;
      int row = m0 + r, kb = k0 + wd * 4;
      uint32_t v = 0;
      if (row < p.m) {
        const int8_t* src = p.q + static_cast<int64_t>(row) * p.k + kb;
        if (kb + 3 < p.k && ((reinterpret_cast<uintptr_t>(src) & 3u) == 0)) {
          v = *reinterpret_cast<const uint32_t*>(src);
        } else {
#pragma unroll
          for (int i = 0; i < 4; i++)
            if (kb + i < p.k) v |= static_cast<uint32_t>(static_cast<uint8_t>(src[i])) << (8 * i);
        }
      }
      qs[r][wd] = v;
    }
    {  // weights: 64 rows x 16 float-encoded bytes; four bytes (eight weights, two words) per thread
      int r = t >> 2, part = t & 3;
      int row = min(n0 + r, p.n - 1);
      uint32_t lo = 0, hi = 0;  // words 2*part and 2*part+1
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int kk = k0 + part * 8 + i * 2;  // the byte holds k = kk (low nibble) and kk + 1 (high nibble)
        uint32_t byte = kk < p.k ? static_cast<uint32_t>(p.packed[row * rstride + kk / 2]) : 0x88u;
        uint32_t w0 = ((byte & 15u) - 8u) & 0xffu;
        uint32_t w1 = kk + 1 < p.k ? (((byte >> 4) - 8u) & 0xffu) : 0u;
        if (kk >= p.k) w0 = 0u;
        uint32_t pair = w0 | (w1 << 8);
        if (i < 2) lo |= pair << (16 * i);
        else hi |= pair << (16 * (i - 2));
      }
      ws[r][part * 2] = lo;
      ws[r][part * 2 + 1] = hi;
    }
    __syncthreads();
    int wsum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int wd = 0; wd < 8; wd++) {
      uint32_t qv[2], wv[4];
#pragma unroll
      for (int r = 0; r < 2; r++) qv[r] = qs[ty * 2 + r][wd];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        wv[c] = ws[tx * 4 + c][wd];
        wsum[c] = __dp4a(static_cast<int>(wv[c]), 0x01010101, wsum[c]);
      }
#pragma unroll
      for (int r = 0; r < 2; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) iacc[r][c] = __dp4a(static_cast<int>(qv[r]), static_cast<int>(wv[c]), iacc[r][c]);
    }
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
      for (int c = 0; c < 4; c++) iacc[r][c] += off[r] * wsum[c];

    if ((k0 + 32) % p.bs == 0 || k0 + 32 >= p.k) {
      const int blk = k0 / p.bs;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int col = min(n0 + tx * 4 + c, p.n - 1);
        const float s = p.packed[wcount + static_cast<int64_t>(col) * nblocks + blk];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          if (p.iacc_out != nullptr) {
            int row = m0 + ty * 2 + r, cc = n0 + tx * 4 + c;
            if (row < p.m && cc < p.n) p.iacc_out[(static_cast<int64_t>(row) * p.n + cc) * nblocks + blk] = iacc[r][c];
          }
          float x = __fmul_rn(static_cast<float>(iacc[r][c]), s);
          main_acc[r][c] = first ? x : __fadd_rn(main_acc[r][c], x);  // (the first block assigns: keeps -0)
          iacc[r][c] = 0;
        }
      }
      first = false;
    }
  }

#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int row = m0 + ty * 2 + r;
    if (row >= p.m) continue;
    const float recip = p.recip[row];
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const int col = n0 + tx * 4 + c;
      if (col >= p.n) continue;
      float v = __fmul_rn(main_acc[r][c], recip);
      if (p.has_bias) v = __fadd_rn(v, p.packed[wcount + static_cast<int64_t>(p.n) * nblocks + col]);
      const float hi = p.out_bf16 ? 3.38953139e38f : 3.40282347e38f;
      v = v < -hi ? -hi : v;  // (std::max / std::min: NaN passes)
      v = hi < v ? hi : v;
      const int64_t o = static_cast<int64_t>(row) * p.n + col;
      if (p.out_bf16) static_cast<uint16_t*>(p.out)[o] = static_cast<uint16_t>(__float_as_uint(v) >> 16);  // truncation
      else static_cast<float*>(p.out)[o] = v;
    }
  }
}

int check_shape(int64_t m, int64_t n, int64_t k, int64_t bs) {
  TVB_REQUIRE(m >= 0 && n >= 0 && k > 0 && bs > 0, "tvb_qmm4: bad size");
  TVB_REQUIRE(bs == k || (bs % 32 == 0 && k % bs == 0), "tvb_qmm4: block size must be k or a multiple of 32 dividing k");
  TVB_REQUIRE(m * (k > n ? k : n) < (int64_t(1) << 31) && n * k < (int64_t(1) << 32), "tvb_qmm4: sizes beyond 32 bits");
  return 0;
}

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" int tvb_qmm4_pack(int device, const uint8_t* weights, int64_t nw, const void* scales, int scales_dtype, int64_t ns,
                             const void* bias, int bias_dtype, int64_t nbias, float* packed) {
  TVB_REQUIRE(nw >= 0 && ns >= 0 && nbias >= 0, "tvb_qmm4_pack: negative size");
  TVB_REQUIRE(scales_dtype == TVB_F32 || scales_dtype == TVB_BF16 || scales_dtype == TVB_F16 || scales_dtype == TVB_F64,
              "tvb_qmm4_pack: scales must be a float tensor");
  TVB_REQUIRE(nbias == 0 || bias_dtype == TVB_F32 || bias_dtype == TVB_BF16 || bias_dtype == TVB_F16 || bias_dtype == TVB_F64,
              "tvb_qmm4_pack: bias must be a float tensor");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  int64_t total = nw + ns + nbias;
  if (total == 0) return 0;
  TVB_REQUIRE(packed != nullptr && (nw == 0 || weights != nullptr) && (ns == 0 || scales != nullptr) &&
                  (nbias == 0 || bias != nullptr),
              "tvb_qmm4_pack: NULL pointer");
  int grid = static_cast<int>(std::min<int64_t>(ceil_div(total, 256), static_cast<int64_t>(sm_count(device)) * 16));
  qmm4_pack_kernel<<<grid, 256, 0, stream>>>(weights, nw, scales, scales_dtype, ns, bias, bias_dtype, nbias, packed);
  return launched("qmm4_pack", dim3(grid), dim3(256), 0, stream);
}

extern "C" int tvb_qmm4_quantize(int device, const void* inp, int dtype, int64_t m, int64_t k, int groupwise, int8_t* q,
                                 float* recip, int32_t* neg_zp) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_BF16, "tvb_qmm4_quantize: input must be float32 or bfloat16");
  TVB_REQUIRE(m >= 0 && k > 0 && m * k < (int64_t(1) << 31), "tvb_qmm4_quantize: bad size");
  if (m == 0) return 0;
  TVB_REQUIRE(inp != nullptr && q != nullptr && recip != nullptr && neg_zp != nullptr, "tvb_qmm4_quantize: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  dim3 grid(static_cast<unsigned>(m));
  if (dtype == TVB_F32)
    qmm4_quantize_kernel<TVB_F32><<<grid, 256, 0, stream>>>(inp, static_cast<int>(k), groupwise, q, recip, neg_zp);
  else
    qmm4_quantize_kernel<TVB_BF16><<<grid, 256, 0, stream>>>(inp, static_cast<int>(k), groupwise, q, recip, neg_zp);
  return launched("qmm4_quantize", grid, dim3(256), 0, stream);
}

extern "C" int tvb_qmm4_matmul(int device, const int8_t* q, const float* recip, const int32_t* neg_zp, const float* packed,
                               int has_bias, void* out, int dtype, int64_t m, int64_t n, int64_t k, int64_t bs,
                               int32_t* iacc_out) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_BF16, "tvb_qmm4_matmul: output must be float32 or bfloat16");
  if (check_shape(m, n, k, bs) != 0) return -1;
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(q != nullptr && recip != nullptr && neg_zp != nullptr && packed != nullptr && out != nullptr,
              "tvb_qmm4_matmul: NULL pointer");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  Q4Params p{};
  p.q = q;
  p.recip = recip;
  p.neg_zp = neg_zp;
  p.packed = packed;
  p.out = out;
  p.iacc_out = iacc_out;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.bs = static_cast<int>(bs);
  p.has_bias = has_bias;
  p.out_bf16 = dtype == TVB_BF16;
  dim3 grid(static_cast<unsigned>(ceil_div(n, kTN)), static_cast<unsigned>(ceil_div(m, kTM)));
  TVB_REQUIRE(grid.y <= 65535, "tvb_qmm4_matmul: too many rows for one launch");
  qmm4_matmul_kernel<<<grid, 256, 0, stream>>>(p);
  return launched("qmm4_matmul", grid, dim3(256), 0, stream);
}

extern "C" uint64_t tvb_qmm4_workspace_bytes(int64_t m, int64_t k) {
  uint64_t q = (static_cast<uint64_t>(m) * static_cast<uint64_t>(k) + 255) & ~uint64_t(255);
  uint64_t rows = (static_cast<uint64_t>(m) * 4 + 255) & ~uint64_t(255);
  return q + 2 * rows;
}

extern "C" int tvb_qmm4(int device, const void* inp, int dtype, const float* packed, int has_bias, void* out, int64_t m,
                        int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes) {
  if (check_shape(m, n, k, bs) != 0) return -1;
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(workspace != nullptr && workspace_bytes >= tvb_qmm4_workspace_bytes(m, k), "tvb_qmm4: workspace too small");
  uint64_t qbytes = (static_cast<uint64_t>(m) * static_cast<uint64_t>(k) + 255) & ~uint64_t(255);
  uint64_t rbytes = (static_cast<uint64_t>(m) * 4 + 255) & ~uint64_t(255);
  int8_t* q = static_cast<int8_t*>(workspace);
  float* recip = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + qbytes);
  int32_t* neg_zp = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + qbytes + rbytes);
  if (tvb_qmm4_quantize(device, inp, dtype, m, k, bs != k ? 1 : 0, q, recip, neg_zp) != 0) return -1;
  return tvb_qmm4_matmul(device, q, recip, neg_zp, packed, has_bias, out, dtype, m, n, k, bs, nullptr);
}

// aten::_scaled_mm, the plain kernel: any strides, any float8 pair, any size (and, without scales, aten::mm / addmm
// of float32, float16 or bfloat16 matrices that the tcgen05 kernel does not take).
//
// Follows the reference's emulated product step by step (crates/pyvk/csrc/quant.cpp:283-299):
// each operand upcast exactly to float32 and multiplied by its scale (a 0-dim scale or a
// row-wise [m, 1] / [1, n] one), a float32 product sum, the bias added, float8 outputs
// multiplied by 1 / scale_result, one rounding to the output type. The reference spends
// seven dispatches and a generic float32 GEMM on this (quant.cpp:283-299, linalg.cpp:285-321);
// here it is one kernel: 64 x 64 output tiles, 16 values of k staged per step, 4 x 4 outputs
// per thread. The tcgen05 kernel in scaled_mm_tc.cu takes the large aligned shapes; this one
// takes the rest (odd sizes, transposed layouts, tiny problems).
#include "../core/common.h"
#include "numerics.cuh"
#include "scaled_mm.h"

namespace tvb {
namespace {

constexpr int kBM = 64, kBN = 64, kTK = 16;

__global__ void __launch_bounds__(256) scaled_mm_plain_kernel(const ScaledMmParams p) {
  __shared__ float as[kTK][kBM + 1];
  __shared__ float bs[kTK][kBN + 1];
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int64_t row0 = static_cast<int64_t>(blockIdx.y) * kBM, col0 = static_cast<int64_t>(blockIdx.x) * kBN;
  const bool scaled = p.scale_a != nullptr;  // (aten::mm / addmm come through here without scales)
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

  for (int64_t k0 = 0; k0 < p.k; k0 += kTK) {
    __syncthreads();
    for (int e = t; e < kBM * kTK; e += 256) {
      // consecutive threads along whichever of A's dimensions is contiguous
      int r = p.a_s1 == 1 ? e / kTK : e % kBM, kk = p.a_s1 == 1 ? e % kTK : e / kBM;
      int64_t gm = row0 + r, gk = k0 + kk;
      float v = 0.0f;
      if (gm < p.m && gk < p.k) {
        v = load_float_rt(p.a, gm * p.a_s0 + gk * p.a_s1, p.a_dtype);
        if (scaled) v *= p.scale_a[p.rowwise ? gm : 0];
      }
      as[kk][r] = v;
    }
    for (int e = t; e < kBN * kTK; e += 256) {
      int c = p.b_s0 == 1 ? e / kTK : e % kBN, kk = p.b_s0 == 1 ? e % kTK : e / kBN;
      int64_t gn = col0 + c, gk = k0 + kk;
      float v = 0.0f;
      if (gn < p.n && gk < p.k) {
        v = load_float_rt(p.b, gk * p.b_s0 + gn * p.b_s1, p.b_dtype);
        if (scaled) v *= p.scale_b[p.rowwise ? gn : 0];
      }
      bs[kk][c] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = as[kk][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = bs[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }

  const bool f8_out = p.out_dtype == TVB_E4M3 || p.out_dtype == TVB_E5M2 || p.out_dtype == TVB_E4M3FNUZ || p.out_dtype == TVB_E5M2FNUZ;
  const float inv = f8_out && p.scale_result != nullptr ? 1.0f / p.scale_result[0] : 1.0f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int64_t gm = row0 + ty + 16 * i;
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int64_t gn = col0 + tx + 16 * j;
      if (gn >= p.n) continue;
      float v = acc[i][j];
      if (p.bias != nullptr) v += load_float_rt(p.bias, gn, p.bias_dtype);
      if (p.residual != nullptr) v += load_float_rt(p.residual, gm * p.residual_ld + gn, p.residual_dtype);
      if (f8_out) v *= inv;
      store_float_rt(p.out, gm * p.n + gn, p.out_dtype, v);
    }
  }
}

}  // namespace

int scaled_mm_plain(cudaStream_t stream, const ScaledMmParams& p) {
  dim3 grid(static_cast<unsigned>(ceil_div(p.n, kBN)), static_cast<unsigned>(ceil_div(p.m, kBM)));
  if (grid.y > 65535) return fail("tvb_scaled_mm: too many rows for one launch");
  scaled_mm_plain_kernel<<<grid, 256, 0, stream>>>(p);
  return launched("scaled_mm_plain", grid, dim3(256), 0, stream);
}

}  // namespace tvb

// Parameters shared by the two aten::_scaled_mm kernels (plain and tcgen05), which also serve aten::mm / addmm
// (operands of one 16- or 32-bit float type, no scales).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace tvb {

// A product whose output columns are one rank's slice of a [m, n_total] output kept on every rank of a node: the epilogue
// stores into every rank's buffer and reports on the channel of tvb_qmm8_gather.
struct ScaledMmGather {
  void* out[8];          // every rank's [m, n_total] buffer (this rank's own included)
  uint32_t* flags[8];    // every rank's arrival counters
  int world, rank;
  uint32_t* seq;         // this rank's product count
  uint32_t independent;
  int64_t n_total;
};

struct ScaledMmParams {
  const void* a;         // [m, k]: element (i, kk) at a[i * a_s0 + kk * a_s1]
  const void* b;         // [k, n]: element (kk, j) at b[kk * b_s0 + j * b_s1]
  const float* scale_a;  // 1 or m values; NULL (with scale_b): no scaling
  const float* scale_b;  // 1 or n values
  const void* bias;      // n values of bias_dtype, or NULL
  const float* scale_result;  // 1 value or NULL (float8 outputs only)
  const void* residual;  // [m, n] of residual_dtype added to the product before the rounding (row i at residual + i * residual_ld), or NULL
  void* out;             // contiguous [m, n] of out_dtype
  int64_t m, n, k;
  int64_t a_s0, a_s1, b_s0, b_s1;
  int64_t residual_ld;
  int a_dtype, b_dtype, bias_dtype, out_dtype, rowwise, residual_dtype;
  const ScaledMmGather* gather = nullptr;  // sharded output (float8 operands on the tcgen05 kernel only)
  int pair = 0;          // 1: the kernel of CTA pairs whatever the shape (variant 3 of the entry points)
};

int scaled_mm_plain(cudaStream_t stream, const ScaledMmParams& p);
// The tcgen05 kernel; `usable` tells whether the layout qualifies (K-major operands,
// 16-byte aligned rows).
bool scaled_mm_tc_usable(const ScaledMmParams& p);
int scaled_mm_tc(int device, cudaStream_t stream, const ScaledMmParams& p);  // float8 (kind::f8f6f4) or float16 / bfloat16 (kind::f16)

}  // namespace tvb

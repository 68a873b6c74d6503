// PHASE 0 of aten::_dyn_quant_matmul_4bit, the per-row arithmetic (crates/vkcore/shaders/qmm4.slang:119-181, which follows
// ATen/native/cpu/int4mm_kernel.cpp's ref_dyn_quant_matmul_4bit_* step by step): from a row's minimum and maximum to its
// scale, 1 / scale and zero point, and from a value to its int8 code. Every float32 operation is an explicit round-to-nearest
// intrinsic (no contraction), so the kernels that share these helpers produce the CPU's bits.
#pragma once

#include <cuda_runtime.h>

namespace tvb {

struct Phase0Row {
  float scale, recip;
  int zero_point;
};

__device__ __forceinline__ Phase0Row phase0_row(float mn, float mx, int groupwise) {
  const float qmin = -128.0f, qmax = 127.0f;
  const float rmin = fminf(0.0f, mn), rmax = fmaxf(0.0f, mx);
  Phase0Row row;
  row.scale = rmin == rmax ? 1.0f : __fdiv_rn(qmax - qmin, __fsub_rn(rmax, rmin));
  row.recip = row.scale != 0.0f ? __fdiv_rn(1.0f, row.scale) : 0.0f;
  const float dmin = __fmul_rn(rmin, row.scale), dmax = __fmul_rn(rmax, row.scale);
  const float err = groupwise ? __fadd_rn(__fadd_rn(__fadd_rn(qmin, dmin), qmax), dmax)
                              : __fadd_rn(__fadd_rn(qmin, dmin), __fadd_rn(qmax, dmax));
  float zp = err > 0.0f ? __fsub_rn(qmin, dmin) : __fsub_rn(qmax, dmax);
  zp = fminf(fmaxf(zp, qmin), qmax);
  row.zero_point = __float2int_rn(zp);  // ties to even
  return row;
}

__device__ __forceinline__ int phase0_code(float x, float scale, int zero_point) {
  const int v = static_cast<int>(roundf(__fmul_rn(x, scale))) + zero_point;  // halfway away from zero
  return max(-128, min(127, v));
}

}  // namespace tvb

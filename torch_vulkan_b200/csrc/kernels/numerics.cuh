// Device-side number formats: loads and rounding stores of the element types
// the quantised products use, bit for bit as the reference's shaders (and c10)
// convert them:
//   bfloat16 store: nearest even, NaN -> 0x7fc0 (qmm8.slang:58-63, cast.slang:31-39)
//   float16 store:  nearest even (_half.slang:8-43)
//   float8:         c10's conversions, which the reference tabulates
//                   (crates/pyvk/csrc/backend.cpp:486-534): e4m3fn has no
//                   infinity and overflows to NaN (0x7f), e5m2 overflows to inf.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "tvb200.h"

namespace tvb {

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t x) { return __uint_as_float(static_cast<uint32_t>(x) << 16); }

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  if (f != f) return 0x7fc0;
  uint32_t u = __float_as_uint(f);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

__device__ __forceinline__ float f16_bits_to_f32(uint16_t x) { return __half2float(__ushort_as_half(x)); }

__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
  if (f != f) return static_cast<uint16_t>(((__float_as_uint(f) >> 16) & 0x8000u) | 0x7e00u);
  return __half_as_ushort(__float2half_rn(f));
}

// kind 0: e4m3fn, kind 1: e5m2, kind 2: e4m3fnuz (bias 8), kind 3: e5m2fnuz (bias 16). The fnuz formats have no
// infinities and no negative zero, and their one NaN is 0x80 (the reference tabulates them from c10's conversions too:
// crates/pyvk/csrc/backend.cpp:471-477).
__device__ __forceinline__ float f8_bits_to_f32(uint8_t c, int kind) {
  if (kind == 1) return __half2float(__ushort_as_half(static_cast<uint16_t>(c) << 8));  // e5m2 is float16's top byte
  const uint32_t sign = static_cast<uint32_t>(c & 0x80u) << 24;
  if (kind >= 2) {
    if (c == 0x80u) return __uint_as_float(0x7fc00000u);
    const int mbits = kind == 2 ? 3 : 2, bias = kind == 2 ? 8 : 16;
    const uint32_t e = (c & 0x7fu) >> mbits, m = c & ((1u << mbits) - 1u);
    // (2^(1 - bias - mbits) and 2^(e - bias) as float32 bit patterns: exact)
    const float v = e == 0 ? static_cast<float>(m) * __uint_as_float(static_cast<uint32_t>(127 + 1 - bias - mbits) << 23)
                           : __uint_as_float(((e + 127u - bias) << 23) | (m << (23 - mbits)));
    return __uint_as_float(__float_as_uint(v) | sign);
  }
  uint32_t e = (c >> 3) & 0xfu, m = c & 7u;
  if ((c & 0x7fu) == 0x7fu) return __uint_as_float(sign | 0x7fc00000u);
  float v;
  if (e == 0) v = static_cast<float>(m) * 0.001953125f;  // m * 2^-9
  else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
  return __uint_as_float(__float_as_uint(v) | sign);
}

__device__ __forceinline__ uint8_t f32_to_f8_bits(float f, int kind) {
  const bool fnuz = kind >= 2;
  const int mbits = (kind & 1) == 0 ? 3 : 2, bias = ((kind & 1) == 0 ? 7 : 15) + (fnuz ? 1 : 0);
  uint32_t u = __float_as_uint(f);
  uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
  uint32_t mag = u & 0x7fffffffu;
  if (fnuz && mag >= 0x7f800000u) return 0x80;  // NaN and the infinities: the one NaN
  if (mag > 0x7f800000u) return sign | 0x7f;
  if (mag == 0x7f800000u) return sign | (kind == 0 ? 0x7f : 0x7c);
  if (mag < 0x00800000u) return fnuz ? 0 : sign;  // zero and float32 denormals: far below half the smallest float8
  int e = static_cast<int>(mag >> 23) - 127;
  uint32_t m = (mag & 0x7fffffu) | 0x800000u;
  int emin = 1 - bias;
  int shift = 23 - mbits + (e < emin ? emin - e : 0);
  if (shift > 24) return fnuz ? 0 : sign;  // below half of the smallest denormal (24: exactly half or less -> 0 or tie to even 0)
  uint32_t half = 1u << (shift - 1);
  uint32_t r = m >> shift, rem = m & ((1u << shift) - 1u);
  if (rem > half || (rem == half && (r & 1u))) r++;
  uint32_t code = e < emin ? r : (static_cast<uint32_t>(e - emin + 1) << mbits) + (r - (1u << mbits));
  if (fnuz) {
    if (code > 0x7fu) return 0x80;  // beyond the largest value: NaN (no saturation)
    return code == 0u ? 0 : sign | static_cast<uint8_t>(code);  // (no negative zero)
  }
  if (kind == 0) code = code > 0x7eu ? 0x7fu : code;
  else code = code > 0x7cu ? 0x7cu : code;
  return sign | static_cast<uint8_t>(code);
}

// Loads element i of a float tensor of `dtype` (F32, F16, BF16) as float32.
template <int DT>
__device__ __forceinline__ float load_float(const void* p, int64_t i) {
  if (DT == TVB_F32) return static_cast<const float*>(p)[i];
  if (DT == TVB_F16) return f16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
  return bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
}

// Rounds once (to nearest even) and stores element i of a tensor of `dtype`.
template <int DT>
__device__ __forceinline__ void store_float(void* p, int64_t i, float v) {
  if (DT == TVB_F32) static_cast<float*>(p)[i] = v;
  else if (DT == TVB_F16) static_cast<uint16_t*>(p)[i] = f32_to_f16_bits(v);
  else static_cast<uint16_t*>(p)[i] = f32_to_bf16_bits(v);
}

// Runtime-dtype variants for the epilogues that take an output / bias dtype.
__device__ __forceinline__ float load_float_rt(const void* p, int64_t i, int dtype) {
  switch (dtype) {
    case TVB_F32: return static_cast<const float*>(p)[i];
    case TVB_F16: return f16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
    case TVB_BF16: return bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
    case TVB_E4M3: return f8_bits_to_f32(static_cast<const uint8_t*>(p)[i], 0);
    case TVB_E5M2: return f8_bits_to_f32(static_cast<const uint8_t*>(p)[i], 1);
    case TVB_E4M3FNUZ: return f8_bits_to_f32(static_cast<const uint8_t*>(p)[i], 2);
    case TVB_E5M2FNUZ: return f8_bits_to_f32(static_cast<const uint8_t*>(p)[i], 3);
    case TVB_F64: return static_cast<float>(static_cast<const double*>(p)[i]);
    default: return 0.0f;
  }
}

__device__ __forceinline__ void store_float_rt(void* p, int64_t i, int dtype, float v) {
  switch (dtype) {
    case TVB_F32: static_cast<float*>(p)[i] = v; break;
    case TVB_F16: static_cast<uint16_t*>(p)[i] = f32_to_f16_bits(v); break;
    case TVB_BF16: static_cast<uint16_t*>(p)[i] = f32_to_bf16_bits(v); break;
    case TVB_E4M3: static_cast<uint8_t*>(p)[i] = f32_to_f8_bits(v, 0); break;
    case TVB_E5M2: static_cast<uint8_t*>(p)[i] = f32_to_f8_bits(v, 1); break;
    case TVB_E4M3FNUZ: static_cast<uint8_t*>(p)[i] = f32_to_f8_bits(v, 2); break;
    case TVB_E5M2FNUZ: static_cast<uint8_t*>(p)[i] = f32_to_f8_bits(v, 3); break;
    default: break;
  }
}

}  // namespace tvb

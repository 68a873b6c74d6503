/*
 * CPU restatement of torch-vulkan's quantised matrix products, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker that the CUDA kernels are
 * compared against; nothing that ships calls it. Only tests, the smoke check
 * and the benchmark's CPU-baseline leg may load the library built from it.
 *
 * Each function follows the reference's own statement of the arithmetic:
 *
 *   oracle_qmm8_*        crates/vkcore/shaders/qmm8.slang:45-67 (load / round
 *                        rules), :78-111 (matrix-vector path), :113-173 (tiles)
 *   oracle_qmm4_pack     crates/pyvk/csrc/quant.cpp:127-144
 *   oracle_qmm4_quantize crates/vkcore/shaders/qmm4.slang:132-181 (PHASE 0)
 *   oracle_qmm4_matmul   crates/vkcore/shaders/qmm4.slang:183-247 (PHASE 1)
 *   oracle_scaled_mm     crates/pyvk/csrc/quant.cpp:283-299 (the emulated
 *                        float8 product), cast.slang:31-39 (bfloat16 RNE),
 *                        _half.slang:8-43 (float16 RNE), backend.cpp:486-534
 *                        (float8 tables = c10's conversions)
 *
 * The shaders copy PyTorch's CPU kernels (ATen/native/cpu/int8mm_kernel.cpp,
 * int4mm_kernel.cpp ref_dyn_quant_matmul_4bit_*, ScaledBlas.cpp
 * _scaled_mm_out_cpu_emulated; the reference pins torch 2.14.1). Parity is
 * pinned by checking this restatement bit for bit against the installed
 * PyTorch's CPU ops on the reference's own test shapes (tests/test_oracle.py)
 * and against the committed golden vectors made from those ops.
 *
 * Build with -ffp-contract=off: the dyn-int4 arithmetic must not be fused.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* ---- 16-bit float formats ------------------------------------------------ */

float oracle_bf16_to_f32(uint16_t x) { return bits_f32((uint32_t)x << 16); }

/* qmm8.slang:58-63 / cast.slang:31-39: nearest even, NaN -> 0x7fc0. */
uint16_t oracle_f32_to_bf16(float f) {
  if (isnan(f)) return 0x7fc0;
  uint32_t u = f32_bits(f);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ff;
  if (e == 0) {
    if (m == 0) return bits_f32(sign);
    float v = (float)m * 5.9604644775390625e-8f; /* m * 2^-24 */
    return sign ? -v : v;
  }
  if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
  return bits_f32(sign | ((e + 112) << 23) | (m << 13));
}

/* _half.slang:8-43: float32 -> float16, round to nearest even. */
uint16_t oracle_f32_to_f16(float f) {
  uint32_t u = f32_bits(f);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t mag = u & 0x7fffffffu;
  if (mag > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);            /* NaN */
  if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);           /* >= 65520 -> inf */
  if (mag < 0x33000001u) return (uint16_t)sign;                        /* <= 2^-25 -> 0 */
  int e = (int)(mag >> 23) - 127;
  uint32_t m = (mag & 0x7fffffu) | 0x800000u;
  int shift = e < -14 ? 13 + (-14 - e) : 13;
  uint32_t half = 1u << (shift - 1);
  uint32_t r = m >> shift, rem = m & ((1u << shift) - 1);
  if (rem > half || (rem == half && (r & 1u))) r++;
  uint32_t out = e < -14 ? r : ((uint32_t)(e + 15) << 10) + (r - 0x400u);
  return (uint16_t)(sign | out);
}

/* ---- float8 (c10's conversions: the reference builds its tables from them,
 *      backend.cpp:486-534) ------------------------------------------------ */

/* kind 0: e4m3fn (bias 7, no inf, NaN 0x7f), kind 1: e5m2 (IEEE-like), kind 2: e4m3fnuz (bias 8), kind 3: e5m2fnuz
 * (bias 16). The fnuz formats have no infinities and no negative zero; their one NaN is 0x80 (backend.cpp:471-477). */
float oracle_f8_to_f32(uint8_t c, int kind) {
  int fnuz = kind >= 2, ebits = (kind & 1) == 0 ? 4 : 5, mbits = 7 - ebits;
  int bias = (ebits == 4 ? 7 : 15) + fnuz;
  int sign = c >> 7, e = (c >> mbits) & ((1 << ebits) - 1), m = c & ((1 << mbits) - 1);
  float v;
  if (fnuz && c == 0x80) return NAN;
  if (kind == 0 && (c & 0x7f) == 0x7f) v = NAN;
  else if (kind == 1 && e == 31) v = m ? NAN : INFINITY;
  else if (e == 0) v = ldexpf((float)m, 1 - bias - mbits);
  else v = ldexpf((float)(m | (1 << mbits)), e - bias - mbits);
  return sign ? -v : v;
}

uint8_t oracle_f32_to_f8(float f, int kind) {
  int fnuz = kind >= 2, ebits = (kind & 1) == 0 ? 4 : 5, mbits = 7 - ebits;
  int bias = (ebits == 4 ? 7 : 15) + fnuz;
  uint32_t u = f32_bits(f);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t mag = u & 0x7fffffffu;
  if (fnuz && mag >= 0x7f800000u) return 0x80;                          /* NaN and infinities: the one NaN */
  if (mag > 0x7f800000u) return (uint8_t)(sign | 0x7f);                 /* NaN */
  if (mag == 0x7f800000u) return (uint8_t)(sign | (kind == 0 ? 0x7f : 0x7c));
  if (mag == 0) return fnuz ? 0 : sign;
  int e = (int)(mag >> 23) - 127;
  uint64_t m = (mag & 0x7fffffu) | 0x800000u;           /* value = m * 2^(e-23) */
  if (mag < 0x00800000u) { e = -126; m = mag; }          /* float32 denormal */
  int emin = 1 - bias;
  int shift = 23 - mbits + (e < emin ? emin - e : 0);
  if (shift > 40) return fnuz ? 0 : sign;
  uint64_t half = 1ull << (shift - 1);
  uint64_t r = m >> shift, rem = m & ((1ull << shift) - 1);
  if (rem > half || (rem == half && (r & 1u))) r++;
  uint32_t code;
  if (e < emin) code = (uint32_t)r;                      /* denormal (may round up to the first normal) */
  else code = ((uint32_t)(e - emin + 1) << mbits) + (uint32_t)(r - (1u << mbits));
  if (fnuz) {
    if (code > 0x7f) return 0x80;                        /* beyond the largest value: NaN (no saturation) */
    return code == 0 ? 0 : (uint8_t)(sign | code);       /* no negative zero */
  }
  if (kind == 0) { if (code > 0x7e) code = 0x7f; }       /* beyond 448: NaN (no saturation) */
  else { if (code > 0x7c) code = 0x7c; }                 /* beyond 57344: inf */
  return (uint8_t)(sign | code);
}

/* ---- int8 weight-only ---------------------------------------------------- */

/* dtype: 0 float32, 1 float16, 2 bfloat16 (A, scales and C share it). */
static inline float ld_t(const void* p, int64_t i, int dtype) {
  if (dtype == 0) return ((const float*)p)[i];
  if (dtype == 1) return oracle_f16_to_f32(((const uint16_t*)p)[i]);
  return oracle_bf16_to_f32(((const uint16_t*)p)[i]);
}
static inline void st_t(void* p, int64_t i, int dtype, float v) {
  if (dtype == 0) ((float*)p)[i] = v;
  else if (dtype == 1) ((uint16_t*)p)[i] = oracle_f32_to_f16(v);
  else ((uint16_t*)p)[i] = oracle_f32_to_bf16(v);
}

/* qmm8.slang:78-111: each weight dequantised as float(b) * scale, products
 * accumulated in float32 (k ascending here; the shader's lanes stride k and
 * add 32 partial sums, another order of the same float32 sum), rounded once. */
void oracle_qmm8(const void* a, int64_t a_sm, const int8_t* b, const void* scales, void* c,
                 int64_t m, int64_t n, int64_t k, int dtype) {
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      float scale = ld_t(scales, j, dtype);
      float acc = 0.0f;
      for (int64_t kk = 0; kk < k; kk++) {
        float w = (float)(int)b[j * k + kk] * scale;
        acc += ld_t(a, i * a_sm + kk, dtype) * w;
      }
      st_t(c, i * n + j, dtype, acc);
    }
}

/* The same sum in float64, unrounded, plus the magnitude sum |a| . |b s| that
 * the reference's test bounds the error with (tests/python/test_quant.py:36-40). */
void oracle_qmm8_f64(const void* a, int64_t a_sm, const int8_t* b, const void* scales, double* c, double* mag,
                     int64_t m, int64_t n, int64_t k, int dtype) {
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      double scale = (double)ld_t(scales, j, dtype), acc = 0.0, ma = 0.0;
      for (int64_t kk = 0; kk < k; kk++) {
        double p = (double)ld_t(a, i * a_sm + kk, dtype) * ((double)b[j * k + kk] * scale);
        acc += p;
        ma += fabs(p);
      }
      c[i * n + j] = acc;
      if (mag) mag[i * n + j] = ma;
    }
}

/* ---- dynamic int8 activations x int4 weights ----------------------------- */

/* quant.cpp:139-143: cat(float(weight bytes), float(scales), float(bias)).
 * scales_dtype: 0 float32, 2 bfloat16. bias may be NULL. */
void oracle_qmm4_pack(const uint8_t* w, int64_t nw, const void* scales, int64_t ns, int scales_dtype,
                      const float* bias, int64_t nbias, float* packed) {
  for (int64_t i = 0; i < nw; i++) packed[i] = (float)w[i];
  for (int64_t i = 0; i < ns; i++) packed[nw + i] = ld_t(scales, i, scales_dtype);
  if (bias)
    for (int64_t i = 0; i < nbias; i++) packed[nw + ns + i] = bias[i];
}

/* qmm4.slang:132-181. inp dtype 0 float32 / 2 bfloat16, contiguous [m, k].
 * q int32 [m, k]; recip float [m]; neg_zp int32 [m] (the shader's rows[2m],
 * rows[2m+1]); scale_out float [m] optional. Nothing here may be fused. */
void oracle_qmm4_quantize(const void* inp, int dtype, int64_t m, int64_t k, int groupwise,
                          int32_t* q, float* recip_out, int32_t* neg_zp_out, float* scale_out) {
  const float qmin = -128.0f, qmax = 127.0f;
  for (int64_t r = 0; r < m; r++) {
    float mn = 3.40282347e38f, mx = -3.40282347e38f;
    for (int64_t kk = 0; kk < k; kk++) {
      float v = ld_t(inp, r * k + kk, dtype);
      mn = v < mn ? v : mn;
      mx = v > mx ? v : mx;
    }
    float rmin = mn < 0.0f ? mn : 0.0f, rmax = mx > 0.0f ? mx : 0.0f;
    volatile float range = rmax - rmin;
    float scale = rmin == rmax ? 1.0f : (qmax - qmin) / range;
    float recip = scale != 0.0f ? 1.0f / scale : 0.0f;
    volatile float dmin = rmin * scale, dmax = rmax * scale;
    volatile float e1 = qmin + dmin;
    float err;
    if (groupwise) {
      volatile float e2 = e1 + qmax;
      err = e2 + dmax;
    } else {
      volatile float e2 = qmax + dmax;
      err = e1 + e2;
    }
    float zp = err > 0.0f ? qmin - dmin : qmax - dmax;
    zp = zp < qmin ? qmin : zp;
    zp = zp > qmax ? qmax : zp;
    int izp = (int)rintf(zp); /* ties to even (the default rounding mode) */
    recip_out[r] = recip;
    neg_zp_out[r] = -izp;
    if (scale_out) scale_out[r] = scale;
    for (int64_t kk = 0; kk < k; kk++) {
      volatile float scaled = ld_t(inp, r * k + kk, dtype) * scale;
      int v = (int)roundf(scaled) + izp; /* halfway away from zero */
      q[r * k + kk] = v < -128 ? -128 : (v > 127 ? 127 : v);
    }
  }
}

/* qmm4.slang:183-247. packed: the float32 vector of oracle_qmm4_pack.
 * out dtype 0 float32 / 2 bfloat16 (truncating store). iacc_out (optional):
 * int32 [m, n, nblocks], every block's integer sum. */
void oracle_qmm4_matmul(const int32_t* q, const float* recip, const int32_t* neg_zp, const float* packed,
                        void* out, int dtype, int64_t m, int64_t n, int64_t k, int64_t bs, int has_bias,
                        int32_t* iacc_out) {
  int64_t rstride = (k + 1) / 2, wcount = n * k / 2, nblocks = (k + bs - 1) / bs;
  for (int64_t r = 0; r < m; r++) {
    int off = neg_zp[r];
    for (int64_t j = 0; j < n; j++) {
      float main_acc = 0.0f;
      int first = 1;
      int32_t iacc = 0;
      for (int64_t k0 = 0; k0 < k; k0 += 32) {
        int64_t kend = k - k0 < 32 ? k - k0 : 32;
        for (int64_t kk = 0; kk < kend; kk++) {
          int64_t kg = k0 + kk;
          uint32_t byte = (uint32_t)packed[j * rstride + kg / 2];
          int w = (kg & 1) ? (int)(byte >> 4) - 8 : (int)(byte & 15u) - 8;
          iacc += q[r * k + kg] * w;
          iacc += off * w;
        }
        if ((k0 + 32) % bs == 0 || k0 + 32 >= k) {
          int64_t blk = k0 / bs;
          float s = packed[wcount + j * nblocks + blk];
          if (iacc_out) iacc_out[(r * n + j) * nblocks + blk] = iacc;
          volatile float x = (float)iacc * s;
          if (first) main_acc = x;
          else { volatile float t = main_acc + x; main_acc = t; }
          first = 0;
          iacc = 0;
        }
      }
      { volatile float t = main_acc * recip[r]; main_acc = t; }
      if (has_bias) { volatile float t = main_acc + packed[wcount + n * nblocks + j]; main_acc = t; }
      const float hi = dtype == 2 ? 3.38953139e38f : 3.40282347e38f;
      main_acc = main_acc < -hi ? -hi : main_acc; /* NaN passes */
      main_acc = hi < main_acc ? hi : main_acc;
      if (dtype == 2) ((uint16_t*)out)[r * n + j] = (uint16_t)(f32_bits(main_acc) >> 16);
      else ((float*)out)[r * n + j] = main_acc;
    }
  }
}

/* ---- float8 _scaled_mm ---------------------------------------------------- */

/* quant.cpp:283-299. a: float8 codes [m, k], element (i, kk) at a[i*a_s0 + kk*a_s1];
 * b: float8 codes [k, n], element (kk, j) at b[kk*b_s0 + j*b_s1].
 * scale_a / scale_b: one float (rowwise 0) or m / n floats (rowwise 1).
 * bias: n floats (already widened) or NULL. inv_scale_result: multiplies the
 * sum when the output is float8 (1 / scale_result), else pass 1.
 * out_kind: 0 float32, 1 float16, 2 bfloat16, 3 e4m3fn, 4 e5m2, 5 e4m3fnuz, 6 e5m2fnuz.
 * acc64: 0 accumulates in float32 (k ascending), 1 in float64 and also stores
 * the unrounded sum in ref64 (optional) for the ulp check. */
void oracle_scaled_mm(const uint8_t* a, int a_kind, int64_t a_s0, int64_t a_s1,
                      const uint8_t* b, int b_kind, int64_t b_s0, int64_t b_s1,
                      const float* scale_a, const float* scale_b, int rowwise,
                      const float* bias, float inv_scale_result,
                      void* out, int out_kind, int64_t m, int64_t n, int64_t k, int acc64, double* ref64) {
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      float sa = rowwise ? scale_a[i] : scale_a[0], sb = rowwise ? scale_b[j] : scale_b[0];
      float accf = 0.0f;
      double accd = 0.0;
      for (int64_t kk = 0; kk < k; kk++) {
        float av = oracle_f8_to_f32(a[i * a_s0 + kk * a_s1], a_kind) * sa;
        float bv = oracle_f8_to_f32(b[kk * b_s0 + j * b_s1], b_kind) * sb;
        if (acc64) accd += (double)av * (double)bv;
        else accf += av * bv;
      }
      float r;
      if (acc64) {
        if (bias) accd += (double)bias[j];
        if (out_kind >= 3) accd *= (double)inv_scale_result;
        if (ref64) ref64[i * n + j] = accd;
        r = (float)accd;
      } else {
        r = accf;
        if (bias) r += bias[j];
        if (out_kind >= 3) r *= inv_scale_result;
      }
      int64_t o = i * n + j;
      switch (out_kind) {
        case 0: ((float*)out)[o] = r; break;
        case 1: ((uint16_t*)out)[o] = oracle_f32_to_f16(r); break;
        case 2: ((uint16_t*)out)[o] = oracle_f32_to_bf16(r); break;
        case 3: ((uint8_t*)out)[o] = oracle_f32_to_f8(r, 0); break;
        case 4: ((uint8_t*)out)[o] = oracle_f32_to_f8(r, 1); break;
        case 5: ((uint8_t*)out)[o] = oracle_f32_to_f8(r, 2); break;
        default: ((uint8_t*)out)[o] = oracle_f32_to_f8(r, 3); break;
      }
    }
}

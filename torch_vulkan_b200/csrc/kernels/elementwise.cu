// Data movement for tensors on the device: strided copies with dtype conversion
// and fills. These are the slice of the reference's cast / move / fill kernels
// (crates/vkcore/shaders/cast.slang, move.slang, and the float8 tables of
// crates/pyvk/csrc/backend.cpp:538-586) that the quantised products, their
// argument preparation (scales.to(A.dtype), .contiguous()) and their tests need.
// Conversions follow c10's static_casts: 16- and 8-bit floats are rounded from
// float32 (nearest even), integers truncate toward zero and wrap.
#include "../core/common.h"
#include "numerics.cuh"

namespace tvb {
namespace {

constexpr int kMaxDims = 8;

struct CopyParams {
  int64_t sizes[kMaxDims];
  int64_t dst_strides[kMaxDims];
  int64_t src_strides[kMaxDims];
  int64_t numel;
  int ndim;
  int dst_dtype, src_dtype;
};

struct Value {
  double d;
  int64_t i;
  bool is_int;
};

__device__ __forceinline__ Value load_value(const void* p, int64_t idx, int dtype) {
  Value v{0.0, 0, false};
  switch (dtype) {
    case TVB_F32: v.d = static_cast<const float*>(p)[idx]; break;
    case TVB_F64: v.d = static_cast<const double*>(p)[idx]; break;
    case TVB_F16: case TVB_BF16: case TVB_E4M3: case TVB_E5M2: case TVB_E4M3FNUZ: case TVB_E5M2FNUZ:
      v.d = load_float_rt(p, idx, dtype);
      break;
    case TVB_I8: v.i = static_cast<const int8_t*>(p)[idx]; v.is_int = true; break;
    case TVB_U8: v.i = static_cast<const uint8_t*>(p)[idx]; v.is_int = true; break;
    case TVB_BOOL: v.i = static_cast<const uint8_t*>(p)[idx] != 0; v.is_int = true; break;
    case TVB_I16: v.i = static_cast<const int16_t*>(p)[idx]; v.is_int = true; break;
    case TVB_I32: v.i = static_cast<const int32_t*>(p)[idx]; v.is_int = true; break;
    case TVB_I64: v.i = static_cast<const int64_t*>(p)[idx]; v.is_int = true; break;
    default: break;
  }
  return v;
}

__device__ __forceinline__ void store_value(void* p, int64_t idx, int dtype, const Value& v) {
  switch (dtype) {
    case TVB_F64: static_cast<double*>(p)[idx] = v.is_int ? static_cast<double>(v.i) : v.d; break;
    case TVB_F32: case TVB_F16: case TVB_BF16: case TVB_E4M3: case TVB_E5M2: case TVB_E4M3FNUZ: case TVB_E5M2FNUZ: {
      float f = v.is_int ? static_cast<float>(v.i) : static_cast<float>(v.d);
      store_float_rt(p, idx, dtype, f);
      break;
    }
    case TVB_BOOL: static_cast<uint8_t*>(p)[idx] = v.is_int ? (v.i != 0) : (v.d != 0.0); break;
    default: {
      int64_t i = v.is_int ? v.i : static_cast<int64_t>(v.d);
      if (dtype == TVB_I8) static_cast<int8_t*>(p)[idx] = static_cast<int8_t>(i);
      else if (dtype == TVB_U8) static_cast<uint8_t*>(p)[idx] = static_cast<uint8_t>(i);
      else if (dtype == TVB_I16) static_cast<int16_t*>(p)[idx] = static_cast<int16_t>(i);
      else if (dtype == TVB_I32) static_cast<int32_t*>(p)[idx] = static_cast<int32_t>(i);
      else if (dtype == TVB_I64) static_cast<int64_t*>(p)[idx] = i;
      break;
    }
  }
}

__global__ void copy_strided_kernel(void* dst, const void* src, CopyParams p) {
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < p.numel; e += stride) {
    int64_t rem = e, so = 0, d_o = 0;
    for (int d = p.ndim - 1; d >= 0; d--) {
      int64_t c = rem % p.sizes[d];
      rem /= p.sizes[d];
      so += c * p.src_strides[d];
      d_o += c * p.dst_strides[d];
    }
    store_value(dst, d_o, p.dst_dtype, load_value(src, so, p.src_dtype));
  }
}

// Same dtype, both contiguous: moves 16 bytes per thread where alignment allows.
__global__ void copy_bytes_kernel(uint8_t* dst, const uint8_t* src, int64_t nbytes) {
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  int64_t vec = aligned ? nbytes / 16 : 0;
  for (int64_t i = tid; i < vec; i += stride) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  for (int64_t i = vec * 16 + tid; i < nbytes; i += stride) dst[i] = src[i];
}

struct FillParams {
  int64_t sizes[kMaxDims];
  int64_t strides[kMaxDims];
  int64_t numel;
  int ndim;
  int itemsize;
  uint64_t bits;
};

__global__ void fill_strided_kernel(void* dst, FillParams p) {
  int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < p.numel; e += stride) {
    int64_t rem = e, o = 0;
    for (int d = p.ndim - 1; d >= 0; d--) {
      o += (rem % p.sizes[d]) * p.strides[d];
      rem /= p.sizes[d];
    }
    switch (p.itemsize) {
      case 1: static_cast<uint8_t*>(dst)[o] = static_cast<uint8_t>(p.bits); break;
      case 2: static_cast<uint16_t*>(dst)[o] = static_cast<uint16_t>(p.bits); break;
      case 4: static_cast<uint32_t*>(dst)[o] = static_cast<uint32_t>(p.bits); break;
      default: static_cast<uint64_t*>(dst)[o] = p.bits; break;
    }
  }
}

// c[i, j] = float32(c[i, j]) + float32(v[j]), rounded once to c's dtype: a Linear's bias (or any row vector) added in place.
__global__ void add_rowvec_kernel(void* c, int c_dtype, int64_t c_sm, const void* v, int v_dtype, int64_t m, int64_t n) {
  const int64_t total = m * n;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t i = e / n, j = e - i * n;
    const int64_t o = i * c_sm + j;
    store_float_rt(c, o, c_dtype, load_float_rt(c, o, c_dtype) + load_float_rt(v, j, v_dtype));
  }
}

int grid_for(int device, int64_t numel, int block) {
  int64_t want = ceil_div(numel, block);
  int64_t cap = static_cast<int64_t>(sm_count(device)) * 16;
  return static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
}

bool contiguous(const int64_t* sizes, const int64_t* strides, int ndim) {
  int64_t expect = 1;
  for (int d = ndim - 1; d >= 0; d--) {
    if (sizes[d] == 1) continue;
    if (strides[d] != expect) return false;
    expect *= sizes[d];
  }
  return true;
}

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" int tvb_copy_strided(int device, void* dst, int dst_dtype, const int64_t* dst_strides, const void* src,
                                int src_dtype, const int64_t* src_strides, const int64_t* sizes, int ndim) {
  TVB_REQUIRE(ndim >= 0 && ndim <= kMaxDims, "tvb_copy_strided: at most 8 dimensions");
  TVB_REQUIRE(dtype_size(dst_dtype) != 0 && dtype_size(src_dtype) != 0, "tvb_copy_strided: unknown dtype");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  CopyParams p{};
  p.ndim = ndim;
  p.numel = 1;
  for (int d = 0; d < ndim; d++) {
    p.sizes[d] = sizes[d];
    p.dst_strides[d] = dst_strides[d];
    p.src_strides[d] = src_strides[d];
    p.numel *= sizes[d];
  }
  p.dst_dtype = dst_dtype;
  p.src_dtype = src_dtype;
  if (p.numel == 0) return 0;
  TVB_REQUIRE(dst != nullptr && src != nullptr, "tvb_copy_strided: NULL pointer");
  if (dst_dtype == src_dtype && contiguous(sizes, dst_strides, ndim) && contiguous(sizes, src_strides, ndim)) {
    int64_t nbytes = p.numel * dtype_size(dst_dtype);
    int grid = grid_for(device, ceil_div(nbytes, 16), 256);
    copy_bytes_kernel<<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), nbytes);
    return launched("copy_bytes", dim3(grid), dim3(256), 0, stream);
  }
  int grid = grid_for(device, p.numel, 256);
  copy_strided_kernel<<<grid, 256, 0, stream>>>(dst, src, p);
  return launched("copy_strided", dim3(grid), dim3(256), 0, stream);
}

extern "C" int tvb_fill_strided(int device, void* dst, int itemsize, uint64_t bits, const int64_t* strides,
                                const int64_t* sizes, int ndim) {
  TVB_REQUIRE(ndim >= 0 && ndim <= kMaxDims, "tvb_fill_strided: at most 8 dimensions");
  TVB_REQUIRE(itemsize == 1 || itemsize == 2 || itemsize == 4 || itemsize == 8, "tvb_fill_strided: itemsize must be 1, 2, 4 or 8");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  FillParams p{};
  p.ndim = ndim;
  p.numel = 1;
  for (int d = 0; d < ndim; d++) {
    p.sizes[d] = sizes[d];
    p.strides[d] = strides[d];
    p.numel *= sizes[d];
  }
  p.itemsize = itemsize;
  p.bits = bits;
  if (p.numel == 0) return 0;
  TVB_REQUIRE(dst != nullptr, "tvb_fill_strided: NULL pointer");
  int grid = grid_for(device, p.numel, 256);
  fill_strided_kernel<<<grid, 256, 0, stream>>>(dst, p);
  return launched("fill_strided", dim3(grid), dim3(256), 0, stream);
}

extern "C" int tvb_add_rowvec(int device, void* c, int c_dtype, int64_t c_sm, const void* v, int v_dtype, int64_t m, int64_t n) {
  auto is_float = [](int dt) { return dt == TVB_F32 || dt == TVB_F16 || dt == TVB_BF16; };
  TVB_REQUIRE(is_float(c_dtype) && is_float(v_dtype), "tvb_add_rowvec: float32, float16 or bfloat16 only");
  TVB_REQUIRE(m >= 0 && n >= 0 && c_sm >= n, "tvb_add_rowvec: bad shape");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(c != nullptr && v != nullptr, "tvb_add_rowvec: NULL pointer");
  int grid = grid_for(device, m * n, 256);
  add_rowvec_kernel<<<grid, 256, 0, stream>>>(c, c_dtype, c_sm, v, v_dtype, m, n);
  return launched("add_rowvec", dim3(grid), dim3(256), 0, stream);
}

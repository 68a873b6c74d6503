// Internal helpers shared by the runtime and the kernel launchers of libtvb200.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <algorithm>
#include <string>

#include "tvb200.h"

namespace tvb {

// Records `message` as the calling thread's last error and returns -1
// (the reference's fail(), crates/pyvk/src/ffi.rs:17-21).
int fail(const std::string& message);
int fail_cuda(const char* what, cudaError_t err);

// Makes `device` current and returns its stream through `stream`; -1 with a
// message if the device does not exist or is not an sm_100 part.
int enter(int device, cudaStream_t* stream);

// Counts one kernel launch (tvb_dispatch_count) and, with TVB200_TRACE=1,
// prints it and waits for it (as TORCH_VK_TRACE, ffi.rs:135-148).
int launched(const char* name, dim3 grid, dim3 block, size_t smem, cudaStream_t stream);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int dtype_size(int dtype) {
  switch (dtype) {
    case TVB_F64: case TVB_I64: return 8;
    case TVB_F32: case TVB_I32: return 4;
    case TVB_F16: case TVB_BF16: case TVB_I16: return 2;
    case TVB_E4M3: case TVB_E5M2: case TVB_E4M3FNUZ: case TVB_E5M2FNUZ: case TVB_I8: case TVB_U8: case TVB_BOOL: return 1;
    default: return 0;
  }
}

// Number of SMs of `device` (cached).
int sm_count(int device);

// Device scratch owned by the runtime, one buffer per `slot` (0..3), grown on
// demand and zero-filled whenever it is (re)allocated. Kernels that use it are
// queued on the device's stream, so uses are ordered; kernels must leave any
// counters in it at zero when they finish.
int workspace(int device, int slot, uint64_t bytes, void** out);

// The device's kernel status word (device pointer, zero while all is well).
// Kernels whose bounded waits run out store a nonzero code here;
// tvb_synchronize reports and clears it.
int status_word(int device, int** out);

}  // namespace tvb

#define TVB_CUDA(expr)                                             \
  do {                                                             \
    cudaError_t err__ = (expr);                                    \
    if (err__ != cudaSuccess) return ::tvb::fail_cuda(#expr, err__); \
  } while (0)

#define TVB_REQUIRE(cond, msg)                   \
  do {                                           \
    if (!(cond)) return ::tvb::fail(msg);        \
  } while (0)

// Shared declarations of the ATen layer: the PrivateUse1 backend (named "vk" by the
// Python package, as the reference names its device) on top of libtvb200's C ABI.
// It plays the part of the reference's crates/pyvk/csrc/vk.h: check(), dtype labels,
// device addresses of tensors, and the strict no-fallback policy.
#pragma once

#include <ATen/ATen.h>

#include <cstdint>
#include <string>

#include "tvb200.h"

namespace vkb {

constexpr c10::DeviceType kDevice = c10::DeviceType::PrivateUse1;

// Raises RuntimeError with the runtime's message when a C-ABI call failed (vk.h:75-77).
inline void check(int rc) { TORCH_CHECK(rc == 0, "torch_vulkan_b200: ", tvb_last_error()); }

inline bool is_vk(const at::Tensor& t) { return t.defined() && t.device().type() == kDevice; }

// TvbDtype of a scalar type, or -1 where the kernels cannot hold it.
int dtype_code(at::ScalarType t);

// Device pointer of the tensor's first element (the data pointer is the device address).
inline const void* gpu_address(const at::Tensor& t) { return t.numel() == 0 ? nullptr : t.const_data_ptr(); }
inline void* gpu_address_out(const at::Tensor& t) { return t.numel() == 0 ? nullptr : t.mutable_data_ptr(); }

c10::Allocator* allocator();

// The device index operations on `t` run on; makes it current.
int enter_device(const at::Tensor& t);

// Strict semantics (the reference's TORCH_VK_STRICT, crates/pyvk/csrc/backend.cpp:1749-1788,
// is the only mode here): an operand on another device, or a case a kernel does not take,
// raises instead of running on the CPU.
[[noreturn]] void no_fallback(const char* op, const std::string& why);

// Drops the forms of weights that the ops derive and keep per weight tensor (ops_quant.cpp): prepared int4 weights, widened
// int8 weights.
void clear_weight_caches();

// aten::_weight_int8pack_mm followed by the two adds of a Linear (bias [n], residual [m, n]; either may be undefined), in one
// launch where the decode kernel runs (ops_quant.cpp).
at::Tensor int8_linear(const at::Tensor& A, const at::Tensor& B, const at::Tensor& scales, const at::Tensor& bias,
                       const at::Tensor& residual);

void register_backend();
void shutdown_backend();

}  // namespace vkb

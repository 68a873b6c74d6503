// The Python extension module torch_vulkan_b200._native: registers the backend at
// import and exposes the runtime's housekeeping, mirroring the functions of the
// reference's crates/pyvk/src/lib.rs:180-202 that apply to this backend
// (synchronize, device_name, dispatch_count, capabilities, memory_stats,
// empty_cache, fallback_counts, shutdown), plus zero-copy views between "vk" and
// torch.cuda tensors so that torch.distributed (NCCL) can move "vk" memory.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/csrc/utils/pybind.h>

#include <string>
#include <tuple>
#include <vector>

#include "backend.h"

namespace py = pybind11;

namespace {

std::string device_name(int device) {
  char buf[256] = {0};
  vkb::check(tvb_device_name(device, buf, sizeof(buf)));
  return std::string(buf);
}

int device_count() {
  int n = tvb_device_count();
  return n < 0 ? 0 : n;
}

std::tuple<uint64_t, uint64_t, uint64_t> memory_stats(int device) {
  uint64_t a = 0, r = 0, b = 0;
  tvb_memory_stats(device, &a, &r, &b);
  return {a, r, b};
}

// A tensor on `to` aliasing the memory of `t` (which must be on `from`); `t` stays alive while the alias does.
at::Tensor alias_on(const at::Tensor& t, c10::DeviceType from, c10::DeviceType to) {
  TORCH_CHECK(t.defined() && t.device().type() == from, "expected a tensor on ", c10::DeviceTypeName(from, true), ", got ",
              t.device());
  at::Tensor keep = t;
  void* data = t.numel() == 0 ? nullptr : t.mutable_data_ptr();
  return at::from_blob(
      data, t.sizes(), t.strides(), [keep](void*) mutable { keep.reset(); },
      t.options().device(c10::Device(to, t.device().index())), c10::Device(to, t.device().index()));
}

}  // namespace

PYBIND11_MODULE(_native, m) {
  vkb::register_backend();
  m.def("device_count", &device_count);
  m.def("device_name", &device_name, py::arg("device") = 0);
  m.def("capabilities", [](int device) { return tvb_capabilities(device); }, py::arg("device") = 0);
  m.def("synchronize", [](int device) { vkb::check(tvb_synchronize(device)); }, py::arg("device") = 0);
  m.def("dispatch_count", [] { return tvb_dispatch_count(); });
  m.def("memory_stats", &memory_stats, py::arg("device") = 0);
  m.def(
      "empty_cache",
      [](int device) {
        vkb::clear_weight_caches();  // (the derived forms of weights kept by the ops: they are rebuilt on demand)
        vkb::check(tvb_empty_cache(device));
      },
      py::arg("device") = 0);
  m.def("stream", [](int device) { return reinterpret_cast<uintptr_t>(tvb_stream(device)); }, py::arg("device") = 0);
  m.def("set_stream", [](int device, uintptr_t s) { vkb::check(tvb_set_stream(device, reinterpret_cast<void*>(s))); });
  m.def("set_device", [](int device) { vkb::check(tvb_set_device(device)); });
  // Always empty: no op of this backend can run on the CPU (kept so that the reference's on_gpu() test helper ports).
  m.def("fallback_counts", [] { return std::vector<std::pair<std::string, uint64_t>>(); });
  m.def("as_cuda", [](const at::Tensor& t) { return alias_on(t, vkb::kDevice, c10::DeviceType::CUDA); });
  m.def("from_cuda", [](const at::Tensor& t) { return alias_on(t, c10::DeviceType::CUDA, vkb::kDevice); });
  m.def(
      "int8_linear",
      [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& scales, const std::optional<at::Tensor>& bias,
         const std::optional<at::Tensor>& residual) {
        return vkb::int8_linear(a, b, scales, bias.value_or(at::Tensor()), residual.value_or(at::Tensor()));
      },
      py::arg("a"), py::arg("b"), py::arg("scales"), py::arg("bias") = py::none(), py::arg("residual") = py::none());
  m.def("shutdown", &vkb::shutdown_backend);
}

// The PrivateUse1 backend: allocator, device guard, hooks, tensor factories, views,
// copies and fills for tensors that live in B200 memory, on top of libtvb200's C ABI.
//
// It is the minimal slice of the reference's crates/pyvk/csrc/backend.cpp that the
// quantised matrix products and their tests stand on: the allocator (backend.cpp:118-160),
// the device guard (:286-308), the hooks (:351-369), empty / empty_strided (:391-409),
// views, _copy_from with dtype conversion (:634-790), _local_scalar_dense, fill_, and the
// boxed fallback (:1938-1940) reduced to its strict end state: an op without a kernel
// here raises NotImplementedError; nothing ever runs on the CPU on the backend's behalf.
#include "backend.h"

#include <ATen/EmptyTensor.h>
#include <ATen/InferSize.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <ATen/native/Resize.h>
#include <ATen/ops/as_strided_cpu_dispatch.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/core/impl/alloc_cpu.h>
#include <torch/library.h>

#include <cstring>
#include <vector>

namespace vkb {

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return TVB_F32;
    case at::kHalf: return TVB_F16;
    case at::kBFloat16: return TVB_BF16;
    case at::kFloat8_e4m3fn: return TVB_E4M3;
    case at::kFloat8_e5m2: return TVB_E5M2;
    case at::kFloat8_e4m3fnuz: return TVB_E4M3FNUZ;
    case at::kFloat8_e5m2fnuz: return TVB_E5M2FNUZ;
    case at::kChar: return TVB_I8;
    case at::kByte: return TVB_U8;
    case at::kInt: return TVB_I32;
    case at::kLong: return TVB_I64;
    case at::kDouble: return TVB_F64;
    case at::kBool: return TVB_BOOL;
    case at::kShort: return TVB_I16;
    default: return -1;
  }
}

[[noreturn]] void no_fallback(const char* op, const std::string& why) {
  TORCH_CHECK_NOT_IMPLEMENTED(false, op, ": ", why, " (device \"vk\" never falls back to the CPU)");
}

namespace {

thread_local c10::DeviceIndex g_current = 0;

int device_count() {
  static int n = [] {
    int c = tvb_device_count();
    return c < 0 ? 0 : c;
  }();
  return n;
}

void set_current(c10::DeviceIndex d) {
  if (d < 0) return;
  check(tvb_set_device(d));
  g_current = d;
}

// ---------------------------------------------------------------- allocator

void delete_block(void* handle) { tvb_free(handle); }

struct VkAllocator final : c10::Allocator {
  c10::DataPtr allocate(size_t nbytes) override {
    c10::Device dev(kDevice, g_current);
    if (nbytes == 0) return {nullptr, nullptr, &delete_block, dev};
    TvbAlloc a{};
    check(tvb_alloc(g_current, nbytes, &a));
    return {a.ptr, a.handle, &delete_block, dev};
  }
  c10::DeleterFnPtr raw_deleter() const override { return nullptr; }
  void copy_data(void* dest, const void* src, std::size_t count) const override {
    check(tvb_memcpy_d2d(g_current, dest, src, count));
  }
};

VkAllocator g_allocator;

// Page-locked host memory for tensor.pin_memory() (the reference's pinned allocator, backend.cpp:313-340).
void delete_pinned(void* ptr) { tvb_host_free(ptr); }

struct PinnedAllocator final : c10::Allocator {
  c10::DataPtr allocate(size_t nbytes) override {
    void* ptr = nullptr;
    if (nbytes != 0) check(tvb_host_alloc(nbytes, &ptr));
    return {ptr, ptr, &delete_pinned, c10::Device(c10::DeviceType::CPU)};
  }
  c10::DeleterFnPtr raw_deleter() const override { return &delete_pinned; }
  void copy_data(void* dest, const void* src, std::size_t count) const override { std::memcpy(dest, src, count); }
};

PinnedAllocator g_pinned;

// ---------------------------------------------------------------- device guard

struct VkGuardImpl final : c10::impl::DeviceGuardImplInterface {
  c10::DeviceType type() const override { return kDevice; }
  c10::Device exchangeDevice(c10::Device d) const override {
    c10::Device old(kDevice, g_current);
    set_current(d.index());
    return old;
  }
  c10::Device getDevice() const override { return c10::Device(kDevice, g_current); }
  void setDevice(c10::Device d) const override { set_current(d.index()); }
  void uncheckedSetDevice(c10::Device d) const noexcept override {
    if (d.index() >= 0 && tvb_set_device(d.index()) == 0) g_current = d.index();
  }
  c10::Stream getStream(c10::Device d) const override { return c10::Stream(c10::Stream::DEFAULT, d); }
  c10::Stream getDefaultStream(c10::Device d) const override { return c10::Stream(c10::Stream::DEFAULT, d); }
  c10::Stream exchangeStream(c10::Stream s) const override { return c10::Stream(c10::Stream::DEFAULT, s.device()); }
  c10::DeviceIndex deviceCount() const noexcept override { return static_cast<c10::DeviceIndex>(device_count()); }
  bool queryStream(const c10::Stream&) const override { return true; }
  void synchronizeStream(const c10::Stream& s) const override { check(tvb_synchronize(s.device_index())); }
  void synchronizeDevice(const c10::DeviceIndex d) const override { check(tvb_synchronize(d)); }
  void record(void**, const c10::Stream&, const c10::DeviceIndex, const c10::EventFlag) const override {
    TORCH_CHECK_NOT_IMPLEMENTED(false, "events are not implemented for device \"vk\"");
  }
  void block(void*, const c10::Stream&) const override {}
  bool queryEvent(void*) const override { return true; }
  void destroyEvent(void*, const c10::DeviceIndex) const noexcept override {}
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, VkGuardImpl);

// ---------------------------------------------------------------- hooks

struct VkHooks final : at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return device_count() > 0; }
  bool hasPrimaryContext(c10::DeviceIndex) const override { return true; }
  at::Device getDeviceFromPtr(void*) const override { return at::Device(kDevice, g_current); }
  bool isPinnedPtr(const void* data) const override { return tvb_host_is_pinned(data) != 0; }
  c10::Allocator* getPinnedMemoryAllocator() const override { return &g_pinned; }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const override {
    c10::StorageImpl* impl = storage.unsafeGetStorageImpl();
    TORCH_CHECK(impl->resizable(), "Trying to resize storage that is not resizable");
    size_t old = impl->nbytes();
    if (newsize == old) return;
    c10::DeviceIndex dev = storage.device().index();
    c10::DeviceIndex saved = g_current;
    set_current(dev);
    c10::DataPtr fresh = g_allocator.allocate(newsize);
    size_t keep = std::min(old, newsize);
    if (keep > 0 && impl->data() != nullptr) check(tvb_memcpy_d2d(dev, fresh.get(), impl->data(), keep));
    impl->set_data_ptr_noswap(std::move(fresh));
    impl->set_nbytes(newsize);
    set_current(saved);
  }
};

// ---------------------------------------------------------------- factories and views

at::Tensor empty_memory_format(at::IntArrayRef size, std::optional<at::ScalarType> dtype, std::optional<at::Layout> layout,
                               std::optional<at::Device> device, std::optional<bool> pin_memory,
                               std::optional<at::MemoryFormat> memory_format) {
  TORCH_CHECK(!layout || *layout == at::kStrided, "device \"vk\" holds strided tensors only");
  at::Device dev = device.value_or(at::Device(kDevice, g_current));
  c10::DeviceIndex idx = dev.has_index() ? dev.index() : g_current;
  TORCH_CHECK(idx >= 0 && idx < device_count(), "invalid device vk:", static_cast<int>(idx), " (", device_count(), " device(s))");
  c10::DeviceIndex saved = g_current;
  set_current(idx);
  const c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  at::Tensor t = at::detail::empty_generic(size, &g_allocator, ks, c10::dtype_or_default(dtype), memory_format);
  set_current(saved);
  return t;
}

at::Tensor empty_strided(at::IntArrayRef size, at::IntArrayRef stride, std::optional<at::ScalarType> dtype,
                         std::optional<at::Layout> layout, std::optional<at::Device> device, std::optional<bool> pin_memory) {
  TORCH_CHECK(!layout || *layout == at::kStrided, "device \"vk\" holds strided tensors only");
  at::Device dev = device.value_or(at::Device(kDevice, g_current));
  c10::DeviceIndex idx = dev.has_index() ? dev.index() : g_current;
  TORCH_CHECK(idx >= 0 && idx < device_count(), "invalid device vk:", static_cast<int>(idx), " (", device_count(), " device(s))");
  c10::DeviceIndex saved = g_current;
  set_current(idx);
  const c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  at::Tensor t = at::detail::empty_strided_generic(size, stride, &g_allocator, ks, c10::dtype_or_default(dtype));
  set_current(saved);
  return t;
}

at::Tensor as_strided(const at::Tensor& self, at::IntArrayRef size, at::IntArrayRef stride, std::optional<int64_t> offset) {
  return at::cpu::as_strided(self, size, stride, offset);  // (metadata only: shares the storage)
}

at::Tensor view(const at::Tensor& self, at::IntArrayRef size) {
  at::DimVector shape = at::infer_size_dv(size, self.numel());
  auto stride = at::detail::computeStride(self.sizes(), self.strides(), shape);
  TORCH_CHECK(stride.has_value(),
              "view size is not compatible with input tensor's size and stride (at least one dimension spans across two "
              "contiguous subspaces). Use .reshape(...) instead.");
  return at::cpu::as_strided(self, shape, *stride, self.storage_offset());
}

at::Tensor reshape_alias(const at::Tensor& self, at::IntArrayRef size, at::IntArrayRef stride) {
  return at::cpu::as_strided(self, size, stride, self.storage_offset());
}

const at::Tensor& resize_(const at::Tensor& self, at::IntArrayRef size, std::optional<at::MemoryFormat> memory_format) {
  TORCH_CHECK(!memory_format || *memory_format == at::MemoryFormat::Contiguous,
              "device \"vk\": resize_ supports the contiguous memory format only");
  c10::TensorImpl* impl = self.unsafeGetTensorImpl();
  int64_t numel = 1;
  for (int64_t s : size) numel *= s;
  size_t need = static_cast<size_t>(impl->storage_offset() + numel) * self.element_size();
  if (numel > 0 && need > self.storage().nbytes()) at::native::resize_bytes_nocuda(self.storage(), need);
  impl->set_sizes_contiguous(size);
  return self;
}

at::Tensor& set_storage(at::Tensor& self, at::Storage source, int64_t offset, at::IntArrayRef size, at::IntArrayRef stride) {
  c10::TensorImpl* impl = self.unsafeGetTensorImpl();
  impl->set_storage_keep_dtype(std::move(source));
  impl->set_storage_offset(offset);
  if (stride.data() == nullptr) impl->set_sizes_contiguous(size);
  else impl->set_sizes_and_strides(size, stride);
  return self;
}

// ---------------------------------------------------------------- copies

std::vector<int64_t> vec(at::IntArrayRef a) { return std::vector<int64_t>(a.begin(), a.end()); }

void device_copy(const at::Tensor& dst, const at::Tensor& src) {
  // both on "vk" (same device): one strided conversion kernel, src broadcast to dst's shape
  int sd = dtype_code(src.scalar_type()), dd = dtype_code(dst.scalar_type());
  if (sd < 0 || dd < 0) no_fallback("aten::copy_", "no kernel converts " + std::string(c10::toString(src.scalar_type())) + " to " +
                                                       c10::toString(dst.scalar_type()));
  at::Tensor s = src.sizes() == dst.sizes() ? src : src.expand(dst.sizes());
  TORCH_CHECK(dst.dim() <= 8, "device \"vk\": copies of more than 8 dimensions are not supported");
  auto sizes = vec(dst.sizes()), dstr = vec(dst.strides()), sstr = vec(s.strides());
  int dev = dst.device().index();
  check(tvb_copy_strided(dev, gpu_address_out(dst), dd, dstr.data(), gpu_address(s), sd, sstr.data(), sizes.data(),
                         static_cast<int>(dst.dim())));
}

at::Tensor copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  // dst.copy_(self)
  TORCH_CHECK(self.defined() && dst.defined(), "copy of an undefined tensor");
  if (dst.numel() == 0) return dst;
  const bool src_vk = is_vk(self), dst_vk = is_vk(dst);
  if (src_vk && dst_vk) {
    if (self.device() == dst.device()) {
      device_copy(dst, self);
    } else {
      // another GPU: through a contiguous staging copy on the source device, then a peer copy
      at::Tensor s = self.to(dst.scalar_type()).expand(dst.sizes()).contiguous();
      at::Tensor d = dst.is_contiguous() ? dst : at::empty_like(dst, at::MemoryFormat::Contiguous);
      check(tvb_synchronize(self.device().index()));
      check(tvb_memcpy_d2d(dst.device().index(), gpu_address_out(d), gpu_address(s), d.nbytes()));
      check(tvb_synchronize(dst.device().index()));
      if (!d.is_same(dst)) device_copy(dst, d);
    }
    return dst;
  }
  if (dst_vk) {
    TORCH_CHECK(self.device().is_cpu(), "device \"vk\": copies come from the CPU or from \"vk\", not from ", self.device());
    // host -> device: the bytes go up as they are; any conversion or striding happens on the device
    at::Tensor host = self.sizes() == dst.sizes() && self.is_contiguous() ? self : self.expand(dst.sizes()).contiguous();
    int dev = dst.device().index();
    if (host.scalar_type() == dst.scalar_type() && dst.is_contiguous()) {
      check(tvb_memcpy_h2d(dev, gpu_address_out(dst), host.const_data_ptr(), host.nbytes()));
    } else {
      at::Tensor staged = at::empty(host.sizes(), dst.options().dtype(host.scalar_type()));
      check(tvb_memcpy_h2d(dev, gpu_address_out(staged), host.const_data_ptr(), host.nbytes()));
      device_copy(dst, staged);
    }
    // the host buffer may be pinned (the copy is then asynchronous) and must outlive it
    // (a temporary made above is released on return: wait for the copy then too)
    if (!non_blocking || !host.is_same(self)) check(tvb_synchronize(dev));
    return dst;
  }
  TORCH_CHECK(src_vk && dst.device().is_cpu(), "device \"vk\": copies go to the CPU or to \"vk\", not to ", dst.device());
  // device -> host: convert / gather on the device, bring the bytes down (this waits)
  int dev = self.device().index();
  at::Tensor s = self.sizes() == dst.sizes() ? self : self.expand(dst.sizes());
  at::Tensor staged = s;
  if (s.scalar_type() != dst.scalar_type() || !s.is_contiguous()) {
    staged = at::empty(dst.sizes(), self.options().dtype(dst.scalar_type()));
    device_copy(staged, s);
  }
  if (dst.is_contiguous() && non_blocking && staged.is_same(s) && tvb_host_is_pinned(dst.const_data_ptr()) != 0) {
    // into page-locked memory, caller synchronises (the source is the caller's tensor, alive until then)
    check(tvb_memcpy_d2h_async(dev, dst.mutable_data_ptr(), gpu_address(staged), staged.nbytes()));
  } else if (dst.is_contiguous()) {
    check(tvb_memcpy_d2h(dev, dst.mutable_data_ptr(), gpu_address(staged), staged.nbytes()));
  } else {
    at::Tensor host = at::empty(dst.sizes(), dst.options().memory_format(at::MemoryFormat::Contiguous));
    check(tvb_memcpy_d2h(dev, host.mutable_data_ptr(), gpu_address(staged), staged.nbytes()));
    dst.copy_(host);
  }
  return dst;
}

at::Tensor copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  if (dst.numel() == 0 && is_vk(dst)) resize_(dst, self.sizes(), std::nullopt);
  TORCH_CHECK(self.sizes() == dst.sizes(), "_copy_from_and_resize: shapes differ");
  return copy_from(self, dst, false);
}

at::Scalar local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  at::Tensor host = at::empty({}, self.options().device(at::kCPU));
  copy_from(self.reshape({}), host, false);
  return host.item();
}

// ---------------------------------------------------------------- fill

at::Tensor& fill_scalar(at::Tensor& self, const at::Scalar& value) {
  if (self.numel() == 0) return self;
  TORCH_CHECK(dtype_code(self.scalar_type()) >= 0, "device \"vk\": fill_ of ", self.scalar_type(), " is not supported");
  // the value's bytes in the tensor's dtype, as the CPU converts it
  at::Tensor one = at::empty({1}, self.options().device(at::kCPU));
  one.fill_(value);
  uint64_t bits = 0;
  std::memcpy(&bits, one.const_data_ptr(), self.element_size());
  auto sizes = vec(self.sizes()), strides = vec(self.strides());
  TORCH_CHECK(self.dim() <= 8, "device \"vk\": fills of more than 8 dimensions are not supported");
  check(tvb_fill_strided(self.device().index(), gpu_address_out(self), static_cast<int>(self.element_size()), bits,
                         strides.data(), sizes.data(), static_cast<int>(self.dim())));
  return self;
}

at::Tensor& fill_tensor(at::Tensor& self, const at::Tensor& value) {
  TORCH_CHECK(value.dim() == 0, "fill_ only supports 0-dimension value tensor but got tensor with ", value.dim(), " dimensions.");
  return fill_scalar(self, value.item());
}

at::Tensor& zero_(at::Tensor& self) { return fill_scalar(self, 0); }

// ---------------------------------------------------------------- bias

// self += other for the two shapes a quantised Linear needs: `other` a vector over self's last dimension (its bias), or
// a contiguous tensor of self's own shape (the residual stream its output joins); alpha 1, floating dtypes. Anything else
// is not implemented on this device (and is never run on the CPU instead).
at::Tensor& add_rowvec_(at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha) {
  TORCH_CHECK_NOT_IMPLEMENTED(is_vk(self) && is_vk(other) && self.device() == other.device(),
                              "add_ on device \"vk\": both tensors must be on the same \"vk\" device");
  TORCH_CHECK_NOT_IMPLEMENTED(alpha.to<double>() == 1.0, "add_ on device \"vk\": only alpha = 1 is implemented");
  const bool same_shape = self.dim() >= 2 && other.sizes() == self.sizes() && self.is_contiguous() && other.is_contiguous();
  TORCH_CHECK_NOT_IMPLEMENTED(same_shape || (self.dim() >= 1 && other.dim() == 1 && other.size(0) == self.size(-1) && other.is_contiguous()),
                              "add_ on device \"vk\": only a contiguous vector over the last dimension (a bias) or a contiguous "
                              "tensor of the same shape can be added, got ", self.sizes(), " += ", other.sizes());
  const int cd = dtype_code(self.scalar_type()), vd = dtype_code(other.scalar_type());
  TORCH_CHECK_NOT_IMPLEMENTED(at::isFloatingType(self.scalar_type()) && at::isFloatingType(other.scalar_type()) && cd >= 0 && vd >= 0,
                              "add_ on device \"vk\": floating dtypes only");
  if (self.numel() == 0) return self;
  if (same_shape) {  // one row of numel values
    check(tvb_add_rowvec(self.device().index(), gpu_address_out(self), cd, self.numel(), gpu_address(other), vd, 1, self.numel()));
    return self;
  }
  const int64_t n = self.size(-1);
  TORCH_CHECK_NOT_IMPLEMENTED(self.stride(-1) == 1, "add_ on device \"vk\": the last dimension must be dense");
  if (self.dim() <= 2) {
    const int64_t m = self.dim() == 2 ? self.size(0) : 1;
    const int64_t sm = self.dim() == 2 && m > 1 ? self.stride(0) : n;
    check(tvb_add_rowvec(self.device().index(), gpu_address_out(self), cd, sm, gpu_address(other), vd, m, n));
  } else {
    TORCH_CHECK_NOT_IMPLEMENTED(self.is_contiguous(), "add_ on device \"vk\": more than two dimensions need a contiguous tensor");
    check(tvb_add_rowvec(self.device().index(), gpu_address_out(self), cd, n, gpu_address(other), vd, self.numel() / n, n));
  }
  return self;
}

at::Tensor add_rowvec(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha) {
  // (the result of two dtypes would take the promoted one; only the in-place form, which keeps self's, mixes them)
  TORCH_CHECK_NOT_IMPLEMENTED(self.scalar_type() == other.scalar_type(), "add on device \"vk\": both tensors must have one dtype, got ",
                              self.scalar_type(), " and ", other.scalar_type());
  at::Tensor out = at::empty_like(self, at::MemoryFormat::Contiguous);
  out.copy_(self);
  return add_rowvec_(out, other, alpha);
}

// ---------------------------------------------------------------- everything else

void strict_fallback(const c10::OperatorHandle& op, torch::jit::Stack*) {
  TORCH_CHECK_NOT_IMPLEMENTED(false, op.schema().operator_name(),
                              " has no B200 kernel on device \"vk\" (this backend implements the quantised matrix products "
                              "and never runs an op on the CPU instead)");
}

}  // namespace

c10::Allocator* allocator() { return &g_allocator; }

int enter_device(const at::Tensor& t) {
  int dev = t.device().index();
  check(tvb_set_device(dev));
  return dev;
}

void register_backend() {
  static bool done = false;
  if (done) return;
  done = true;
  c10::SetAllocator(kDevice, &g_allocator);
  at::RegisterPrivateUse1HooksInterface(new VkHooks());
}

void shutdown_backend() {
  clear_weight_caches();  // (their tensors go back to the pool before the pool goes)
  tvb_shutdown();
}

}  // namespace vkb

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  using namespace vkb;
  m.impl("empty.memory_format", &empty_memory_format);
  m.impl("empty_strided", &empty_strided);
  m.impl("as_strided", &as_strided);
  m.impl("view", &view);
  m.impl("_unsafe_view", &view);
  m.impl("_reshape_alias", &reshape_alias);
  m.impl("resize_", &resize_);
  m.impl("set_.source_Storage_storage_offset", &set_storage);
  m.impl("_copy_from", &copy_from);
  m.impl("_copy_from_and_resize", &copy_from_and_resize);
  m.impl("_local_scalar_dense", &local_scalar_dense);
  m.impl("fill_.Scalar", &fill_scalar);
  m.impl("fill_.Tensor", &fill_tensor);
  m.impl("zero_", &zero_);
  m.impl("add_.Tensor", &add_rowvec_);
  m.impl("add.Tensor", &add_rowvec);
}

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) {
  m.fallback(torch::CppFunction::makeFromBoxedFunction<&vkb::strict_fallback>());
}

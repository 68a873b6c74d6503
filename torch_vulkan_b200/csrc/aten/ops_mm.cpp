// aten::mm / aten::addmm on device "vk" for float32, float16 and bfloat16: the unquantised matrix products either side
// of the quantised ones in a model (a Linear that was left in 16 bits, the LM head, an attention projection). The
// reference serves them with its gemm shaders (crates/pyvk/csrc/linalg.cpp:227-321); here 16-bit operands go to the
// tcgen05 main loop the float8 product uses (tvb_mm), everything else to the plain kernel. nn.Linear and F.linear reach
// these through aten::linear's decomposition (addmm for 2-D inputs, a view + mm otherwise).
#include <ATen/native/Resize.h>
#include <torch/library.h>

#include "backend.h"

namespace vkb {
namespace {

void check_operands(const char* op, const at::Tensor& a, const at::Tensor& b) {
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, op, ": both arguments must be matrices, got ", a.dim(), "-D and ", b.dim(), "-D");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "expected m1 and m2 to have the same dtype, but got: ", a.scalar_type(),
              " != ", b.scalar_type());
  TORCH_CHECK(a.size(1) == b.size(0), "mat1 and mat2 shapes cannot be multiplied (", a.size(0), "x", a.size(1), " and ",
              b.size(0), "x", b.size(1), ")");
  for (const at::Tensor* t : {&a, &b})
    if (!is_vk(*t)) no_fallback(op, "an operand is not on \"vk\"");
  const int d = dtype_code(a.scalar_type());
  if (d != TVB_F32 && d != TVB_F16 && d != TVB_BF16)
    no_fallback(op, std::string("no kernel multiplies ") + c10::toString(a.scalar_type()) + " matrices");
}

// out = a @ b (+ bias) (+ residual): `bias` is undefined or a vector of n values, `residual` undefined or an [m, n] matrix
// (which may be `out` itself: every element is read by the thread that then writes it).
void product(const at::Tensor& a_in, const at::Tensor& b_in, const at::Tensor& bias, const at::Tensor& residual_in,
             at::Tensor& out) {
  const int64_t M = a_in.size(0), K = a_in.size(1), N = b_in.size(1);
  at::native::resize_output(out, {M, N});
  if (out.numel() == 0) return;
  const int d = dtype_code(a_in.scalar_type());
  at::Tensor a = a_in, b = b_in;
  // The tensor-core kernel wants both operands K-major: A row-major, B column-major (a transposed weight matrix, the way
  // a Linear passes it). A large row-major B is transposed once on the device rather than left to the plain kernel.
  const bool sixteen = d != TVB_F32;
  const bool large = M * N >= int64_t(128) * 256 * 8 && K >= 64;
  if (sixteen && large) {
    if (a.stride(1) != 1 || a.stride(0) % 8 != 0 || a.stride(0) < K) a = a.contiguous();
    if (b.stride(0) != 1 || b.stride(1) % 8 != 0 || b.stride(1) < K) b = b.t().contiguous().t();
  }
  at::Tensor residual = residual_in;
  if (residual.defined() && M > 1 && (residual.stride(1) != 1 || residual.stride(0) < N)) residual = residual.contiguous();
  at::Tensor dst = out.is_contiguous() ? out : at::empty({M, N}, out.options());
  at::Tensor bv;
  int bias_dtype = TVB_F32;
  if (bias.defined()) {
    bv = bias.contiguous();
    bias_dtype = dtype_code(bv.scalar_type());
  }
  const int dev = enter_device(a);
  check(tvb_addmm(dev, gpu_address(a), d, a.stride(0), a.stride(1), gpu_address(b), b.stride(0), b.stride(1),
                  bias.defined() ? gpu_address(bv) : nullptr, bias_dtype, residual.defined() ? gpu_address(residual) : nullptr,
                  residual.defined() ? dtype_code(residual.scalar_type()) : TVB_F32,
                  residual.defined() ? (M > 1 ? residual.stride(0) : N) : 0, gpu_address_out(dst), dtype_code(out.scalar_type()), M,
                  N, K, 0));
  if (!dst.is_same(out)) out.copy_(dst);
}

at::Tensor& mm_out(const at::Tensor& self, const at::Tensor& mat2, at::Tensor& out) {
  check_operands("aten::mm", self, mat2);
  TORCH_CHECK(out.scalar_type() == self.scalar_type(), "Expected out tensor to have dtype ", self.scalar_type(), ", but got ",
              out.scalar_type(), " instead");
  if (!is_vk(out)) no_fallback("aten::mm", "out is not on \"vk\"");
  product(self, mat2, at::Tensor(), at::Tensor(), out);
  return out;
}

at::Tensor mm(const at::Tensor& self, const at::Tensor& mat2) {
  at::Tensor out = at::empty({0}, self.options());
  return mm_out(self, mat2, out);
}

at::Tensor& addmm_out(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                      const at::Scalar& alpha, at::Tensor& out) {
  check_operands("aten::addmm", mat1, mat2);
  TORCH_CHECK(self.scalar_type() == mat1.scalar_type(), "self and mat2 must have the same dtype, but got ", self.scalar_type(),
              " and ", mat1.scalar_type());
  if (!is_vk(self) || !is_vk(out)) no_fallback("aten::addmm", "an operand is not on \"vk\"");
  const int64_t N = mat2.size(1);
  const int64_t M = mat1.size(0);
  // what a Linear passes: its bias, one value per output column; or a full matrix (the residual stream a block adds its
  // projection to); beta = alpha = 1 either way
  const bool row_bias = (self.dim() == 1 && self.size(0) == N) || (self.dim() == 2 && self.size(0) == 1 && self.size(1) == N);
  const bool matrix = self.dim() == 2 && self.size(0) == M && self.size(1) == N;
  TORCH_CHECK_NOT_IMPLEMENTED((row_bias || matrix) && beta.to<double>() == 1.0 && alpha.to<double>() == 1.0,
                              "aten::addmm on device \"vk\": only a bias vector of ", N, " values or a matrix of ", M, " x ", N,
                              " with beta = alpha = 1 is implemented (got self of shape ", self.sizes(), ")");
  TORCH_CHECK(out.scalar_type() == mat1.scalar_type(), "Expected out tensor to have dtype ", mat1.scalar_type());
  if (row_bias) product(mat1, mat2, self.reshape({N}), at::Tensor(), out);
  else product(mat1, mat2, at::Tensor(), self, out);
  return out;
}

at::Tensor addmm(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                 const at::Scalar& alpha) {
  at::Tensor out = at::empty({0}, mat1.options());
  return addmm_out(self, mat1, mat2, beta, alpha, out);
}

}  // namespace
}  // namespace vkb

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  using namespace vkb;
  m.impl("mm", &mm);
  m.impl("mm.out", &mm_out);
  m.impl("addmm", &addmm);
  m.impl("addmm.out", &addmm_out);
}

// The four quantised matrix products as aten kernels of device "vk":
//
//   _weight_int8pack_mm                    -> tvb_qmm8
//   _dyn_quant_pack_4bit_weight            -> tvb_qmm4_pack
//   _dyn_quant_matmul_4bit                 -> tvb_qmm4 (quantise + multiply)
//   _scaled_mm, _scaled_mm.out             -> tvb_scaled_mm
//
// Same schemas, argument checks and error messages as the reference's entry points
// (crates/pyvk/csrc/quant.cpp:59-119, :127-144, :146-204, :234-310), which are in turn
// the CPU kernels' (ATen/native/LinearAlgebra.cpp, ScaledBlas.cpp); registered the same
// way (quant.cpp:315-322). Where the reference would hand an unsupported case to the CPU
// (operands elsewhere, sizes past 2^31: quant.cpp:75-78, :134-138, :159-164, :238-241)
// this layer raises: strict semantics are the only mode.
#include <ATen/native/Resize.h>
#include <torch/library.h>

#include <algorithm>
#include <cstdlib>
#include <list>
#include <mutex>
#include <sstream>

#include "backend.h"

namespace vkb {
namespace {

void require_vk(const char* op, std::initializer_list<const at::Tensor*> tensors) {
  for (const at::Tensor* t : tensors) {
    if (t != nullptr && t->defined() && !is_vk(*t)) {
      std::ostringstream why;
      why << "an operand is on " << t->device() << ", not on \"vk\"";
      no_fallback(op, why.str());
    }
  }
}

// ------------------------------------------------------------------ int8 weight-only

uint32_t tensor_version(const at::Tensor& t) { return t.is_inference() ? 0u : t._version(); }

// With many rows of A (prefill) the product is a 16-bit GEMM over the weights widened to A's dtype, and the widening pass
// (3 bytes of traffic per weight) is worth keeping when the same weights come back call after call: widened copies are kept
// per (weight tensor, scales tensor, dtype) within TORCH_VK_QMM8_CACHE_MB megabytes (default 16384: a 7-billion-parameter
// model's worth of bfloat16 copies on a 180 GB part; 0 turns the cache off). An entry is dropped when either tensor's storage
// dies or its version counter moves.
struct WidenedWeights {
  c10::weak_intrusive_ptr<c10::StorageImpl> b_storage, s_storage;
  const void *b_data, *s_data;
  int64_t n, k;
  uint32_t b_version, s_version;
  int dtype;
  at::Tensor widened;
};

std::mutex g_widened_mutex;
std::list<WidenedWeights> g_widened;  // most recently used first
uint64_t g_widened_bytes = 0;

uint64_t widened_budget() {
  static const uint64_t budget = [] {
    const char* v = std::getenv("TORCH_VK_QMM8_CACHE_MB");
    return static_cast<uint64_t>(v != nullptr ? std::max<long long>(0, std::atoll(v)) : 16384) << 20;
  }();
  return budget;
}

// The widened copy of (B, scales) in `dtype`, from the cache or made now; an undefined tensor when it does not fit the budget.
at::Tensor widened_weights(const at::Tensor& B, const at::Tensor& s, int dev, int dtype, int64_t n, int64_t k) {
  const uint64_t bytes = tvb_qmm8_widened_bytes(n, k);
  std::lock_guard<std::mutex> lock(g_widened_mutex);
  c10::StorageImpl* bi = B.storage().unsafeGetStorageImpl();
  c10::StorageImpl* si = s.storage().unsafeGetStorageImpl();
  for (auto it = g_widened.begin(); it != g_widened.end();) {
    if (it->b_storage.expired() || it->s_storage.expired()) {
      g_widened_bytes -= it->widened.numel();
      it = g_widened.erase(it);
      continue;
    }
    if (it->b_storage._unsafe_get_target() == bi && it->s_storage._unsafe_get_target() == si && it->b_data == B.const_data_ptr() &&
        it->s_data == s.const_data_ptr() && it->n == n && it->k == k && it->dtype == dtype && it->b_version == tensor_version(B) &&
        it->s_version == tensor_version(s)) {
      g_widened.splice(g_widened.begin(), g_widened, it);
      return g_widened.front().widened;
    }
    if (it->b_storage._unsafe_get_target() == bi && it->b_data == B.const_data_ptr() && it->dtype == dtype) {
      // the same weights under an older version (or other scales): that copy is of no use any more
      g_widened_bytes -= it->widened.numel();
      it = g_widened.erase(it);
      continue;
    }
    ++it;
  }
  // No eviction: when the budget is used up, further weights take the kernels that need no copy (a model larger than the
  // budget would otherwise widen every layer on every call). Entries leave with their tensors or through empty_cache().
  if (g_widened_bytes + bytes > widened_budget()) return at::Tensor();
  at::Tensor widened = at::empty({static_cast<int64_t>(bytes)}, B.options().dtype(at::kByte));
  check(tvb_qmm8_widen(dev, static_cast<const int8_t*>(gpu_address(B)), gpu_address(s), dtype, n, k, gpu_address_out(widened), bytes));
  g_widened.push_front(WidenedWeights{c10::weak_intrusive_ptr<c10::StorageImpl>(B.storage().getWeakStorageImpl()),
                                      c10::weak_intrusive_ptr<c10::StorageImpl>(s.storage().getWeakStorageImpl()), B.const_data_ptr(),
                                      s.const_data_ptr(), n, k, tensor_version(B), tensor_version(s), dtype, widened});
  g_widened_bytes += bytes;
  return widened;
}

at::Tensor weight_int8pack_mm(const at::Tensor& A, const at::Tensor& B, const at::Tensor& scales) {
  constexpr const char* fn = "_weight_int8pack_mm_cpu";  // (the messages name the CPU kernel, as the reference's do)
  const int64_t M = A.size(0), N = B.size(0), K = A.size(1);
  TORCH_CHECK(A.dtype() == at::kBFloat16 || A.dtype() == at::kHalf || A.dtype() == at::kFloat, fn,
              " : expect A to be either 32-bit or 16-bit float tensor.");
  TORCH_CHECK(A.dim() == 2, fn, " : expect A to be 2D tensor.");
  TORCH_CHECK(A.stride(1) == 1, fn, " : A must be contiguous on the last dimension.");
  TORCH_CHECK(B.dtype() == at::kChar, fn, " : expect B to be int8 tensor.");
  TORCH_CHECK(B.is_contiguous(), fn, " : expect B to be contiguous.");
  TORCH_CHECK(B.size(1) == K, fn, " : expect B.size(1) == ", K);
  TORCH_CHECK(scales.dim() == 1 && scales.size(0) == N, fn, " : expect scales to be 1d tensor with size ", N);
  require_vk("aten::_weight_int8pack_mm", {&A, &B, &scales});

  at::Tensor C = at::empty({M, N}, A.options());
  if (C.numel() == 0) return C;
  at::Tensor s = scales.to(A.scalar_type()).contiguous();  // (the CPU reads the scales in A's dtype)
  const int dev = enter_device(A);
  const int dt = dtype_code(A.scalar_type());
  // More rows than one pass of the decode kernel takes (64, when k is a multiple of 128; else 32), 16-bit A, aligned rows: the
  // GEMM over cached widened weights (keyed on the caller's own scales tensor, so only when no converted copy of it was
  // needed). It is faster than widening in the main loop at every such m (62 against 95 us at m = 512 on a 14336 x 4096
  // layer).
  if (M > (K % 128 == 0 ? 64 : 32) && (dt == TVB_BF16 || dt == TVB_F16) && K % 16 == 0 && A.stride(0) % 8 == 0 && A.stride(0) >= K &&
      (reinterpret_cast<uintptr_t>(gpu_address(A)) & 15u) == 0 && (reinterpret_cast<uintptr_t>(gpu_address(B)) & 15u) == 0 &&
      s.is_same(scales)) {
    at::Tensor widened = widened_weights(B, s, dev, dt, N, K);
    if (widened.defined()) {
      check(tvb_qmm8_widened(dev, gpu_address(A), dt, A.stride(0), gpu_address(widened), gpu_address_out(C), M, N, K));
      return C;
    }
  }
  check(tvb_qmm8(dev, gpu_address(A), dtype_code(A.scalar_type()), A.stride(0), static_cast<const int8_t*>(gpu_address(B)),
                 gpu_address(s), gpu_address_out(C), M, N, K, 0));
  return C;
}

}  // namespace

// The int8 weight-only Linear in one call: the product, + bias, + residual (each defined or not), rounded step by step as
// the three ops would. At most 32 rows of 16-bit A: one launch of the decode kernel does all three (tvb_qmm8_linear).
// More rows: the op above (with its cached widened weights), then the adds.
at::Tensor int8_linear(const at::Tensor& A, const at::Tensor& B, const at::Tensor& scales, const at::Tensor& bias,
                       const at::Tensor& residual) {
  if (!bias.defined() && !residual.defined()) return weight_int8pack_mm(A, B, scales);
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.size(1) == B.size(1), "int8_linear: A [m, k] and B [n, k] expected");
  const int64_t M = A.size(0), N = B.size(0), K = A.size(1);
  require_vk("int8_linear", {&A, &B, &scales, &bias, &residual});
  TORCH_CHECK(!bias.defined() || (bias.dim() == 1 && bias.size(0) == N && bias.scalar_type() == A.scalar_type()),
              "int8_linear: the bias must hold ", N, " values of A's dtype");
  TORCH_CHECK(!residual.defined() || (residual.dim() == 2 && residual.size(0) == M && residual.size(1) == N &&
                                      residual.scalar_type() == A.scalar_type()),
              "int8_linear: the residual must be [", M, ", ", N, "] of A's dtype");
  const int dt = dtype_code(A.scalar_type());
  const bool decode = M >= 1 && M <= 32 && (dt == TVB_BF16 || dt == TVB_F16) && A.stride(1) == 1 && B.is_contiguous() &&
                      B.scalar_type() == at::kChar && scales.dim() == 1 && scales.size(0) == N &&
                      scales.scalar_type() == A.scalar_type() && scales.is_contiguous();
  if (!decode) {
    at::Tensor C = weight_int8pack_mm(A, B, scales);
    if (bias.defined()) C.add_(bias.contiguous());
    if (residual.defined()) C.add_(residual.contiguous());
    return C;
  }
  at::Tensor C = at::empty({M, N}, A.options());
  at::Tensor bv = bias.defined() ? bias.contiguous() : at::Tensor();
  at::Tensor rv = residual.defined() ? residual.contiguous() : at::Tensor();
  const int dev = enter_device(A);
  check(tvb_qmm8_linear(dev, gpu_address(A), dt, A.stride(0), static_cast<const int8_t*>(gpu_address(B)), gpu_address(scales),
                        bv.defined() ? gpu_address(bv) : nullptr, rv.defined() ? gpu_address(rv) : nullptr, gpu_address_out(C), M,
                        N, K));
  return C;
}

namespace {

// ------------------------------------------------------------------ dynamic int8 x int4

void check_group_size(const char* fn, int64_t block_size, int64_t in_features) {
  TORCH_CHECK(block_size == in_features || (!(block_size % 32) && !(in_features % block_size)), fn,
              ": Group size should be multiple of 32, in_features [", in_features, "]. Provided ", block_size);
}

at::Tensor dyn_quant_pack_4bit_weight(const at::Tensor& weights, const at::Tensor& scales_zeros,
                                      const std::optional<at::Tensor>& bias, int64_t block_size, int64_t in_features,
                                      int64_t out_features) {
  TORCH_CHECK(weights.dtype() == at::kByte, "_dyn_quant_pack_4bit_weight_cpu", " : expect weight to be kByte.");
  check_group_size("_dyn_quant_pack_4bit_weight_cpu", block_size, in_features);
  const at::Tensor* b = bias.has_value() && bias->defined() ? &*bias : nullptr;
  require_vk("aten::_dyn_quant_pack_4bit_weight", {&weights, &scales_zeros, b});
  // One float32 vector: the weights' bytes, the scales, the bias (the CPU's layout, so that packing on
  // either device serves either device's product). One kernel writes all three parts.
  at::Tensor w = weights.contiguous(), s = scales_zeros.contiguous();
  at::Tensor bv = b != nullptr ? b->contiguous() : at::Tensor();
  const int sd = dtype_code(s.scalar_type());
  TORCH_CHECK(sd == TVB_F32 || sd == TVB_BF16 || sd == TVB_F16 || sd == TVB_F64,
              "_dyn_quant_pack_4bit_weight: scales must be a floating point tensor, got ", s.scalar_type());
  const int64_t nb = bv.defined() ? bv.numel() : 0;
  at::Tensor packed = at::empty({w.numel() + s.numel() + nb}, weights.options().dtype(at::kFloat));
  if (packed.numel() == 0) return packed;
  const int dev = enter_device(weights);
  check(tvb_qmm4_pack(dev, static_cast<const uint8_t*>(gpu_address(w)), w.numel(), gpu_address(s), sd, s.numel(),
                      nb ? gpu_address(bv) : nullptr, nb ? dtype_code(bv.scalar_type()) : TVB_F32, nb,
                      static_cast<float*>(gpu_address_out(packed))));
  return packed;
}

// The tensor-core kernel reads the weights as int8 [n, k]; unpacking the packed vector's float-encoded bytes costs
// about as much as a small product, so the result is kept per packed tensor: keyed by its storage, offset and size,
// and dropped when the tensor's version counter moves (an in-place write) or its storage dies.
struct PreparedWeights {
  c10::weak_intrusive_ptr<c10::StorageImpl> storage;
  const void* data;
  int64_t numel, n, k, bs;
  uint32_t version;
  int kind;       // 0: int8 weights for the exact tensor-core kernel; 1: float16 weight * scale for the fast route;
                  // 2: nibbles and scales tiled for the decode kernel; 3: float16 weights for the float16 form of the exact kernel
  int inexact;    // kind 1: some weight * scale product is not exact in float16 (the fast route must not be used)
  at::Tensor prepared;
};

std::mutex g_prepared_mutex;
std::list<PreparedWeights> g_prepared;  // most recently used first
constexpr size_t kMaxPrepared = 16;

uint32_t version_of(const at::Tensor& t) { return t.is_inference() ? 0u : t._version(); }

at::Tensor prepared_weights(const at::Tensor& packed, int dev, int64_t n, int64_t k, int64_t bs, int kind, int* inexact) {
  std::lock_guard<std::mutex> lock(g_prepared_mutex);
  c10::StorageImpl* impl = packed.storage().unsafeGetStorageImpl();
  for (auto it = g_prepared.begin(); it != g_prepared.end();) {
    if (it->storage.expired()) {
      it = g_prepared.erase(it);
      continue;
    }
    if (it->storage._unsafe_get_target() == impl && it->data == packed.const_data_ptr() && it->numel == packed.numel() &&
        it->n == n && it->k == k && it->bs == bs && it->kind == kind && it->version == version_of(packed)) {
      g_prepared.splice(g_prepared.begin(), g_prepared, it);
      if (inexact != nullptr) *inexact = g_prepared.front().inexact;
      return g_prepared.front().prepared;
    }
    ++it;
  }
  const uint64_t bytes = kind == 0 ? tvb_qmm4_prepared_bytes(n, k)
                                   : (kind == 1 ? tvb_qmm4_fast_prepared_bytes(n, k)
                                                : (kind == 2 ? tvb_qmm4_decode_prepared_bytes(n, k, bs) : tvb_qmm4_prepared16_bytes(n, k)));
  at::Tensor prepared = at::empty({static_cast<int64_t>(bytes)}, packed.options().dtype(at::kByte));
  int flag = 0;
  if (kind == 0)
    check(tvb_qmm4_prepare(dev, static_cast<const float*>(gpu_address(packed)), n, k, bs, gpu_address_out(prepared), bytes));
  else if (kind == 2)
    check(tvb_qmm4_decode_prepare(dev, static_cast<const float*>(gpu_address(packed)), n, k, bs, gpu_address_out(prepared), bytes));
  else if (kind == 3)
    check(tvb_qmm4_prepare16(dev, static_cast<const float*>(gpu_address(packed)), n, k, bs, gpu_address_out(prepared), bytes));
  else
    check(tvb_qmm4_fast_prepare(dev, static_cast<const float*>(gpu_address(packed)), n, k, bs, gpu_address_out(prepared), bytes, &flag));
  if (inexact != nullptr) *inexact = flag;
  g_prepared.push_front(PreparedWeights{c10::weak_intrusive_ptr<c10::StorageImpl>(packed.storage().getWeakStorageImpl()),
                                        packed.const_data_ptr(), packed.numel(), n, k, bs, version_of(packed), kind, flag, prepared});
  while (g_prepared.size() > kMaxPrepared) g_prepared.pop_back();
  return prepared;
}

at::Tensor dyn_quant_matmul_4bit(const at::Tensor& inp, const at::Tensor& packed_weights, int64_t block_size,
                                 int64_t in_features, int64_t out_features) {
  constexpr const char* fn = "_dyn_quant_matmul_4bit_cpu";
  TORCH_CHECK(inp.dtype() == at::kFloat || (inp.dtype() == at::kBFloat16 && block_size == in_features), fn,
              " : expect input to be float32 or bfloat16 tensor.");
  check_group_size(fn, block_size, in_features);
  TORCH_CHECK(inp.dim() == 2 && inp.size(1) == in_features, "_dyn_quant_matmul_4bit: expected input of shape [M, ", in_features,
              "], got ", inp.sizes());
  require_vk("aten::_dyn_quant_matmul_4bit", {&inp, &packed_weights});
  const int64_t M = inp.size(0), N = out_features, K = in_features;
  if (M * std::max(K, N) >= (int64_t(1) << 31) || packed_weights.numel() >= (int64_t(1) << 32))
    no_fallback("aten::_dyn_quant_matmul_4bit", "sizes beyond 32-bit offsets");
  at::Tensor out = at::empty({M, N}, inp.options());
  const int64_t weight_elements = N * K / 2, scale_elements = N * (K / block_size);
  TORCH_CHECK(packed_weights.numel() >= weight_elements + scale_elements, "Invalid packed weight tensor size");
  const int64_t bias_elements = packed_weights.numel() - (weight_elements + scale_elements);
  if (bias_elements != 0) TORCH_CHECK(bias_elements == N, "Expected bias length to match output dimension");
  if (out.numel() == 0) return out;
  at::Tensor x = inp.contiguous();
  at::Tensor packed = packed_weights.to(at::kFloat).contiguous();
  const int dev = enter_device(inp);
  // Both kernels are bit for bit the CPU's arithmetic; the tensor-core one takes every shape it can (k and the
  // block size multiples of 32), the CUDA-core one the rest, and up to 16 rows go to the decode kernel where it takes
  // the shape. TORCH_VK_QMM4=plain forces the CUDA-core kernel, =tc keeps small m on the tensor-core kernel (as the
  // reference's TORCH_VK_GEMM switches kernels for its tests).
  // TORCH_VK_QMM4=fast opts into the float16 GEMM route: not bit for bit (float32 accumulation over the whole of k
  // instead of per block), within rtol 1e-5 of the exact routes. It applies when every weight * scale is exact in
  // float16 (block scales that came from bfloat16) and the packed vector is the caller's own float32 tensor.
  const char* mode_env = std::getenv("TORCH_VK_QMM4");
  const std::string mode = mode_env != nullptr ? mode_env : "";
  const bool force_plain = mode == "plain";
  // (up to 32 rows as two passes of the 16-row decode kernel: still faster than one 128-row tensor-core tile)
  const bool decode = !force_plain && mode != "tc" && M <= 32 && tvb_qmm4_decode_usable(std::min<int64_t>(M, 16), N, K, block_size) != 0 &&
                      packed.is_same(packed_weights);
  if (mode == "fast" && !decode && K % 8 == 0 && packed.is_same(packed_weights)) {
    int inexact = 0;
    at::Tensor prepared = prepared_weights(packed_weights, dev, N, K, block_size, 1, &inexact);
    if (inexact == 0) {
      const uint64_t fbytes = tvb_qmm4_fast_workspace_bytes(M, K);
      at::Tensor fws = at::empty({static_cast<int64_t>(fbytes)}, inp.options().dtype(at::kByte));
      check(tvb_qmm4_fast(dev, gpu_address(x), dtype_code(x.scalar_type()), static_cast<const float*>(gpu_address(packed)),
                          bias_elements != 0 ? 1 : 0, gpu_address(prepared), gpu_address_out(out), M, N, K, block_size,
                          gpu_address_out(fws), fbytes));
      return out;
    }
  }
  if (decode) {
    // decoding (at most 16 rows): the int4 weights, re-tiled once per packed tensor, streamed from HBM once
    at::Tensor prepared = prepared_weights(packed_weights, dev, N, K, block_size, 2, nullptr);
    for (int64_t r0 = 0; r0 < M; r0 += 16) {
      const int64_t rows = std::min<int64_t>(16, M - r0);
      const uint64_t dbytes = tvb_qmm4_decode_workspace_bytes(rows, K);
      at::Tensor dws = at::empty({static_cast<int64_t>(dbytes)}, inp.options().dtype(at::kByte));
      at::Tensor xr = x.narrow(0, r0, rows), outr = out.narrow(0, r0, rows);  // (whole rows of contiguous matrices)
      check(tvb_qmm4_decode(dev, gpu_address(xr), dtype_code(x.scalar_type()), static_cast<const float*>(gpu_address(packed)),
                            bias_elements != 0 ? 1 : 0, gpu_address(prepared), gpu_address_out(outr), rows, N, K, block_size,
                            gpu_address_out(dws), dbytes));
    }
    return out;
  }
  if (!force_plain && mode != "i8" && block_size == 32 && K % 32 == 0 && packed.is_same(packed_weights)) {
    // Blocks of 32 values (the groupwise form the op is usually given, its scales from bfloat16): the float16 form of the
    // exact kernel, whose per-block drain is one fma per output. Same bits as the int8 form (TORCH_VK_QMM4=i8 keeps that).
    at::Tensor prepared = prepared_weights(packed_weights, dev, N, K, block_size, 3, nullptr);
    const uint64_t tc_bytes = tvb_qmm4_tc16_workspace_bytes(M, K);
    at::Tensor tc_ws = at::empty({static_cast<int64_t>(tc_bytes)}, inp.options().dtype(at::kByte));
    check(tvb_qmm4_tc16(dev, gpu_address(x), dtype_code(x.scalar_type()), static_cast<const float*>(gpu_address(packed)),
                        bias_elements != 0 ? 1 : 0, gpu_address(prepared), gpu_address_out(out), M, N, K, block_size,
                        gpu_address_out(tc_ws), tc_bytes));
    return out;
  }
  if (!force_plain && K % 32 == 0 && block_size % 32 == 0) {
    // the cache keys on the caller's tensor when it is already the float32 vector (the usual case)
    const bool own = packed.is_same(packed_weights);
    at::Tensor prepared = own ? prepared_weights(packed_weights, dev, N, K, block_size, 0, nullptr) : at::Tensor();
    if (!own) {
      const uint64_t bytes = tvb_qmm4_prepared_bytes(N, K);
      prepared = at::empty({static_cast<int64_t>(bytes)}, inp.options().dtype(at::kByte));
      check(tvb_qmm4_prepare(dev, static_cast<const float*>(gpu_address(packed)), N, K, block_size, gpu_address_out(prepared), bytes));
    }
    const uint64_t tc_bytes = tvb_qmm4_tc_workspace_bytes(M, K);
    at::Tensor tc_ws = at::empty({static_cast<int64_t>(tc_bytes)}, inp.options().dtype(at::kByte));
    check(tvb_qmm4_tc(dev, gpu_address(x), dtype_code(x.scalar_type()), static_cast<const float*>(gpu_address(packed)),
                      bias_elements != 0 ? 1 : 0, gpu_address(prepared), gpu_address_out(out), M, N, K, block_size,
                      gpu_address_out(tc_ws), tc_bytes));
    return out;
  }
  const uint64_t ws_bytes = tvb_qmm4_workspace_bytes(M, K);
  at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, inp.options().dtype(at::kByte));
  check(tvb_qmm4(dev, gpu_address(x), dtype_code(x.scalar_type()), static_cast<const float*>(gpu_address(packed)),
                 bias_elements != 0 ? 1 : 0, gpu_address_out(out), M, N, K, block_size, gpu_address_out(ws), ws_bytes));
  return out;
}

// ------------------------------------------------------------------ float8

bool tensorwise_scale(const at::Tensor& t, const at::Tensor& scale) {
  return at::isFloat8Type(t.scalar_type()) && scale.scalar_type() == at::kFloat && scale.numel() == 1;
}

bool rowwise_scale(const at::Tensor& t, const at::Tensor& scale) {
  return at::isFloat8Type(t.scalar_type()) && scale.scalar_type() == at::kFloat && scale.dim() == 2 &&
         scale.size(0) == t.size(0) && scale.size(1) == 1 && scale.is_contiguous();
}

// (ScaledBlas.cpp's message for a scale layout that is neither tensor-wise nor row-wise)
[[noreturn]] void bad_scaling(const at::Tensor& a, const at::Tensor& b, const at::Tensor& sa, const at::Tensor& sb) {
  std::ostringstream msg;
  msg << "Invalid scaling configuration.\n"
      << "- For TensorWise scaling, a and b should be float8, scales should be float and singletons.\n"
      << "- For RowWise scaling, a and b should be float8, scales should be float, scale_a should be (" << a.size(0)
      << ", 1) and scale_b should be (1, " << b.size(1) << "), and both should be contiguous.\n"
      << "Got mat_a.dtype()=" << a.scalar_type() << ", scale_a.dtype()=" << sa.scalar_type()
      << ", scale_a.size()=" << sa.sizes() << ", scale_a.stride()=" << sa.strides() << ", mat_b.dtype()=" << b.scalar_type()
      << ", scale_b.dtype()=" << sb.scalar_type() << ", scale_b.size()=" << sb.sizes()
      << " and scale_b.stride()=" << sb.strides();
  TORCH_CHECK_VALUE(false, msg.str());
}

at::Tensor& scaled_mm_out(const at::Tensor& mat1, const at::Tensor& mat2, const at::Tensor& scale_a, const at::Tensor& scale_b,
                          const std::optional<at::Tensor>& bias, const std::optional<at::Tensor>& scale_result,
                          std::optional<c10::ScalarType> out_dtype, bool use_fast_accum, at::Tensor& out) {
  const at::Tensor* bias_t = bias.has_value() && bias->defined() ? &*bias : nullptr;
  const at::Tensor* result_t = scale_result.has_value() && scale_result->defined() ? &*scale_result : nullptr;
  require_vk("aten::_scaled_mm", {&mat1, &mat2, &out});
  TORCH_CHECK_VALUE(!out_dtype || *out_dtype == out.scalar_type(), "out_dtype must match output matrix type");
  bool rowwise = false;
  if (!(tensorwise_scale(mat1, scale_a) && tensorwise_scale(mat2.t(), scale_b.t()))) {
    if (!(rowwise_scale(mat1, scale_a) && rowwise_scale(mat2.t(), scale_b.t()))) bad_scaling(mat1, mat2, scale_a, scale_b);
    rowwise = true;
  }
  TORCH_CHECK(mat1.dim() == 2, "mat1 must be a matrix");
  TORCH_CHECK(mat2.dim() == 2, "mat2 must be a matrix");
  TORCH_CHECK(mat1.sizes()[1] == mat2.sizes()[0], "mat_a and mat_b shapes cannot be multiplied (", mat1.sizes()[0], "x",
              mat1.sizes()[1], " and ", mat2.sizes()[0], "x", mat2.sizes()[1], ")");
  const bool both_f8 = at::isFloat8Type(mat1.scalar_type()) && at::isFloat8Type(mat2.scalar_type());
  if (!rowwise) {
    TORCH_CHECK_VALUE(both_f8, "mat1 and mat2 must be fp8 types, got: ", mat1.scalar_type(), mat2.scalar_type());
    TORCH_CHECK_VALUE(scale_a.numel() == 1 && scale_a.scalar_type() == at::kFloat, "scale_a must have 1 Float element");
    TORCH_CHECK_VALUE(scale_b.numel() == 1 && scale_b.scalar_type() == at::kFloat, "scale_b must have 1 Float element");
  } else {
    TORCH_CHECK_VALUE(both_f8, "mat1 and mat_b must be fp8 types, got: ", mat1.scalar_type(), mat2.scalar_type());
    TORCH_CHECK_VALUE(scale_a.size(0) == mat1.size(0) && scale_a.size(1) == 1, "scale_a must have shape [", mat1.size(0),
                      ", 1], got [", scale_a.sizes(), "]");
    TORCH_CHECK_VALUE(scale_a.numel() == mat1.size(0) && scale_a.scalar_type() == at::kFloat, "scale_a must have ",
                      mat1.size(0), " Float elements, got ", scale_a.numel());
    TORCH_CHECK_VALUE(scale_b.numel() == mat2.size(1) && scale_b.scalar_type() == at::kFloat, "scale_b must have ",
                      mat2.size(1), " Float elements, got ", scale_b.numel());
    TORCH_CHECK_VALUE(scale_a.stride(1) == 1, "expected scale_a.stride(1) to be 1, but got ", scale_a.stride(1));
    TORCH_CHECK_VALUE(scale_b.stride(1) == 1, "expected scale_b.stride(1) to be 1, but got ", scale_b.stride(1));
  }
  TORCH_CHECK(result_t == nullptr || (result_t->numel() == 1 && result_t->scalar_type() == at::kFloat),
              "scale_result must be a float scalar");
  TORCH_CHECK(bias_t == nullptr || bias_t->numel() == mat2.sizes()[1], "Bias must be size ", mat2.sizes()[1], " but got ",
              bias_t == nullptr ? 0 : bias_t->numel());
  TORCH_CHECK(at::isFloat8Type(mat1.scalar_type()), "Expected mat1 to be Float8 matrix got ", mat1.scalar_type());
  TORCH_CHECK(at::isFloat8Type(mat2.scalar_type()), "Expected mat2 to be Float8 matrix got ", mat2.scalar_type());
  require_vk("aten::_scaled_mm", {&scale_a, &scale_b, bias_t, result_t});

  const int64_t M = mat1.size(0), K = mat1.size(1), N = mat2.size(1);
  at::native::resize_output(out, {M, N});
  if (out.numel() == 0) return out;
  const int ad = dtype_code(mat1.scalar_type()), bd = dtype_code(mat2.scalar_type()), od = dtype_code(out.scalar_type());
  auto is_f8 = [](int dt) { return dt == TVB_E4M3 || dt == TVB_E5M2 || dt == TVB_E4M3FNUZ || dt == TVB_E5M2FNUZ; };
  if (!is_f8(ad) || !is_f8(bd)) no_fallback("aten::_scaled_mm", "only the four float8 formats have kernels");
  if (od != TVB_F32 && od != TVB_F16 && od != TVB_BF16 && !is_f8(od))
    no_fallback("aten::_scaled_mm", std::string("no kernel writes ") + c10::toString(out.scalar_type()));
  // The kernels write a contiguous [M, N]; any other `out` receives a copy of one.
  at::Tensor dst = out.is_contiguous() ? out : at::empty({M, N}, out.options());
  at::Tensor sa = scale_a.contiguous(), sb = scale_b.contiguous();
  at::Tensor bv;
  int bias_dtype = TVB_F32;
  if (bias_t != nullptr) {
    bv = bias_t->contiguous();
    bias_dtype = dtype_code(bv.scalar_type());
    if (bias_dtype != TVB_F32 && bias_dtype != TVB_F16 && bias_dtype != TVB_BF16) {
      bv = bv.to(at::kFloat);
      bias_dtype = TVB_F32;
    }
  }
  const int dev = enter_device(mat1);
  check(tvb_scaled_mm(dev, gpu_address(mat1), ad, mat1.stride(0), mat1.stride(1), gpu_address(mat2), bd, mat2.stride(0),
                      mat2.stride(1), static_cast<const float*>(gpu_address(sa)), static_cast<const float*>(gpu_address(sb)),
                      rowwise ? 1 : 0, bias_t != nullptr ? gpu_address(bv) : nullptr, bias_dtype,
                      result_t != nullptr ? static_cast<const float*>(gpu_address(*result_t)) : nullptr, gpu_address_out(dst),
                      od, M, N, K, 0));
  if (!dst.is_same(out)) out.copy_(dst);
  return out;
}

at::Tensor scaled_mm(const at::Tensor& mat_a, const at::Tensor& mat_b, const at::Tensor& scale_a, const at::Tensor& scale_b,
                     const std::optional<at::Tensor>& bias, const std::optional<at::Tensor>& scale_result,
                     std::optional<c10::ScalarType> out_dtype, bool use_fast_accum) {
  at::Tensor out = at::empty({0}, mat_a.options().dtype(out_dtype.value_or(mat_a.scalar_type())));
  return scaled_mm_out(mat_a, mat_b, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out);
}

}  // namespace

void clear_weight_caches() {
  {
    std::lock_guard<std::mutex> lock(g_prepared_mutex);
    g_prepared.clear();
  }
  std::lock_guard<std::mutex> lock(g_widened_mutex);
  g_widened.clear();
  g_widened_bytes = 0;
}

}  // namespace vkb

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  using namespace vkb;
  m.impl("_weight_int8pack_mm", &weight_int8pack_mm);
  m.impl("_dyn_quant_pack_4bit_weight", &dyn_quant_pack_4bit_weight);
  m.impl("_dyn_quant_matmul_4bit", &dyn_quant_matmul_4bit);
  m.impl("_scaled_mm", &scaled_mm);
  m.impl("_scaled_mm.out", &scaled_mm_out);
}

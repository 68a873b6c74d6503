"""ctypes bindings of the C ABI in include/tvb200.h (lib/libtvb200.so).

This is the same boundary the C++ ATen layer binds; tests and the benchmark
call through it directly with device pointers (for example those of
torch.cuda tensors). There is no fallback: if the library was not built, or
no B200 is present, the calls raise.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libtvb200.so")

F32, F16, BF16, E4M3, E5M2, I8, U8, I32, I64, F64, BOOL, I16, E4M3FNUZ, E5M2FNUZ = range(14)

_c = ctypes
_vp, _i, _i64, _u64, _u32 = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_uint64, _c.c_uint32


class TvbAlloc(ctypes.Structure):
    _fields_ = [("handle", _vp), ("ptr", _vp), ("size", _u64), ("device", _c.c_int32), ("pad", _c.c_int32)]


class TvbChainItem(ctypes.Structure):
    _fields_ = [("a", _vp), ("a_sm", _i64), ("b", _vp), ("scales", _vp), ("c_ranks", _c.POINTER(_vp)), ("m", _i64),
                ("n_local", _i64), ("k", _i64), ("independent", _c.c_int32), ("reserved", _c.c_int32)]


class TvbGroupItem(ctypes.Structure):
    _fields_ = [("a", _vp), ("a_sm", _i64), ("b", _vp), ("scales", _vp), ("c_ranks", _c.POINTER(_vp)), ("m", _i64), ("c_host", _vp)]


# name -> (restype, argtypes): every entry point include/tvb200.h declares
SIGNATURES = {
    "tvb_last_error": (_c.c_char_p, []),
    "tvb_device_count": (_i, []),
    "tvb_set_device": (_i, [_i]),
    "tvb_current_device": (_i, []),
    "tvb_device_name": (_i, [_i, _c.c_char_p, _c.c_size_t]),
    "tvb_capabilities": (_u32, [_i]),
    "tvb_alloc": (_i, [_i, _u64, _c.POINTER(TvbAlloc)]),
    "tvb_free": (None, [_vp]),
    "tvb_synchronize": (_i, [_i]),
    "tvb_empty_cache": (_i, [_i]),
    "tvb_memory_stats": (None, [_i, _c.POINTER(_u64), _c.POINTER(_u64), _c.POINTER(_u64)]),
    "tvb_stream": (_vp, [_i]),
    "tvb_set_stream": (_i, [_i, _vp]),
    "tvb_dispatch_count": (_u64, []),
    "tvb_shutdown": (None, []),
    "tvb_host_alloc": (_i, [_u64, _c.POINTER(_vp)]),
    "tvb_host_free": (None, [_vp]),
    "tvb_host_is_pinned": (_i, [_vp]),
    "tvb_host_register": (_i, [_vp, _u64, _c.POINTER(_vp)]),
    "tvb_host_unregister": (_i, [_vp]),
    "tvb_memcpy_h2d": (_i, [_i, _vp, _vp, _u64]),
    "tvb_memcpy_d2h": (_i, [_i, _vp, _vp, _u64]),
    "tvb_memcpy_d2d": (_i, [_i, _vp, _vp, _u64]),
    "tvb_memcpy_d2h_async": (_i, [_i, _vp, _vp, _u64]),
    "tvb_memcpy_d2h_overlapped": (_i, [_i, _vp, _vp, _u64]),
    "tvb_join_copies": (_i, [_i]),
    "tvb_copy_strided": (_i, [_i, _vp, _i, _c.POINTER(_i64), _vp, _i, _c.POINTER(_i64), _c.POINTER(_i64), _i]),
    "tvb_fill_strided": (_i, [_i, _vp, _i, _u64, _c.POINTER(_i64), _c.POINTER(_i64), _i]),
    "tvb_add_rowvec": (_i, [_i, _vp, _i, _i64, _vp, _i, _i64, _i64]),
    "tvb_qmm8_widened_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm8_widen": (_i, [_i, _vp, _vp, _i, _i64, _i64, _vp, _u64]),
    "tvb_qmm8_widened": (_i, [_i, _vp, _i, _i64, _vp, _vp, _i64, _i64, _i64]),
    "tvb_mm": (_i, [_i, _vp, _i, _i64, _i64, _vp, _i64, _i64, _vp, _i, _vp, _i, _i64, _i64, _i64, _i]),
    "tvb_addmm": (_i, [_i, _vp, _i, _i64, _i64, _vp, _i64, _i64, _vp, _i, _vp, _i, _i64, _vp, _i, _i64, _i64, _i64, _i]),
    "tvb_qmm8": (_i, [_i, _vp, _i, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i]),
    "tvb_qmm8_linear": (_i, [_i, _vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64]),
    "tvb_qmm8_gather": (_i, [_i, _vp, _i, _i64, _vp, _vp, _c.POINTER(_vp), _c.POINTER(_vp), _i, _i, _vp, _i, _i64, _i64, _i64]),
    "tvb_wait_flags": (_i, [_i, _vp, _i, _vp]),
    "tvb_set_wait_limit_ms": (_i, [_i]),
    "tvb_qmm8_group": (_i, [_i, _i, _c.POINTER(TvbGroupItem), _i, _i64, _i64]),
    "tvb_qmm8_group_gather": (_i, [_i, _i, _c.POINTER(TvbGroupItem), _i, _c.POINTER(_vp), _i, _i, _vp, _i, _i64, _i64]),
    "tvb_qmm8_chain_create": (_i, [_i, _i, _c.POINTER(TvbChainItem), _i, _c.POINTER(_vp), _i, _i, _vp, _i, _c.POINTER(_vp)]),
    "tvb_qmm8_chain_run": (_i, [_i, _vp]),
    "tvb_qmm8_chain_destroy": (None, [_vp]),
    "tvb_comm_unique_id": (_i, [_c.c_char_p]),
    "tvb_comm_init_rank": (_i, [_i, _c.c_char_p, _i, _i, _i, _c.POINTER(_vp)]),
    "tvb_comm_init_all": (_i, [_c.POINTER(_i), _i, _c.POINTER(_vp)]),
    "tvb_all_gather": (_i, [_vp, _vp, _vp, _u64]),
    "tvb_all_gather_columns": (_i, [_vp, _vp, _vp, _i, _i64, _i64]),
    "tvb_comm_wait": (_i, [_vp, _i]),
    "tvb_comm_abort": (_i, [_vp]),
    "tvb_comm_destroy": (_i, [_vp]),
    "tvb_graph_begin": (_i, [_i]),
    "tvb_graph_end": (_i, [_i, _c.POINTER(_vp)]),
    "tvb_graph_launch": (_i, [_i, _vp]),
    "tvb_graph_destroy": (None, [_vp]),
    "tvb_ipc_export": (_i, [_i, _vp, _c.c_char_p, _c.POINTER(_u64)]),
    "tvb_ipc_import": (_i, [_i, _c.c_char_p, _u64, _c.POINTER(_vp)]),
    "tvb_qmm8_static_scratch": (_i, [_i, _vp, _i, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tvb_qmm8_static_scratch_status": (_i, [_i, _vp, _c.POINTER(_i)]),
    "tvb_qmm4_pack": (_i, [_i, _vp, _i64, _vp, _i, _i64, _vp, _i, _i64, _vp]),
    "tvb_qmm4_quantize": (_i, [_i, _vp, _i, _i64, _i64, _i, _vp, _vp, _vp]),
    "tvb_qmm4_matmul": (_i, [_i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i64, _i64, _i64, _i64, _vp]),
    "tvb_qmm4_workspace_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4": (_i, [_i, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_prepared_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_prepare": (_i, [_i, _vp, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_tc_workspace_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_decode_usable": (_i, [_i64, _i64, _i64, _i64]),
    "tvb_qmm4_decode_prepared_bytes": (_u64, [_i64, _i64, _i64]),
    "tvb_qmm4_decode_prepare": (_i, [_i, _vp, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_decode_workspace_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_decode": (_i, [_i, _vp, _i, _vp, _i, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_tc": (_i, [_i, _vp, _i, _vp, _i, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_prepared16_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_prepare16": (_i, [_i, _vp, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_tc16_workspace_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_tc16": (_i, [_i, _vp, _i, _vp, _i, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _u64]),
    "tvb_qmm4_fast_prepared_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_fast_prepare": (_i, [_i, _vp, _i64, _i64, _i64, _vp, _u64, _c.POINTER(_i)]),
    "tvb_qmm4_fast_workspace_bytes": (_u64, [_i64, _i64]),
    "tvb_qmm4_fast": (_i, [_i, _vp, _i, _vp, _i, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _u64]),
    "tvb_scaled_mm_gather": (_i, [_i, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _vp, _vp, _i, _vp, _i, _vp, _c.POINTER(_vp), _i,
                                  _c.POINTER(_vp), _i, _i, _vp, _i, _i64, _i64, _i64]),
    "tvb_scaled_mm": (_i, [_i, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i64, _i64,
                           _i64, _i]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m torch_vulkan_b200._build` "
                               "(there is no fallback without the CUDA library)")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


class TvbError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise TvbError(lib().tvb_last_error().decode("utf-8", "replace"))


def _dtype_code(dtype):
    import torch

    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2,
            torch.int8: I8, torch.uint8: U8, torch.int32: I32, torch.int64: I64, torch.float64: F64, torch.bool: BOOL,
            torch.int16: I16, torch.float8_e4m3fnuz: E4M3FNUZ, torch.float8_e5m2fnuz: E5M2FNUZ}[dtype]


def _ptr(t):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


def _dev(t):
    return t.device.index if t.device.index is not None else 0


def synchronize(device=0):
    check(lib().tvb_synchronize(device))


# ---- op-level wrappers over device tensors (torch.cuda tensors or any tensor whose data_ptr is a device pointer)

def qmm8(a, b, scales, variant=0):
    """tvb_qmm8 on device tensors: A [m, k] (last dim contiguous), int8 B [n, k], scales [n] in A's dtype."""
    import torch

    m, k = a.shape
    n = b.shape[0]
    assert scales.dtype == a.dtype and b.dtype == torch.int8 and b.is_contiguous()
    c = torch.empty((m, n), dtype=a.dtype, device=a.device)
    check(lib().tvb_qmm8(_dev(a), _ptr(a), _dtype_code(a.dtype), a.stride(0), _ptr(b), _ptr(scales), _ptr(c), m, n, k, variant))
    return c


def qmm8_linear(a, b, scales, bias=None, residual=None, out=None):
    """tvb_qmm8_linear on device tensors: the product of `qmm8`, + bias [n], + residual [m, n] (A's dtype; either may be None).
    `out` may be the residual itself where the decode kernel runs (at most 32 rows)."""
    import torch

    m, k = a.shape
    n = b.shape[0]
    assert scales.dtype == a.dtype and b.dtype == torch.int8 and b.is_contiguous()
    assert bias is None or (bias.dtype == a.dtype and bias.shape == (n,) and bias.is_contiguous())
    assert residual is None or (residual.dtype == a.dtype and residual.shape == (m, n) and residual.is_contiguous())
    c = torch.empty((m, n), dtype=a.dtype, device=a.device) if out is None else out
    check(lib().tvb_qmm8_linear(_dev(a), _ptr(a), _dtype_code(a.dtype), a.stride(0), _ptr(b), _ptr(scales), _ptr(bias),
                                _ptr(residual), _ptr(c), m, n, k))
    return c


def qmm4_pack(weights, scales, bias):
    import torch

    w = weights.contiguous().reshape(-1)
    s = scales.contiguous().reshape(-1)
    nb = 0 if bias is None else bias.numel()
    bvec = None if bias is None else bias.contiguous().reshape(-1)
    packed = torch.empty(w.numel() + s.numel() + nb, dtype=torch.float32, device=w.device)
    check(lib().tvb_qmm4_pack(_dev(w), _ptr(w), w.numel(), _ptr(s), _dtype_code(s.dtype), s.numel(), _ptr(bvec),
                              _dtype_code(bvec.dtype) if bvec is not None else F32, nb, _ptr(packed)))
    return packed


def qmm4_quantize(x, groupwise):
    import torch

    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    recip = torch.empty(m, dtype=torch.float32, device=x.device)
    neg_zp = torch.empty(m, dtype=torch.int32, device=x.device)
    check(lib().tvb_qmm4_quantize(_dev(x), _ptr(x), _dtype_code(x.dtype), m, k, 1 if groupwise else 0, _ptr(q), _ptr(recip),
                                  _ptr(neg_zp)))
    return q, recip, neg_zp


def qmm4_matmul(q, recip, neg_zp, packed, n, k, bs, out_dtype, return_iacc=False):
    import torch

    m = q.shape[0]
    nblocks = (k + bs - 1) // bs
    has_bias = 1 if packed.numel() - (n * k // 2 + n * nblocks) else 0
    out = torch.empty((m, n), dtype=out_dtype, device=q.device)
    iacc = torch.empty((m, n, nblocks), dtype=torch.int32, device=q.device) if return_iacc else None
    check(lib().tvb_qmm4_matmul(_dev(q), _ptr(q), _ptr(recip), _ptr(neg_zp), _ptr(packed), has_bias, _ptr(out),
                                _dtype_code(out_dtype), m, n, k, bs, _ptr(iacc)))
    return (out, iacc) if return_iacc else out


def qmm4(x, packed, bs, k, n):
    import torch

    m = x.shape[0]
    nblocks = (k + bs - 1) // bs
    has_bias = 1 if packed.numel() - (n * k // 2 + n * nblocks) else 0
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    nbytes = lib().tvb_qmm4_workspace_bytes(m, k)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    check(lib().tvb_qmm4(_dev(x), _ptr(x), _dtype_code(x.dtype), _ptr(packed), has_bias, _ptr(out), m, n, k, bs, _ptr(ws),
                         nbytes))
    return out


def qmm4_prepare(packed, n, k, bs):
    import torch

    nbytes = lib().tvb_qmm4_prepared_bytes(n, k)
    prepared = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
    check(lib().tvb_qmm4_prepare(_dev(packed), _ptr(packed), n, k, bs, _ptr(prepared), nbytes))
    return prepared


def qmm4_tc(x, packed, prepared, bs, k, n):
    import torch

    m = x.shape[0]
    nblocks = (k + bs - 1) // bs
    has_bias = 1 if packed.numel() - (n * k // 2 + n * nblocks) else 0
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    nbytes = lib().tvb_qmm4_tc_workspace_bytes(m, k)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    check(lib().tvb_qmm4_tc(_dev(x), _ptr(x), _dtype_code(x.dtype), _ptr(packed), has_bias, _ptr(prepared), _ptr(out), m, n, k,
                            bs, _ptr(ws), nbytes))
    return out


def qmm4_prepare16(packed, n, k, bs):
    import torch

    nbytes = lib().tvb_qmm4_prepared16_bytes(n, k)
    prepared = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
    check(lib().tvb_qmm4_prepare16(_dev(packed), _ptr(packed), n, k, bs, _ptr(prepared), nbytes))
    return prepared


def qmm4_tc16(x, packed, prepared, bs, k, n):
    import torch

    m = x.shape[0]
    nblocks = (k + bs - 1) // bs
    has_bias = 1 if packed.numel() - (n * k // 2 + n * nblocks) else 0
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    nbytes = lib().tvb_qmm4_tc16_workspace_bytes(m, k)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    check(lib().tvb_qmm4_tc16(_dev(x), _ptr(x), _dtype_code(x.dtype), _ptr(packed), has_bias, _ptr(prepared), _ptr(out), m, n, k,
                              bs, _ptr(ws), nbytes))
    return out


def qmm4_decode_prepare(packed, n, k, bs):
    import torch

    nbytes = lib().tvb_qmm4_decode_prepared_bytes(n, k, bs)
    prepared = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
    check(lib().tvb_qmm4_decode_prepare(_dev(packed), _ptr(packed), n, k, bs, _ptr(prepared), nbytes))
    return prepared


def qmm4_decode(x, packed, prepared, bs, k, n):
    import torch

    m = x.shape[0]
    has_bias = 1 if packed.numel() - (n * k // 2 + n * (k // bs)) else 0
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    nbytes = lib().tvb_qmm4_decode_workspace_bytes(m, k)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    check(lib().tvb_qmm4_decode(_dev(x), _ptr(x), _dtype_code(x.dtype), _ptr(packed), has_bias, _ptr(prepared), _ptr(out), m, n,
                                k, bs, _ptr(ws), nbytes))
    return out


def qmm4_fast_prepare(packed, n, k, bs):
    """(prepared float16 weights, inexact flag)"""
    import torch

    nbytes = lib().tvb_qmm4_fast_prepared_bytes(n, k)
    prepared = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
    flag = _i(0)
    check(lib().tvb_qmm4_fast_prepare(_dev(packed), _ptr(packed), n, k, bs, _ptr(prepared), nbytes, _c.byref(flag)))
    return prepared, flag.value


def qmm4_fast(x, packed, prepared, bs, k, n):
    import torch

    m = x.shape[0]
    nblocks = (k + bs - 1) // bs
    has_bias = 1 if packed.numel() - (n * k // 2 + n * nblocks) else 0
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    nbytes = lib().tvb_qmm4_fast_workspace_bytes(m, k)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    check(lib().tvb_qmm4_fast(_dev(x), _ptr(x), _dtype_code(x.dtype), _ptr(packed), has_bias, _ptr(prepared), _ptr(out), m, n, k,
                              bs, _ptr(ws), nbytes))
    return out


def scaled_mm(a, b, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None, variant=0):
    import torch

    m, k = a.shape
    n = b.shape[1]
    out_dtype = out_dtype or a.dtype
    rowwise = 0 if (scale_a.numel() == 1 and scale_b.numel() == 1) else 1
    sa = scale_a.contiguous().reshape(-1)
    sb = scale_b.contiguous().reshape(-1)
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    check(lib().tvb_scaled_mm(_dev(a), _ptr(a), _dtype_code(a.dtype), a.stride(0), a.stride(1), _ptr(b), _dtype_code(b.dtype),
                              b.stride(0), b.stride(1), _ptr(sa), _ptr(sb), rowwise, _ptr(bias),
                              _dtype_code(bias.dtype) if bias is not None else F32, _ptr(scale_result), _ptr(out),
                              _dtype_code(out_dtype), m, n, k, variant))
    return out

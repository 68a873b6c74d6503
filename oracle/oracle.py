"""CPU oracle for the quantised matrix products: ctypes bindings of qmm_oracle.c.

TEST INFRASTRUCTURE ONLY: the checker that the CUDA path is compared against.
Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the product never does.

Functions take and return CPU torch tensors and mirror the aten signatures of
the reference's ops (crates/pyvk/csrc/quant.cpp:59-310). Parity is pinned in
tests/test_oracle.py: bit for bit against the installed PyTorch's CPU kernels
for the dyn-int4 ops and the float8/16-bit conversions, within the reference's
own test bound for the int8 and float8 products, and against the committed
golden vectors under tests/golden/.
"""

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_F8 = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1, torch.float8_e4m3fnuz: 2, torch.float8_e5m2fnuz: 3}
_OUT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float8_e4m3fn: 3, torch.float8_e5m2: 4,
        torch.float8_e4m3fnuz: 5, torch.float8_e5m2fnuz: 6}


def build(force=False):
    """Compiles qmm_oracle.c with gcc (oracle/Makefile)."""
    src = os.path.join(_HERE, "qmm_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "_build/liboracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_f32_to_f8.restype = ctypes.c_uint8
        _lib.oracle_f32_to_f8.argtypes = [ctypes.c_float, ctypes.c_int]
        _lib.oracle_f8_to_f32.restype = ctypes.c_float
        _lib.oracle_f8_to_f32.argtypes = [ctypes.c_uint8, ctypes.c_int]
        _lib.oracle_f32_to_f16.restype = ctypes.c_uint16
        _lib.oracle_f32_to_f16.argtypes = [ctypes.c_float]
        _lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
        _lib.oracle_f32_to_bf16.argtypes = [ctypes.c_float]
    return _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _i64(v):
    return ctypes.c_int64(int(v))


def weight_int8pack_mm(a, b, scales):
    """aten::_weight_int8pack_mm as qmm8.slang computes it (quant.cpp:59-119)."""
    m, k = a.shape
    n = b.shape[0]
    assert a.stride(1) == 1 or k == 1
    s = scales.to(a.dtype).contiguous()  # (the CPU reads the scales as A's dtype, quant.cpp:84)
    b = b.contiguous()
    c = torch.empty(m, n, dtype=a.dtype)
    if c.numel():
        lib().oracle_qmm8(_p(a), _i64(a.stride(0)), _p(b), _p(s), _p(c), _i64(m), _i64(n), _i64(k),
                          ctypes.c_int(_DT[a.dtype]))
    return c


def weight_int8pack_mm_f64(a, b, scales):
    """(unrounded float64 sums, magnitude sums |a| . |b s|) for error bounds."""
    m, k = a.shape
    n = b.shape[0]
    s = scales.to(a.dtype).contiguous()
    b = b.contiguous()
    c = torch.empty(m, n, dtype=torch.float64)
    mag = torch.empty(m, n, dtype=torch.float64)
    if c.numel():
        lib().oracle_qmm8_f64(_p(a), _i64(a.stride(0)), _p(b), _p(s), _p(c), _p(mag), _i64(m), _i64(n), _i64(k),
                              ctypes.c_int(_DT[a.dtype]))
    return c, mag


def dyn_quant_pack_4bit_weight(weights, scales_zeros, bias, block_size, in_features, out_features):
    """aten::_dyn_quant_pack_4bit_weight (quant.cpp:127-144)."""
    w = weights.contiguous().reshape(-1)
    sc = scales_zeros.contiguous().reshape(-1)
    if sc.dtype not in (torch.float32, torch.bfloat16):
        sc = sc.float()
    bvec = None if bias is None else bias.float().contiguous().reshape(-1)
    nb = 0 if bvec is None else bvec.numel()
    packed = torch.empty(w.numel() + sc.numel() + nb, dtype=torch.float32)
    lib().oracle_qmm4_pack(_p(w), _i64(w.numel()), _p(sc), _i64(sc.numel()), ctypes.c_int(_DT[sc.dtype]), _p(bvec),
                           _i64(nb), _p(packed))
    return packed


def dyn_quant_quantize(inp, groupwise):
    """qmm4.slang PHASE 0: (q int32 [M,K], 1/scale [M], -zp int32 [M], scale [M])."""
    x = inp.contiguous()
    m, k = x.shape
    q = torch.empty(m, k, dtype=torch.int32)
    recip = torch.empty(m, dtype=torch.float32)
    neg_zp = torch.empty(m, dtype=torch.int32)
    scale = torch.empty(m, dtype=torch.float32)
    lib().oracle_qmm4_quantize(_p(x), ctypes.c_int(_DT[x.dtype]), _i64(m), _i64(k), ctypes.c_int(1 if groupwise else 0),
                               _p(q), _p(recip), _p(neg_zp), _p(scale))
    return q, recip, neg_zp, scale


def dyn_quant_matmul_4bit(inp, packed, block_size, in_features, out_features, return_iacc=False):
    """aten::_dyn_quant_matmul_4bit (quant.cpp:146-204, qmm4.slang)."""
    m, k, n, bs = inp.shape[0], in_features, out_features, block_size
    packed = packed.float().contiguous()
    q, recip, neg_zp, _ = dyn_quant_quantize(inp, bs != k)
    nblocks = (k + bs - 1) // bs
    has_bias = packed.numel() - (n * k // 2 + n * nblocks)
    assert has_bias in (0, n)
    out = torch.empty(m, n, dtype=inp.dtype)
    iacc = torch.empty(m, n, nblocks, dtype=torch.int32) if return_iacc else None
    if out.numel():
        lib().oracle_qmm4_matmul(_p(q), _p(recip), _p(neg_zp), _p(packed), _p(out), ctypes.c_int(_DT[inp.dtype]),
                                 _i64(m), _i64(n), _i64(k), _i64(bs), ctypes.c_int(1 if has_bias else 0), _p(iacc))
    return (out, iacc) if return_iacc else out


def scaled_mm(a, b, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None, acc64=False):
    """aten::_scaled_mm as the reference's emulated product (quant.cpp:283-299).

    acc64=True accumulates in float64 and returns (out, unrounded float64 sums).
    """
    m, k = a.shape
    n = b.shape[1]
    out_dtype = out_dtype or a.dtype
    rowwise = not (scale_a.numel() == 1 and scale_b.numel() == 1)  # (tensor-wise is tested first, quant.cpp:245)
    sa = scale_a.float().contiguous().reshape(-1)
    sb = scale_b.float().contiguous().reshape(-1)
    bvec = None if bias is None else bias.float().contiguous()
    inv = 1.0
    if out_dtype in _F8 and scale_result is not None:
        inv = float(torch.tensor(1.0) / scale_result.float().reshape(()))
    out = torch.empty(m, n, dtype=out_dtype)
    ref64 = torch.empty(m, n, dtype=torch.float64) if acc64 else None
    au, bu = a.view(torch.uint8), b.view(torch.uint8)
    if out.numel():
        lib().oracle_scaled_mm(_p(au), ctypes.c_int(_F8[a.dtype]), _i64(a.stride(0)), _i64(a.stride(1)),
                               _p(bu), ctypes.c_int(_F8[b.dtype]), _i64(b.stride(0)), _i64(b.stride(1)),
                               _p(sa), _p(sb), ctypes.c_int(1 if rowwise else 0), _p(bvec), ctypes.c_float(inv),
                               _p(out.view(torch.uint8) if out_dtype in _F8 else out), ctypes.c_int(_OUT[out_dtype]),
                               _i64(m), _i64(n), _i64(k), ctypes.c_int(1 if acc64 else 0), _p(ref64))
    return (out, ref64) if acc64 else out

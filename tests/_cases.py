"""Seeded inputs shared by the CPU and GPU tests.

The shapes, seeds and distributions of the first three groups are those of the
reference's own tests (tests/python/test_quant.py:20-128); the `config_*`
generators follow the benchmark configurations' shapes and distributions.
"""

import torch

FLOAT8 = [torch.float8_e4m3fn, torch.float8_e5m2]

INT8_SHAPES = [(32, 64, 48), (1, 4096, 300), (5, 100, 17), (70, 33, 5), (65, 1, 66)]
INT8_DTYPES = [torch.float32, torch.float16, torch.bfloat16]
DYN4_CASES = [(1, 64, 4096, 32, False), (32, 128, 11008, 32, True), (5, 96, 70, 96, True), (3, 100, 9, 100, False),
              (4, 256, 16, 64, True), (9, 64, 33, 64, False)]


def gen(seed):
    return torch.Generator().manual_seed(seed)


def int8_case(dtype, m, k, n):
    a = torch.randn(m, k, generator=gen(1)).to(dtype)
    b = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=gen(2))
    s = (torch.rand(n, generator=gen(3)) / 50).to(dtype)
    return a, b, s


def int8_want(a, b, s):
    """The reference test's expected value and error bound (test_quant.py:31-37)."""
    want = (a.float() @ (b.float() * s.float()[:, None]).t()).to(a.dtype)
    mag = a.float().abs() @ (b.float() * s.float()[:, None]).abs().t()
    tol = torch.finfo(a.dtype).eps * want.float().abs() + 2**-20 * mag
    return want, tol


def pack_case(n, k, bs, seed, bias):
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=gen(seed))
    nb = 1 if bs == k else k // bs
    sc = torch.rand(n, nb, generator=gen(seed + 1)) / 10
    sc = sc if bs == k else sc.to(torch.bfloat16)
    return w, sc, (torch.randn(n, generator=gen(seed + 2)) if bias else None)


def dyn4_case(m, k, n, bs, bias, dtype):
    w, sc, bvec = pack_case(n, k, bs, 7, bias)
    x = (torch.randn(m, k, generator=gen(11)) * 3).to(dtype)
    x[0, : k // 2] = 0.0  # a row's quantisation with zeros, and one all negative
    if m > 1:
        x[1] = -x[1].abs()
    return x, w, sc, bvec


def scaled_case(fa, fb, out_dtype, rowwise, m=16, k=32, n=48):
    a = torch.randn(m, k, generator=gen(1)).to(fa)
    b = torch.randn(n, k, generator=gen(2)).to(fb).t()
    sa = torch.rand(m, 1, generator=gen(3)) + 0.5 if rowwise else torch.tensor(1.25)
    sb = torch.rand(1, n, generator=gen(4)) + 0.5 if rowwise else torch.tensor(0.75)
    bias = torch.randn(n, generator=gen(5)).to(torch.bfloat16) if out_dtype == torch.bfloat16 else None
    scale_result = torch.tensor(2.0) if out_dtype == torch.float8_e4m3fn else None
    return a, b, sa, sb, bias, scale_result


def scaled_want(a, b, sa, sb, bias, scale_result, out_dtype):
    """The reference's emulated product in torch ops (quant.cpp:283-299) and the
    test's error bound (test_quant.py:124-126)."""
    out_dtype = out_dtype or a.dtype
    af, bf = a.float() * sa, b.float() * sb
    r = af @ bf
    if bias is not None:
        r = r + bias.float()
    if out_dtype in FLOAT8:
        r = r * (1 / (float(scale_result) if scale_result is not None else 1.0))
    want = r.to(out_dtype)
    mag = af.abs() @ bf.abs() / (float(scale_result) if scale_result is not None and out_dtype in FLOAT8 else 1.0)
    tol = torch.finfo(out_dtype).eps * want.float().abs() + 2**-20 * mag
    return want, tol


# ---- benchmark configurations (synthetic, seeded) ---------------------------

def config_int8(m, k, n, dtype, seed=0):
    """int8 weight-only: A ~ N(0,1); W uniform in [-127,127]; scales uniform in [1e-3, 2e-2]."""
    a = torch.randn(m, k, generator=gen(seed + 1)).to(dtype)
    b = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen(seed + 2))
    s = (torch.rand(n, generator=gen(seed + 3)) * (2e-2 - 1e-3) + 1e-3).to(dtype)
    return a, b, s


def config_dyn4(m, k=4096, n=14336, bs=32, seed=0):
    """dyn-int4: input ~ N(0,1); nibbles uniform; bf16 scales uniform in [5e-3,5e-2]; bias ~ N(0,0.1)."""
    x = torch.randn(m, k, generator=gen(seed + 11))
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=gen(seed + 7))
    sc = (torch.rand(n, k // bs, generator=gen(seed + 8)) * (5e-2 - 5e-3) + 5e-3).to(torch.bfloat16)
    bias = torch.randn(n, generator=gen(seed + 9)) * 0.1
    return x, w, sc, bias


def config_fp8(m, k, n, rowwise, seed=0):
    """fp8: values ~ N(0,1)*64 clamped to +-448; scales 1/64 or uniform in [1/128, 1/32]."""
    a = (torch.randn(m, k, generator=gen(seed + 1)) * 64).clamp(-448, 448).to(torch.float8_e4m3fn)
    b = (torch.randn(n, k, generator=gen(seed + 2)) * 64).clamp(-448, 448).to(torch.float8_e4m3fn).t()
    if rowwise:
        sa = torch.rand(m, 1, generator=gen(seed + 3)) * (1 / 32 - 1 / 128) + 1 / 128
        sb = torch.rand(1, n, generator=gen(seed + 4)) * (1 / 32 - 1 / 128) + 1 / 128
    else:
        sa, sb = torch.tensor(1 / 64), torch.tensor(1 / 64)
    return a, b, sa, sb

"""Pins the CPU oracle (oracle/qmm_oracle.c): against the installed PyTorch's
CPU kernels, which the reference's shaders copy and its tests compare with
(tests/python/test_quant.py), and against the committed golden vectors."""

import ctypes
import hashlib
import json
import os

import pytest
import torch

import _cases as C
from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


F8_KINDS = ((torch.float8_e4m3fn, 0), (torch.float8_e5m2, 1), (torch.float8_e4m3fnuz, 2), (torch.float8_e5m2fnuz, 3))


def test_float8_decode_all_codes():
    for dt, kind in F8_KINDS:
        want = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(dt).float()
        got = torch.tensor([O.lib().oracle_f8_to_f32(c, kind) for c in range(256)])
        assert torch.equal(got.isnan(), want.isnan())
        assert torch.equal(got[~got.isnan()].view(torch.int32), want[~want.isnan()].view(torch.int32))


def _probe_floats():
    g = C.gen(5)
    bits = torch.randint(-2**31, 2**31 - 1, (20000,), generator=g, dtype=torch.int64).to(torch.int32)
    rand = bits.view(torch.float32)
    scaled = torch.randn(20000, generator=g) * torch.tensor([1e-3, 1.0, 100.0, 5e4])[torch.randint(0, 4, (20000,), generator=g)]
    edges = []
    f8 = [dt for dt, _ in F8_KINDS]
    for dt in f8 + [torch.float16, torch.bfloat16]:
        n = 256 if dt in f8 else 65536
        if dt in f8:
            vals = torch.arange(n, dtype=torch.int32).to(torch.uint8).view(dt).float()
        else:
            vals = torch.arange(n, dtype=torch.int32).to(torch.int16).view(dt).float()[::37]
        vals = vals[vals.isfinite()]
        srt = vals.sort().values
        mid = (srt[1:] + srt[:-1]) / 2  # halfway cases
        for v in (srt, mid):
            vb = v.view(torch.int32)
            edges += [v, (vb + 1).view(torch.float32), (vb - 1).view(torch.float32)]
    special = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 448.0, 464.0, 465.0, 480.0, 57344.0,
                            61440.0, 65504.0, 65519.9, 65520.0, 1e-8, 2**-25, 2**-24, 3 * 2**-26, 240.0, 247.9, 248.0, 256.0, -1e-10,
                            2**-11, 3 * 2**-12, 2**-18, 3 * 2**-19, -2**-19])
    return torch.cat([rand, scaled, special] + edges)


def test_float_encoders_match_c10():
    x = _probe_floats()
    lib = O.lib()
    for dt, kind in F8_KINDS:
        want = x.to(dt).view(torch.uint8)
        got = torch.tensor([lib.oracle_f32_to_f8(float(v), kind) for v in x.tolist()], dtype=torch.uint8)
        nan = x.isnan()
        assert torch.equal(got[~nan], want[~nan])
        if kind < 2:
            assert ((got[nan] & 0x7f) == 0x7f).all()
        else:
            assert (got[nan] == 0x80).all()  # (the fnuz formats' one NaN)
    want16 = x.to(torch.float16).view(torch.int16)
    got16 = torch.tensor([lib.oracle_f32_to_f16(float(v)) for v in x.tolist()], dtype=torch.int32).to(torch.int16)
    nan = x.isnan()
    assert torch.equal(got16[~nan], want16[~nan])
    wantb = x.to(torch.bfloat16).view(torch.int16)
    gotb = torch.tensor([lib.oracle_f32_to_bf16(float(v)) for v in x.tolist()], dtype=torch.int32).to(torch.int16)
    assert torch.equal(gotb[~nan], wantb[~nan])


@pytest.mark.parametrize("dtype", C.INT8_DTYPES)
@pytest.mark.parametrize("m,k,n", C.INT8_SHAPES)
def test_int8_oracle_within_reference_bound(dtype, m, k, n):
    a, b, s = C.int8_case(dtype, m, k, n)
    want, tol = C.int8_want(a, b, s)
    got = O.weight_int8pack_mm(a, b, s)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert ((got.float() - want.float()).abs() <= tol).all()
    sliced = O.weight_int8pack_mm(a[::2], b, s)
    assert ((sliced.float() - want[::2].float()).abs() <= tol[::2]).all()
    # the float64 sum agrees too
    ref64, mag = O.weight_int8pack_mm_f64(a, b, s)
    assert ((got.double() - ref64).abs() <= torch.finfo(dtype).eps * ref64.abs() + 2**-20 * mag).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_int8_oracle_vs_cpu_kernel(dtype):
    # PyTorch's own CPU kernel (k a multiple of 16: its AVX bf16 path's limit, test_quant.py:28-30)
    a, b, s = C.int8_case(dtype, 7, 256, 40)
    want = torch._weight_int8pack_mm(a, b, s)
    _, tol = C.int8_want(a, b, s)
    assert ((O.weight_int8pack_mm(a, b, s).float() - want.float()).abs() <= tol).all()


@pytest.mark.parametrize("m,k,n,bs,bias", C.DYN4_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dyn4_oracle_bit_exact_vs_cpu_kernel(m, k, n, bs, bias, dtype):
    if dtype == torch.bfloat16 and bs != k:
        pytest.skip("bfloat16 inputs are channelwise only (the CPU's check)")
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
    packed = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    assert torch.equal(O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n), packed)
    want = torch._dyn_quant_matmul_4bit(x, packed, bs, k, n)
    got = O.dyn_quant_matmul_4bit(x, packed, bs, k, n)
    assert got.dtype == want.dtype
    assert torch.equal(got, want)


def test_dyn4_block_sums_are_the_integer_products():
    x, w, sc, bvec = C.dyn4_case(4, 256, 16, 64, True, torch.float32)
    packed = O.dyn_quant_pack_4bit_weight(w, sc, bvec, 64, 256, 16)
    _, iacc = O.dyn_quant_matmul_4bit(x, packed, 64, 256, 16, return_iacc=True)
    q, recip, neg_zp, scale = O.dyn_quant_quantize(x, True)
    wi = torch.stack([(w & 15).int() - 8, (w >> 4).int() - 8], dim=-1).reshape(16, 256)
    want = torch.einsum("mbk,nbk->mnb", (q + neg_zp[:, None]).reshape(4, 4, 64).long(), wi.reshape(16, 4, 64).long())
    assert torch.equal(iacc.long(), want)
    assert (q >= -128).all() and (q <= 127).all()
    assert torch.equal(recip, 1.0 / scale)


@pytest.mark.parametrize("fa,fb", [(C.FLOAT8[0], C.FLOAT8[0]), (C.FLOAT8[1], C.FLOAT8[0]), (C.FLOAT8[0], C.FLOAT8[1])])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float16, torch.float8_e4m3fn, None])
@pytest.mark.parametrize("rowwise", [False, True])
def test_scaled_mm_oracle_within_reference_bound(fa, fb, out_dtype, rowwise):
    a, b, sa, sb, bias, sr = C.scaled_case(fa, fb, out_dtype, rowwise)
    want, tol = C.scaled_want(a, b, sa, sb, bias, sr, out_dtype)
    got = O.scaled_mm(a, b, sa, sb, bias, sr, out_dtype)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert ((got.float() - want.float()).abs() <= tol).all()
    got64, ref64 = O.scaled_mm(a, b, sa, sb, bias, sr, out_dtype, acc64=True)
    assert ((got64.float() - want.float()).abs() <= tol).all()


def _digest(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def test_golden_vectors():
    """The committed fixtures (made by tests/golden/make_golden.py from PyTorch's
    CPU kernels) still match: bit for bit where the op is exact."""
    with open(os.path.join(GOLDEN, "golden.json")) as f:
        golden = json.load(f)
    for case in golden["dyn4"]:
        m, k, n, bs, bias = case["shape"]
        dtype = getattr(torch, case["dtype"])
        x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
        packed = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
        assert _digest(packed) == case["packed_sha256"]
        got = O.dyn_quant_matmul_4bit(x, packed, bs, k, n)
        assert _digest(got) == case["out_sha256"], case
        assert got.reshape(-1)[:8].float().tolist() == case["out_head"]
    for case in golden["int8"]:
        m, k, n = case["shape"]
        dtype = getattr(torch, case["dtype"])
        a, b, s = C.int8_case(dtype, m, k, n)
        got = O.weight_int8pack_mm(a, b, s)
        want = torch.tensor(case["out_head"])
        _, tol = C.int8_want(a, b, s)
        assert ((got.reshape(-1)[:16].float() - want).abs() <= tol.reshape(-1)[:16]).all()
    for case in golden["fp8"]:
        fa, fb = getattr(torch, case["fa"]), getattr(torch, case["fb"])
        od = getattr(torch, case["out_dtype"]) if case["out_dtype"] else None
        a, b, sa, sb, bias, sr = C.scaled_case(fa, fb, od, case["rowwise"])
        got = O.scaled_mm(a, b, sa, sb, bias, sr, od)
        _, tol = C.scaled_want(a, b, sa, sb, bias, sr, od)
        want = torch.tensor(case["out_head"])
        assert ((got.reshape(-1)[:16].float() - want).abs() <= tol.reshape(-1)[:16]).all()

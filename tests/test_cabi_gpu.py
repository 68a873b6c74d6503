"""GPU parity of the CUDA kernels, called through the C ABI (include/tvb200.h) with
device pointers, against the CPU oracle on the same seeded inputs. The cases are the
reference's own (tests/python/test_quant.py) plus shapes around the kernels' tile
sizes. Bit-exact where the op is integer / defined bit for bit (dyn-int4), within
the reference's error bound elsewhere."""

import pytest
import torch

import _cases as C
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    from torch_vulkan_b200 import cabi

    assert cabi.lib().tvb_device_count() >= 1, cabi.lib().tvb_last_error()
    return cabi


def dev(t):
    return None if t is None else t.cuda()


# ---------------------------------------------------------------- int8 weight-only

@pytest.mark.parametrize("dtype", C.INT8_DTYPES)
@pytest.mark.parametrize("m,k,n", C.INT8_SHAPES)
def test_qmm8_reference_cases(abi, dtype, m, k, n):
    a, b, s = C.int8_case(dtype, m, k, n)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s))
    sliced = abi.qmm8(dev(a)[::2], dev(b), dev(s))
    abi.synchronize()
    assert ((got.cpu().float() - want.float()).abs() <= tol).all()
    assert ((sliced.cpu().float() - want[::2].float()).abs() <= tol[::2]).all()
    oracle = O.weight_int8pack_mm(a, b, s)
    assert ((got.cpu().float() - oracle.float()).abs() <= 2 * tol).all()


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(1, 128, 8), (1, 256, 257), (3, 1024, 255), (8, 4096, 300), (9, 512, 1000), (16, 2048, 4099),
                                   (13, 8192, 520), (33, 256, 77), (64, 384, 513), (17, 1024, 300), (32, 4096, 1000), (40, 2048, 3001),
                                   (64, 8192, 1024), (50, 128, 40)])
def test_qmm8_kernel_variants(abi, variant, dtype, m, k, n):
    a, b, s = C.config_int8(m, k, n, dtype, seed=m + n)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s), variant=variant)
    abi.synchronize()
    err = (got.cpu().float() - want.float()).abs()
    assert (err <= tol).all(), f"max excess {(err - tol).max()}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(17, 64, 8), (128, 128, 256), (130, 144, 264), (64, 4096, 1000), (300, 1024, 515), (1, 256, 300),
                                   (512, 2048 + 16, 768)])
def test_qmm8_tcgen05(abi, dtype, m, k, n):
    a, b, s = C.config_int8(m, k, n, dtype, seed=m + n)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s), variant=3)
    sliced = abi.qmm8(dev(a)[::2], dev(b), dev(s), variant=3) if (k % 8 == 0 and m > 1) else None
    abi.synchronize()
    err = (got.cpu().float() - want.float()).abs()
    assert (err <= tol).all(), f"max excess {(err - tol).max()}"
    if sliced is not None:
        assert ((sliced.cpu().float() - want[::2].float()).abs() <= tol[::2]).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(1024, 512, 768), (1500, 1040, 520), (17, 64, 8), (2048, 4096, 1000)])
def test_qmm8_widened_gemm(abi, dtype, m, k, n):
    # variant 4: the weights widened once into scratch, then the 16-bit tcgen05 GEMM with the scales in its epilogue;
    # a second product with other weights must not see the first one's scratch
    for seed in (m + n, m + n + 1):
        a, b, s = C.config_int8(m, k, n, dtype, seed=seed)
        want, tol = C.int8_want(a, b, s)
        got = abi.qmm8(dev(a), dev(b), dev(s), variant=4)
        abi.synchronize()
        err = (got.cpu().float() - want.float()).abs()
        assert (err <= tol).all(), f"max excess {(err - tol).max()}"
    if m >= 1024:  # the automatic choice from 1024 rows on
        auto = abi.qmm8(dev(a), dev(b), dev(s))
        abi.synchronize()
        assert torch.equal(auto.cpu(), got.cpu())


def test_qmm8_skinny_is_deterministic_and_repeatable(abi):
    a, b, s = C.config_int8(16, 1024, 3000, torch.bfloat16)
    da, db, ds = dev(a), dev(b), dev(s)
    first = abi.qmm8(da, db, ds, variant=2)
    for _ in range(3):
        again = abi.qmm8(da, db, ds, variant=2)
        abi.synchronize()
        assert torch.equal(first, again)


def test_qmm8_skinny_scratch_layout_across_shapes(abi):
    # a narrow product (whose partial sums land in scratch) followed by a wide one (more than 64 tiles of 256 columns,
    # whose tile counters must not alias what the narrow one left behind)
    for m, k, n in ((4, 1024, 300), (4, 256, 20000), (16, 512, 40000), (1, 1024, 700), (8, 256, 33000)):
        a, b, s = C.config_int8(m, k, n, torch.bfloat16, seed=n)
        want, tol = C.int8_want(a, b, s)
        got = abi.qmm8(dev(a), dev(b), dev(s), variant=2)
        abi.synchronize()
        assert ((got.cpu().float() - want.float()).abs() <= tol).all(), (m, k, n)


@pytest.mark.parametrize("m", [1, 16])
def test_qmm8_decode_is_deterministic(abi, m):
    # Tiles are shared between CTAs; whichever of them finishes a tile, by whichever route (a CTA that finds the
    # others' sums waiting takes a shortcut), the additions happen in one fixed order: every run gives the same bits.
    a, b, s = C.config_int8(m, 8192, 7168, torch.bfloat16, seed=5)
    ad, bd, sd = dev(a), dev(b), dev(s)
    first = abi.qmm8(ad, bd, sd, variant=2)
    abi.synchronize()
    first = first.cpu()
    want, tol = C.int8_want(a, b, s)
    assert ((first.float() - want.float()).abs() <= tol).all()
    for _ in range(25):
        again = abi.qmm8(ad, bd, sd, variant=2)
        abi.synchronize()
        assert torch.equal(first.view(torch.int16), again.cpu().view(torch.int16))


def test_qmm8_decode_back_to_back_launches_agree(abi):
    # Launches queued without waiting overlap (programmatic dependent launch): CTAs start at different times, so which
    # contributor of a shared tile arrives last, and through which of the kernel's routes the tile is finished, varies from
    # launch to launch. The result must not: every repeat equals the first, unhurried one bit for bit.
    shapes = [(16, 8192, 7168), (4, 4096, 4096), (1, 8192, 3584), (8, 2048, 12288), (16, 14336, 4096)]
    cases = []
    for i, (m, k, n) in enumerate(shapes):
        a, b, s = C.config_int8(m, k, n, torch.bfloat16, seed=40 + i)
        ad, bd, sd = dev(a), dev(b), dev(s)
        first = abi.qmm8(ad, bd, sd)
        abi.synchronize()
        want, tol = C.int8_want(a, b, s)
        assert ((first.cpu().float() - want.float()).abs() <= tol).all(), (m, k, n)
        cases.append((ad, bd, sd, first.cpu().view(torch.int16)))
    outs = []
    for rep in range(40):
        for ci in ((rep * 3) % 5, (rep * 3 + 1) % 5, (rep * 3 + 2) % 5):
            ad, bd, sd, _ = cases[ci]
            outs.append((ci, abi.qmm8(ad, bd, sd)))
    abi.synchronize()
    for ci, out in outs:
        assert torch.equal(out.cpu().view(torch.int16), cases[ci][3]), shapes[ci]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(1, 256, 257), (5, 1024, 300), (16, 2048, 4099), (16, 8192, 8192), (20, 512, 1000),
                                   (32, 4096, 4096), (8, 14336, 4096), (40, 512, 300), (3, 200, 64)])
def test_qmm8_linear_equals_product_then_adds(abi, dtype, m, k, n):
    # bias and residual added where the decode kernel finishes a tile (m <= 32, k a multiple of 128), by further passes
    # otherwise: either way bit for bit the product followed by the two adds, each rounded to the dtype
    a, b, s = C.config_int8(m, k, n, dtype, seed=3 * m + n)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(dtype)
    res = (torch.randn(m, n, generator=torch.Generator().manual_seed(m)) * 4).to(dtype)
    ad, bd, sd, biasd, resd = dev(a), dev(b), dev(s), dev(bias), dev(res)
    prod = abi.qmm8(ad, bd, sd)
    abi.synchronize()
    prod = prod.cpu()
    both = abi.qmm8_linear(ad, bd, sd, biasd, resd)
    only_bias = abi.qmm8_linear(ad, bd, sd, biasd, None)
    only_res = abi.qmm8_linear(ad, bd, sd, None, resd)
    neither = abi.qmm8_linear(ad, bd, sd)
    abi.synchronize()
    bits = lambda t: t.cpu().view(torch.int16)  # noqa: E731
    assert torch.equal(bits(neither), bits(prod))
    assert torch.equal(bits(only_bias), bits(prod + bias))
    assert torch.equal(bits(only_res), bits(prod + res))
    assert torch.equal(bits(both), bits((prod + bias) + res))
    assert torch.equal(resd.cpu(), res)  # (the operands are left alone)
    if m <= 32 and k % 128 == 0:
        stream = resd.clone()  # x += proj(h): the output over the residual
        abi.qmm8_linear(ad, bd, sd, biasd, stream, out=stream)
        abi.synchronize()
        assert torch.equal(bits(stream), bits((prod + bias) + res))


def test_qmm8_decode_shape_sample(abi):
    # the decode benchmark's k with a slice of its n: every SM's unit range crosses tiles
    a, b, s = C.config_int8(4, 8192, 3584, torch.bfloat16)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s))
    abi.synchronize()
    assert ((got.cpu().float() - want.float()).abs() <= tol).all()


def test_qmm8_fp32_config1(abi):
    a, b, s = C.config_int8(32, 4096, 4096, torch.float32)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s))
    abi.synchronize()
    assert ((got.cpu() - want).abs() <= tol).all()


# ---------------------------------------------------------------- dyn-int4

@pytest.mark.parametrize("m,k,n,bs,bias", C.DYN4_CASES + [(33, 512, 130, 128, True), (70, 1024, 257, 32, True),
                                                             (2, 4096, 512, 32, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qmm4_bit_exact(abi, m, k, n, bs, bias, dtype):
    if dtype == torch.bfloat16 and bs != k:
        pytest.skip("bfloat16 inputs are channelwise only (the CPU's check)")
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
    packed = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want, want_iacc = O.dyn_quant_matmul_4bit(x, packed, bs, k, n, return_iacc=True)
    wq, wrecip, wzp, _ = O.dyn_quant_quantize(x, bs != k)

    packed_dev = abi.qmm4_pack(dev(w), dev(sc), dev(bvec))
    q, recip, neg_zp = abi.qmm4_quantize(dev(x), bs != k)
    got, iacc = abi.qmm4_matmul(q, recip, neg_zp, packed_dev, n, k, bs, dtype, return_iacc=True)
    fused = abi.qmm4(dev(x), dev(packed), bs, k, n)
    abi.synchronize()
    assert torch.equal(packed_dev.cpu(), packed)
    assert torch.equal(q.cpu().int(), wq)
    assert torch.equal(recip.cpu().view(torch.int32), wrecip.view(torch.int32))
    assert torch.equal(neg_zp.cpu(), wzp)
    assert torch.equal(iacc.cpu(), want_iacc)
    assert torch.equal(got.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    assert torch.equal(fused.cpu(), want)


# ---------------------------------------------------------------- float8

@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("fa,fb", [(C.FLOAT8[0], C.FLOAT8[0]), (C.FLOAT8[1], C.FLOAT8[0]), (C.FLOAT8[0], C.FLOAT8[1])])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float16, torch.float8_e4m3fn, None])
@pytest.mark.parametrize("rowwise", [False, True])
def test_scaled_mm_reference_cases(abi, variant, fa, fb, out_dtype, rowwise):
    a, b, sa, sb, bias, sr = C.scaled_case(fa, fb, out_dtype, rowwise)
    want, tol = C.scaled_want(a, b, sa, sb, bias, sr, out_dtype)
    got = abi.scaled_mm(dev(a), dev(b), dev(sa), dev(sb), dev(bias), dev(sr), out_dtype, variant=variant)
    abi.synchronize()
    assert got.dtype == want.dtype and got.shape == want.shape
    assert ((got.cpu().float() - want.float()).abs() <= tol).all()


@pytest.mark.parametrize("fa,fb", [(C.FLOAT8[0], C.FLOAT8[0]), (C.FLOAT8[1], C.FLOAT8[0]), (C.FLOAT8[0], C.FLOAT8[1])])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float16, torch.float8_e4m3fn])
@pytest.mark.parametrize("rowwise", [False, True])
@pytest.mark.parametrize("m,k,n", [(128, 128, 256), (130, 144, 264), (1, 16, 8), (257, 1024, 511), (384, 4096 + 32, 768)])
def test_scaled_mm_tcgen05(abi, fa, fb, out_dtype, rowwise, m, k, n):
    a, b, sa, sb, bias, sr = C.scaled_case(fa, fb, out_dtype, rowwise, m=m, k=k, n=n)
    want, tol = C.scaled_want(a, b, sa, sb, bias, sr, out_dtype)
    got = abi.scaled_mm(dev(a), dev(b), dev(sa), dev(sb), dev(bias), dev(sr), out_dtype, variant=2)
    abi.synchronize()
    err = (got.cpu().float() - want.float()).abs()
    ok = err <= tol
    # float8 outputs: a value within float32 rounding of a rounding boundary may land on either neighbour
    if out_dtype in C.FLOAT8:
        assert ok.float().mean() > 0.999
        up = (want.float().abs() * 2**-2).clamp_min(2**-9)
        assert (err <= up + tol).all()
    else:
        assert ok.all(), f"max excess {(err - tol).max()} at {(err - tol).argmax()}"


@pytest.mark.parametrize("fa,fb", [(C.FLOAT8[0], C.FLOAT8[0]), (C.FLOAT8[1], C.FLOAT8[0])])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float8_e4m3fn])
@pytest.mark.parametrize("rowwise", [False, True])
@pytest.mark.parametrize("m,k,n", [(256, 128, 256), (130, 144, 264), (257, 1024, 511), (384, 4096 + 32, 768), (1100, 512, 1300)])
def test_scaled_mm_cta_pairs(abi, fa, fb, out_dtype, rowwise, m, k, n):
    """The kernel that puts a pair of CTAs on each 256 x 256 tile (variant 3), ragged edges in both dimensions included."""
    a, b, sa, sb, bias, sr = C.scaled_case(fa, fb, out_dtype, rowwise, m=m, k=k, n=n)
    want, tol = C.scaled_want(a, b, sa, sb, bias, sr, out_dtype)
    got = abi.scaled_mm(dev(a), dev(b), dev(sa), dev(sb), dev(bias), dev(sr), out_dtype, variant=3)
    abi.synchronize()
    err = (got.cpu().float() - want.float()).abs()
    ok = err <= tol
    if out_dtype in C.FLOAT8:
        assert ok.float().mean() > 0.999
        up = (want.float().abs() * 2**-2).clamp_min(2**-9)
        assert (err <= up + tol).all()
    else:
        assert ok.all(), f"max excess {(err - tol).max()} at {(err - tol).argmax()}"


def test_scaled_mm_config4_sample(abi):
    for rowwise in (False, True):
        a, b, sa, sb = C.config_fp8(512, 8192, 1024, rowwise)
        want, tol = C.scaled_want(a, b, sa, sb, None, None, torch.bfloat16)
        got = abi.scaled_mm(dev(a), dev(b), dev(sa), dev(sb), None, None, torch.bfloat16)
        abi.synchronize()
        assert ((got.cpu().float() - want.float()).abs() <= tol).all()
        # the benchmark's stated bound: within 2 bfloat16 ulp of the float64-accumulated product
        ref64 = (a.double() * sa.double()) @ (b.double() * sb.double())
        ulp = torch.finfo(torch.bfloat16).eps * ref64.abs().clamp_min(2.0**-8 * ref64.abs().max())
        assert ((got.cpu().double() - ref64).abs() <= 2 * ulp).all()


# ---------------------------------------------------------------- dyn-int4 on the tensor cores (bit-exact too)

@pytest.mark.parametrize("m,k,n,bs,bias", [(1, 64, 4096, 32, False), (32, 128, 11008, 32, True), (5, 96, 70, 96, True),
                                           (4, 256, 16, 64, True), (9, 64, 33, 64, False), (130, 512, 300, 32, True),
                                           (257, 1024, 129, 128, False), (64, 4096, 256, 4096, True), (200, 2048, 520, 2048, False),
                                           (128, 4096, 1024, 32, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qmm4_tensor_core_path_bit_exact(abi, m, k, n, bs, bias, dtype):
    if dtype == torch.bfloat16 and bs != k:
        pytest.skip("bfloat16 inputs are channelwise only (the CPU's check)")
    if m * n * k > 3e8:
        # too slow for the scalar oracle: compare with the bit-exact CUDA-core kernel, itself checked against the oracle
        x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
        packed = abi.qmm4_pack(dev(w), dev(sc), dev(bvec))
        want = abi.qmm4(dev(x), packed, bs, k, n)
        abi.synchronize()
        want = want.cpu()
    else:
        x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
        packed_cpu = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
        want = O.dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
        packed = dev(packed_cpu)
    prepared = abi.qmm4_prepare(packed, n, k, bs)
    got = abi.qmm4_tc(dev(x), packed, prepared, bs, k, n)
    again = abi.qmm4_tc(dev(x), packed, prepared, bs, k, n)
    abi.synchronize()
    view = torch.int16 if dtype == torch.bfloat16 else torch.int32
    assert torch.equal(got.cpu().view(view), want.view(view))
    assert torch.equal(again.cpu().view(view), want.view(view))


@pytest.mark.parametrize("m,k,n,bs,bias", [(1, 64, 4096, 32, False), (32, 128, 11008, 32, True), (5, 96, 70, 96, True),
                                           (4, 256, 16, 64, True), (9, 64, 33, 64, False), (130, 512, 300, 32, True),
                                           (257, 1024, 129, 128, False), (64, 4096, 256, 4096, True), (200, 2048, 520, 2048, False),
                                           (128, 4096, 1024, 32, True), (300, 2080, 260, 32, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qmm4_float16_form_bit_exact(abi, m, k, n, bs, bias, dtype):
    """tvb_qmm4_tc16: float16 copies of the integers on kind::f16; with blocks of 32 values and scales from bfloat16 the
    drain is one fma per output and block. Bit for bit the oracle's (or the CUDA-core kernel's) result either way."""
    if dtype == torch.bfloat16 and bs != k:
        pytest.skip("bfloat16 inputs are channelwise only (the CPU's check)")
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
    if bs == 32:
        sc = sc.clone()
        sc[::3] = -sc[::3]            # negative scales: the sign of a zero block sum's product
        sc[1::5] = sc[1::5] * 2.0**-100   # and tiny ones (still normal, still 8 significant bits)
    if m * n * k > 3e8:
        packed = abi.qmm4_pack(dev(w), dev(sc), dev(bvec))
        want = abi.qmm4(dev(x), packed, bs, k, n)
        abi.synchronize()
        want = want.cpu()
    else:
        packed_cpu = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
        want = O.dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
        packed = dev(packed_cpu)
    prepared = abi.qmm4_prepare16(packed, n, k, bs)
    got = abi.qmm4_tc16(dev(x), packed, prepared, bs, k, n)
    again = abi.qmm4_tc16(dev(x), packed, prepared, bs, k, n)
    abi.synchronize()
    flag = prepared[:4].cpu().view(torch.int32).item()
    assert flag == (0 if bs != k else flag)  # groupwise scales come from bfloat16: the fused drain where bs is 32
    view = torch.int16 if dtype == torch.bfloat16 else torch.int32
    assert torch.equal(got.cpu().view(view), want.view(view))
    assert torch.equal(again.cpu().view(view), want.view(view))


def test_qmm4_float16_form_any_scales(abi):
    # float32 group scales with full mantissas, blocks of 32: the flag says so and the drain multiplies and adds
    m, k, n, bs = 70, 512, 200, 32
    x, w, _, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
    sc = torch.rand(n, k // bs, generator=C.gen(5)) / 10 + 1e-3
    packed_cpu = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = O.dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
    packed = dev(packed_cpu)
    prepared = abi.qmm4_prepare16(packed, n, k, bs)
    got = abi.qmm4_tc16(dev(x), packed, prepared, bs, k, n)
    abi.synchronize()
    assert prepared[:4].cpu().view(torch.int32).item() == 3
    assert torch.equal(got.cpu(), want)


def test_qmm4_tensor_core_path_wide_scales(abi):
    # float32 group scales with full mantissas: the drain must not use the 3*s shortcut
    m, k, n, bs = 20, 256, 96, 64
    x, w, _, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
    sc = torch.rand(n, k // bs, generator=C.gen(5)) / 10 + 1e-3
    packed_cpu = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = O.dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
    packed = dev(packed_cpu)
    prepared = abi.qmm4_prepare(packed, n, k, bs)
    got = abi.qmm4_tc(dev(x), packed, prepared, bs, k, n)
    abi.synchronize()
    assert prepared[:4].cpu().view(torch.int32).item() & 1 == 1
    assert torch.equal(got.cpu(), want)


# ---------------------------------------------------------------- dyn-int4, the decode kernel (at most 16 rows, bit-exact)

@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("k,n,bs,bias", [(512, 8, 32, True), (512, 40, 32, False), (1024, 264, 128, True), (2048, 96, 64, False),
                                          (4096, 1000, 32, True), (4096, 512, 512, True), (512, 2400, 64, True),
                                          (8192, 48, 256, True), (1536, 20000, 32, False)])
def test_qmm4_decode_bit_exact(abi, m, k, n, bs, bias):
    assert abi.lib().tvb_qmm4_decode_usable(m, n, k, bs) == 1
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, torch.float32)
    packed_cpu = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = O.dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
    packed = dev(packed_cpu)
    prepared = abi.qmm4_decode_prepare(packed, n, k, bs)
    got = abi.qmm4_decode(dev(x), packed, prepared, bs, k, n)
    again = abi.qmm4_decode(dev(x), packed, prepared, bs, k, n)
    abi.synchronize()
    assert torch.equal(got.cpu().view(torch.int32), want.view(torch.int32))
    assert torch.equal(again.cpu().view(torch.int32), want.view(torch.int32))


def test_qmm4_decode_full_size_and_limits(abi):
    # the benchmark's weights at m = 16 against the tensor-core kernel (itself checked against the oracle)
    m, k, n, bs = 16, 4096, 14336, 32
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
    packed = abi.qmm4_pack(dev(w), dev(sc), dev(bvec))
    want = abi.qmm4_tc(dev(x), packed, abi.qmm4_prepare(packed, n, k, bs), bs, k, n)
    got = abi.qmm4_decode(dev(x), packed, abi.qmm4_decode_prepare(packed, n, k, bs), bs, k, n)
    abi.synchronize()
    assert torch.equal(got.cpu(), want.cpu())
    lib = abi.lib()
    for shape in ((17, 64, 512, 32), (4, 60, 512, 32), (4, 64, 16384, 32), (4, 64, 4096, 4096), (4, 64, 768, 32), (4, 64, 1024, 96)):
        assert lib.tvb_qmm4_decode_usable(*shape) == 0, shape  # m > 16, n % 8, k too long, one block per row, k % 512, 512 % bs


# ---------------------------------------------------------------- dyn-int4, the opt-in fast route (not bit-exact)

@pytest.mark.parametrize("m,k,n,bs,bias", [(32, 128, 11008, 32, True), (130, 512, 300, 32, True), (257, 1024, 129, 128, False),
                                           (64, 4096, 256, 64, True), (5, 96, 70, 96, True)])
def test_qmm4_fast_route_within_float32_accumulation(abi, m, k, n, bs, bias):
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, torch.float32)
    sc = sc.to(torch.bfloat16)  # (block scales as the groupwise op takes them; channelwise float32 ones are not exact in float16)
    packed_cpu = O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = O.dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
    packed = dev(packed_cpu)
    prepared, inexact = abi.qmm4_fast_prepare(packed, n, k, bs)
    assert inexact == 0
    got = abi.qmm4_fast(dev(x), packed, prepared, bs, k, n)
    abi.synchronize()
    # the benchmark's bound: rtol 1e-5, with a magnitude floor for outputs that cancel to near zero
    assert torch.allclose(got.cpu(), want, rtol=1e-5, atol=1e-5 * float(want.abs().max()))


def test_qmm4_fast_route_flags_inexact_scales(abi):
    m, k, n, bs = 4, 256, 64, 64
    x, w, _, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
    sc = torch.rand(n, k // bs, generator=C.gen(5)) / 10 + 1e-3  # full float32 mantissas
    packed = dev(O.dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n))
    _, inexact = abi.qmm4_fast_prepare(packed, n, k, bs)
    assert inexact == 1


# ---------------------------------------------------------------- sharded product on one GPU, and a wait that runs out

def test_gather_world1_counts_and_chains(abi):
    """tvb_qmm8_gather with a world of one rank: the product lands in the rank's own buffer, every CTA's share adds up to
    1024 per product in the arrival counter, the product count advances, and a second product takes the first one's
    output as its A with no call in between."""
    import ctypes

    lib = abi.lib()
    m, k, n = 4, 1024, 512
    a, b, s = C.config_int8(m, k, n, torch.bfloat16, seed=5)
    s = (s.float() / 20).to(torch.bfloat16)
    _, b2, s2 = C.config_int8(m, n, 384, torch.bfloat16, seed=6)
    da, db, ds, db2, ds2 = dev(a), dev(b), dev(s), dev(b2), dev(s2)
    c1 = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    c2 = torch.zeros(m, 384, dtype=torch.bfloat16, device="cuda")
    state = torch.zeros(64, dtype=torch.int32, device="cuda")  # [0, 32): arrival counters [slot][rank]; [32]: product count
    torch.cuda.synchronize()
    flags = (ctypes.c_void_p * 1)(state.data_ptr())
    seq = state.data_ptr() + 128
    for c, aa, bb, ss, nn, kk in ((c1, da, db, ds, n, k), (c2, c1, db2, ds2, 384, n)):
        outs = (ctypes.c_void_p * 1)(c.data_ptr())
        abi.check(lib.tvb_qmm8_gather(0, aa.data_ptr(), abi.BF16, aa.stride(0), bb.data_ptr(), ss.data_ptr(), outs, flags, 1, 0,
                                      ctypes.c_void_p(seq), 0, m, nn, kk))
    abi.check(lib.tvb_wait_flags(0, state.data_ptr(), 1, ctypes.c_void_p(seq)))
    abi.synchronize()
    st = state.cpu()
    assert st[0].item() == 1024 and st[8].item() == 1024 and st[32].item() == 2  # products 0 and 1: slots 0 and 1
    want1, tol1 = C.int8_want(a, b, s)
    assert ((c1.cpu().float() - want1.float()).abs() <= tol1).all()
    want2, tol2 = C.int8_want(c1.cpu(), b2, s2)
    assert ((c2.cpu().float() - want2.float()).abs() <= tol2).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ms,k,n", [((1, 4, 16), 1024, 4096), ((3, 8), 512, 1000), ((16, 16, 16, 16), 256, 136), ((2,), 8192, 12288),
                                    ((1, 4, 16), 4096, 18432)])
def test_group_products_in_one_launch(abi, dtype, ms, k, n):
    """tvb_qmm8_group: several products of one shape in one launch of the decode kernel. Every product within the reference's
    bound of the CPU result and of tvb_qmm8's; a second launch repeats the first bit for bit."""
    import ctypes

    lib = abi.lib()
    cases = [C.config_int8(m, k, n, dtype, seed=40 + i) for i, m in enumerate(ms)]
    devs = [(dev(a), dev(b), dev(s)) for a, b, s in cases]
    outs = [torch.zeros(m, n, dtype=dtype, device="cuda") for m in ms]
    items = (abi.TvbGroupItem * len(ms))()
    keep = []
    for i, ((da, db, ds), out) in enumerate(zip(devs, outs)):
        ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
        keep.append(ptrs)
        items[i].a, items[i].a_sm, items[i].b, items[i].scales = da.data_ptr(), da.stride(0), db.data_ptr(), ds.data_ptr()
        items[i].c_ranks, items[i].m = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p)), ms[i]
    torch.cuda.synchronize()
    code = abi.BF16 if dtype == torch.bfloat16 else abi.F16
    abi.check(lib.tvb_qmm8_group(0, code, items, len(ms), n, k))
    abi.synchronize()
    first = [o.clone() for o in outs]
    for o in outs:
        o.zero_()
    torch.cuda.synchronize()
    abi.check(lib.tvb_qmm8_group(0, code, items, len(ms), n, k))
    abi.synchronize()
    eps = torch.finfo(dtype).eps
    for (a, b, s), (da, db, ds), out, f in zip(cases, devs, outs, first):
        want, tol = C.int8_want(a, b, s)
        assert ((out.cpu().float() - want.float()).abs() <= tol).all()
        assert torch.equal(out, f)
        single = abi.qmm8(da, db, ds)
        abi.synchronize()
        # (one step of the output type where the sum is not small against its terms; float32 rounding of the terms otherwise)
        assert ((out.float() - single.float()).abs().cpu() <= eps * single.float().abs().cpu() + tol).all()
    # what the entry point refuses
    items[0].m = 17
    assert lib.tvb_qmm8_group(0, code, items, len(ms), n, k) == -1 and b"m <= 16" in lib.tvb_last_error()
    items[0].m = ms[0]
    assert lib.tvb_qmm8_group(0, code, items, 5, n, k) == -1


def test_group_products_into_host_memory(abi):
    """The grouped launch with page-locked host tensors as outputs: the kernel's stores are the copy to the host."""
    from torch_vulkan_b200 import shard

    ms, k, n = (1, 4, 16), 2048, 6144
    cases = [C.config_int8(m, k, n, torch.bfloat16, seed=80 + i) for i, m in enumerate(ms)]
    outs = [torch.zeros(m, n, dtype=torch.bfloat16).pin_memory() for m in ms]
    devs = [(dev(a), dev(b), dev(s)) for a, b, s in cases]
    torch.cuda.synchronize()
    for rep in range(2):
        for o in outs:
            o.zero_()
        got = shard.weight_int8pack_mm_group([d[0] for d in devs], [d[1] for d in devs], [d[2] for d in devs], outs=outs, device_index=0)
        abi.synchronize()
        for (a, b, s), o in zip(cases, got):
            want, tol = C.int8_want(a, b, s)
            assert ((o.float() - want.float()).abs() <= tol).all()


def test_group_gather_world1_counts(abi):
    """tvb_qmm8_group_gather with a world of one rank: three products land in the rank's own buffers, take three product
    numbers on the channel (every CTA reports its share of each), and a following sharded product waits for all three."""
    import ctypes

    lib = abi.lib()
    ms, k, n = (1, 4, 16), 1024, 2048
    cases = [C.config_int8(m, k, n, torch.bfloat16, seed=60 + i) for i, m in enumerate(ms)]
    devs = [(dev(a), dev(b), dev(s)) for a, b, s in cases]
    outs = [torch.zeros(m, n, dtype=torch.bfloat16, device="cuda") for m in ms]
    state = torch.zeros(64, dtype=torch.int32, device="cuda")
    items = (abi.TvbGroupItem * 3)()
    keep = []
    for i, ((da, db, ds), out) in enumerate(zip(devs, outs)):
        ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
        keep.append(ptrs)
        items[i].a, items[i].a_sm, items[i].b, items[i].scales = da.data_ptr(), da.stride(0), db.data_ptr(), ds.data_ptr()
        items[i].c_ranks, items[i].m = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p)), ms[i]
    torch.cuda.synchronize()
    flags = (ctypes.c_void_p * 1)(state.data_ptr())
    seq = ctypes.c_void_p(state.data_ptr() + 128)
    for _ in range(2):  # two launches: products 0-2, then 3-5 (slots 3, 0, 1), the second waiting for the first
        abi.check(lib.tvb_qmm8_group_gather(0, abi.BF16, items, 3, flags, 1, 0, seq, 0, n, k))
    # a single sharded product after them, taking the last group's m = 16 output... as its A would need k == n; use its own A
    a4, b4, s4 = C.config_int8(4, k, 256, torch.bfloat16, seed=70)
    c4 = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    d4 = (dev(a4), dev(b4), dev(s4))
    torch.cuda.synchronize()
    abi.check(lib.tvb_qmm8_gather(0, d4[0].data_ptr(), abi.BF16, d4[0].stride(0), d4[1].data_ptr(), d4[2].data_ptr(),
                                  (ctypes.c_void_p * 1)(c4.data_ptr()), flags, 1, 0, seq, 0, 4, 256, k))
    abi.check(lib.tvb_wait_flags(0, state.data_ptr(), 1, seq))
    abi.synchronize()
    st = state.cpu()
    # products 0..6: slot q % 4 holds 1024 per product reported there
    assert [st[8 * slot].item() for slot in range(4)] == [2048, 2048, 2048, 1024] and st[32].item() == 7
    for (a, b, s), out in zip(cases, outs):
        want, tol = C.int8_want(a, b, s)
        assert ((out.cpu().float() - want.float()).abs() <= tol).all()
    want, tol = C.int8_want(a4, b4, s4)
    assert ((c4.cpu().float() - want.float()).abs() <= tol).all()
    assert lib.tvb_qmm8_group_gather(0, abi.BF16, items, 3, flags, 1, 0, seq, 2, n, k) == -1  # independent + count > 4


def test_wait_for_peers_runs_out_and_is_reported(abi):
    """A wait for a peer that never delivers gives up after the configured limit, without a fault: the host reads status 5
    from tvb_synchronize, the runtime clears the status and the decode kernels' counters, and the next product is right."""
    import ctypes
    import time

    lib = abi.lib()
    abi.check(lib.tvb_set_wait_limit_ms(20))
    try:
        # a channel of two ranks whose other rank does not exist: one product counted, nothing ever arrives
        state = torch.zeros(64, dtype=torch.int32, device="cuda")
        state[32] = 1
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        abi.check(lib.tvb_wait_flags(0, state.data_ptr(), 2, ctypes.c_void_p(state.data_ptr() + 128)))
        rc = lib.tvb_synchronize(0)
        waited = time.perf_counter() - t0
        assert rc == -1 and b"status 5" in lib.tvb_last_error()
        assert waited < 1.0, f"the wait took {waited:.2f} s with a limit of 20 ms"
        # a product kernel waiting for the previous product of such a channel gives up the same way, and still ends
        m, k, n = 2, 512, 256
        a, b, s = C.config_int8(m, k, n, torch.bfloat16, seed=9)
        da, db, ds = dev(a), dev(b), dev(s)
        mine = torch.zeros(m, 2 * n, dtype=torch.bfloat16, device="cuda")
        theirs = torch.zeros(m, 2 * n, dtype=torch.bfloat16, device="cuda")  # (stands in for the missing peer's buffer)
        their_state = torch.zeros(64, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        outs = (ctypes.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
        flags = (ctypes.c_void_p * 2)(state.data_ptr(), their_state.data_ptr())
        abi.check(lib.tvb_qmm8_gather(0, da.data_ptr(), abi.BF16, da.stride(0), db.data_ptr(), ds.data_ptr(), outs, flags, 2, 0,
                                      ctypes.c_void_p(state.data_ptr() + 128), 0, m, n, k))
        assert lib.tvb_synchronize(0) == -1 and b"status 5" in lib.tvb_last_error()
        assert lib.tvb_synchronize(0) == 0  # reported once, then cleared
    finally:
        abi.check(lib.tvb_set_wait_limit_ms(2000))
    a, b, s = C.config_int8(16, 2048, 4099, torch.bfloat16, seed=3)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s), variant=2)
    abi.synchronize()
    assert ((got.cpu().float() - want.float()).abs() <= tol).all()


# ---------------------------------------------------------------- a list of products in one launch

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_chain_is_bit_for_bit_the_single_products(abi, dtype):
    """tvb_qmm8_chain_*: products that feed one another, independent ones, a ragged one, one with several passes of 16 rows and
    one with fewer units than CTAs, all in one persistent launch; every output equals tvb_qmm8's decode kernel on the same
    inputs bit for bit, run after run, also after the inputs were rewritten in place."""
    from torch_vulkan_b200 import shard

    def weights(n, k, seed, shrink=1.0):
        _, b, s = C.config_int8(1, k, n, dtype, seed=seed)
        return dev(b), dev((s.float() * shrink).to(dtype))

    x = dev(torch.randn(4, 1024, generator=C.gen(1)).to(dtype))
    x2 = dev(torch.randn(16, 2048, generator=C.gen(2)).to(dtype))
    x3 = dev(torch.randn(40, 256, generator=C.gen(3)).to(dtype))
    x4 = dev(torch.randn(1, 8192, generator=C.gen(4)).to(dtype))
    w1, s1 = weights(640, 1024, 11, 1 / 30)
    w2, s2 = weights(384, 512, 12, 1 / 20)
    w3, s3 = weights(4099, 2048, 13)
    w4, s4 = weights(300, 256, 14)
    w5, s5 = weights(3584, 8192, 15)
    w6, s6 = weights(16, 128, 16)
    h1 = torch.zeros(4, 640, dtype=dtype, device="cuda")
    h2 = torch.zeros(4, 384, dtype=dtype, device="cuda")
    h3 = torch.zeros(4, 16, dtype=dtype, device="cuda")
    o3 = torch.zeros(16, 4099, dtype=dtype, device="cuda")
    o4 = torch.zeros(40, 300, dtype=dtype, device="cuda")
    o5 = torch.zeros(1, 3584, dtype=dtype, device="cuda")
    torch.cuda.synchronize()
    chain = shard.ProductChain([(x, w1, s1, h1), (h1[:, :512], w2, s2, h2), (x2, w3, s3, o3, 2), (h2[:, :128], w6, s6, h3, 1),
                                (x3, w4, s4, o4, 1), (x4, w5, s5, o5, 3)])
    for run in range(3):
        if run == 2:
            x.copy_(dev(torch.randn(4, 1024, generator=C.gen(9)).to(dtype)))
            x4.mul_(0.5)
            torch.cuda.synchronize()
        chain.run()
        abi.synchronize()
        for a, w, s, got in ((x, w1, s1, h1), (h1[:, :512], w2, s2, h2), (x2, w3, s3, o3), (h2[:, :128], w6, s6, h3),
                             (x3, w4, s4, o4), (x4, w5, s5, o5)):
            want = abi.qmm8(a, w, s, variant=2)
            abi.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"run {run}: {tuple(a.shape)} x {tuple(w.shape)}"
    want, tol = C.int8_want(x4.cpu(), w5.cpu(), s5.cpu())
    assert ((o5.cpu().float() - want.float()).abs() <= tol).all()


# ---------------------------------------------------------------- float32 activations on the tensor cores

@pytest.mark.parametrize("m,k,n", [(1, 64, 17), (8, 4096, 300), (32, 4096, 4096), (33, 1088, 128), (100, 256, 515), (256, 2048, 1000),
                                   (32, 8192, 640)])
def test_qmm8_float32_tensor_core_split(abi, m, k, n):
    """variant 5: float32 A as three bfloat16 terms on tcgen05 (k split over several CTAs for small matrices), against the
    reference's bound for float32 and against the CUDA-core kernel."""
    a, b, s = C.config_int8(m, k, n, torch.float32, seed=m + n)
    want, tol = C.int8_want(a, b, s)
    got = abi.qmm8(dev(a), dev(b), dev(s), variant=5)
    again = abi.qmm8(dev(a), dev(b), dev(s), variant=5)
    plain = abi.qmm8(dev(a), dev(b), dev(s), variant=1)
    abi.synchronize()
    err = (got.cpu() - want).abs()
    assert (err <= tol).all(), f"max excess {(err - tol).max()}"
    assert torch.equal(got, again)  # (the slices of k are added in a fixed order)
    assert ((got.cpu() - plain.cpu()).abs() <= 2 * tol).all()
    # against the float64 product: the error stays a small multiple of float32's rounding of the magnitude sum
    ref64, mag = O.weight_int8pack_mm_f64(a, b, s)
    assert ((got.cpu().double() - ref64).abs() <= torch.finfo(torch.float32).eps * ref64.abs() + 2.0 ** -21 * mag).all()


def test_qmm8_float32_tensor_core_special_values(abi):
    """Infinities and NaNs in A come out as the CUDA-core kernel gives them; rows of A further apart than k are fine."""
    a, b, s = C.config_int8(6, 128, 64, torch.float32, seed=3)
    a[0, 5] = float("inf")
    a[1, 7] = float("nan")
    a[2, :] = 0.0
    a[4, 1] = 1.0e-38
    wide = torch.zeros(6, 200)
    wide[:, :128] = a
    got = abi.qmm8(dev(wide)[:, :128], dev(b), dev(s), variant=5).cpu()
    plain = abi.qmm8(dev(a), dev(b), dev(s), variant=1).cpu()
    abi.synchronize()
    assert torch.equal(torch.isnan(got), torch.isnan(plain)) and torch.equal(torch.isinf(got), torch.isinf(plain))
    finite = torch.isfinite(plain)
    _, tol = C.int8_want(torch.nan_to_num(a, nan=0.0, posinf=0.0, neginf=0.0), b, s)
    assert ((got[finite] - plain[finite]).abs() <= 2 * tol[finite] + 1e-30).all()


def test_scaled_mm_gather_world1(abi):
    """tvb_scaled_mm_gather with a world of one rank equals tvb_scaled_mm's tensor-core kernel bit for bit, counts one product
    on the channel, and runs twice in a row (the second waits for the first)."""
    import ctypes

    lib = abi.lib()
    fa, fb, sa, sb = C.config_fp8(300, 512, 768, True)
    da, db = dev(fa), dev(fb.t().contiguous()).t()
    dsa, dsb = dev(sa.reshape(-1)), dev(sb.reshape(-1))
    want = abi.scaled_mm(da, db, dev(sa), dev(sb), out_dtype=torch.bfloat16, variant=2)
    state = torch.zeros(64, dtype=torch.int32, device="cuda")
    out = torch.zeros(300, 768, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    outs, flags = (ctypes.c_void_p * 1)(out.data_ptr()), (ctypes.c_void_p * 1)(state.data_ptr())
    for _ in range(2):
        abi.check(lib.tvb_scaled_mm_gather(0, da.data_ptr(), abi.E4M3, da.stride(0), da.stride(1), db.data_ptr(), abi.E4M3, db.stride(0),
                                           db.stride(1), dsa.data_ptr(), dsb.data_ptr(), 1, None, abi.F32, None, outs, abi.BF16, flags, 1, 0,
                                           ctypes.c_void_p(state.data_ptr() + 128), 0, 300, 768, 512))
    abi.check(lib.tvb_wait_flags(0, state.data_ptr(), 1, ctypes.c_void_p(state.data_ptr() + 128)))
    abi.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    st = state.cpu()
    assert st[0].item() == 1024 and st[8].item() == 1024 and st[32].item() == 2

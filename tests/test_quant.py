"""The four quantised ops on device "vk" through torch.ops.aten, vs the CPU: the
reference's own test file (tests/python/test_quant.py) carried over case for case,
with the same seeds, shapes, tolerances and error messages. Everything here must run
on the GPU: fallback_counts() stays empty by construction and is asserted."""

import contextlib

import pytest
import torch

import _cases as C

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def tv():
    import torch_vulkan_b200 as tv

    assert tv.is_available()
    yield tv
    tv.synchronize()


@contextlib.contextmanager
def on_gpu():
    """Fails if anything inside ran on the CPU (tests/python/_util.py:30-38), and checks that kernels were launched."""
    import torch_vulkan_b200 as tv

    before, launched = tv.fallback_counts(), tv.dispatch_count()
    yield
    assert tv.fallback_counts() == before == {}
    assert tv.dispatch_count() > launched


@pytest.mark.parametrize("dtype", C.INT8_DTYPES)
@pytest.mark.parametrize("m,k,n", C.INT8_SHAPES)
def test_weight_int8pack_mm(dtype, m, k, n):
    a, b, s = C.int8_case(dtype, m, k, n)
    want, tol = C.int8_want(a, b, s)
    with on_gpu():
        got = torch._weight_int8pack_mm(a.to("vk"), b.to("vk"), s.to("vk"))
        # a row slice (A's rows strided), as LLaMA's LM head passes it
        sliced = torch._weight_int8pack_mm(a.to("vk")[::2], b.to("vk"), s.to("vk"))
    assert got.device.type == "vk"
    assert got.dtype == want.dtype and got.shape == want.shape
    assert ((got.cpu().float() - want.float()).abs() <= tol).all()
    assert ((sliced.cpu().float() - want[::2].float()).abs() <= tol[::2]).all()


def test_weight_int8pack_mm_errors():
    a = torch.randn(4, 8).to("vk")
    b, s = torch.zeros(3, 8, dtype=torch.int8, device="vk"), torch.ones(3, device="vk")
    with pytest.raises(RuntimeError, match="expect B to be int8 tensor"):
        torch._weight_int8pack_mm(a, b.float(), s)
    with pytest.raises(RuntimeError, match="expect scales to be 1d tensor with size 3"):
        torch._weight_int8pack_mm(a, b, s[:2])
    with pytest.raises(RuntimeError, match="A must be contiguous on the last dimension"):
        torch._weight_int8pack_mm(a.t().contiguous().t(), b[:, :4], s)


def test_weight_int8pack_mm_empty_and_mixed_devices():
    a, b, s = C.int8_case(torch.float32, 0, 16, 5)
    assert torch._weight_int8pack_mm(a.to("vk"), b.to("vk"), s.to("vk")).shape == (0, 5)
    a, b, s = C.int8_case(torch.float32, 3, 16, 5)
    with pytest.raises(NotImplementedError, match="never falls back to the CPU"):
        torch._weight_int8pack_mm(a.to("vk"), b, s.to("vk"))


@pytest.mark.parametrize("m,k,n,bs,bias", C.DYN4_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dyn_quant_matmul_4bit_exact(m, k, n, bs, bias, dtype):
    if dtype == torch.bfloat16 and bs != k:
        pytest.skip("bfloat16 inputs are channelwise only (the CPU's check)")
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
    packed = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = torch._dyn_quant_matmul_4bit(x, packed, bs, k, n)
    with on_gpu():
        packed_vk = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), None if bvec is None else bvec.to("vk"),
                                                      bs, k, n)
        got = torch._dyn_quant_matmul_4bit(x.to("vk"), packed_vk, bs, k, n)
        got_cpu_packed = torch._dyn_quant_matmul_4bit(x.to("vk"), packed.to("vk"), bs, k, n)
    assert torch.equal(packed_vk.cpu(), packed)
    assert got.dtype == want.dtype
    assert torch.equal(got.cpu(), want)
    assert torch.equal(got_cpu_packed.cpu(), want)


def test_dyn_quant_matmul_4bit_fast_route_opt_in(monkeypatch):
    # TORCH_VK_QMM4=fast: one float16 GEMM, float32 accumulation over all of k: within rtol 1e-5 (magnitude floor)
    m, k, n, bs = 64, 512, 384, 32
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
    packed = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = torch._dyn_quant_matmul_4bit(x, packed, bs, k, n)
    packed_vk, xv = packed.to("vk"), x.to("vk")
    exact = torch._dyn_quant_matmul_4bit(xv, packed_vk, bs, k, n).cpu()
    assert torch.equal(exact, want)
    monkeypatch.setenv("TORCH_VK_QMM4", "fast")
    fast = torch._dyn_quant_matmul_4bit(xv, packed_vk, bs, k, n).cpu()
    monkeypatch.delenv("TORCH_VK_QMM4")
    assert torch.allclose(fast, want, rtol=1e-5, atol=1e-5 * float(want.abs().max()))
    assert torch.equal(torch._dyn_quant_matmul_4bit(xv, packed_vk, bs, k, n).cpu(), want)  # and exact again by default


def test_dyn_quant_errors():
    x = torch.randn(2, 64).to("vk")
    w, sc, _ = C.pack_case(8, 64, 32, 3, False)
    with pytest.raises(RuntimeError, match="Group size should be multiple of 32"):
        torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), None, 48, 64, 8)
    with pytest.raises(RuntimeError, match="expect weight to be kByte"):
        torch._dyn_quant_pack_4bit_weight(w.to("vk").char(), sc.to("vk"), None, 32, 64, 8)
    packed = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), None, 32, 64, 8)
    with pytest.raises(RuntimeError, match="expect input to be float32 or bfloat16 tensor"):
        torch._dyn_quant_matmul_4bit(x.bfloat16(), packed, 32, 64, 8)
    with pytest.raises(RuntimeError, match="Invalid packed weight tensor size"):
        torch._dyn_quant_matmul_4bit(x, packed[:100], 32, 64, 8)


@pytest.mark.parametrize("fa,fb", [(C.FLOAT8[0], C.FLOAT8[0]), (C.FLOAT8[1], C.FLOAT8[0]), (C.FLOAT8[0], C.FLOAT8[1])])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float16, torch.float8_e4m3fn, None])
@pytest.mark.parametrize("rowwise", [False, True])
def test_scaled_mm(fa, fb, out_dtype, rowwise):
    a, b, sa, sb, bias, scale_result = C.scaled_case(fa, fb, out_dtype, rowwise)
    kw = dict(bias=bias, out_dtype=out_dtype, scale_result=scale_result)
    # (the expectation is the reference's emulated formula: the installed PyTorch's CPU _scaled_mm rejects
    # row-wise scales and takes a oneDNN path the reference excludes, crates/pyvk/csrc/quant.cpp:242)
    want, tol = C.scaled_want(a, b, sa, sb, bias, scale_result, out_dtype)
    vkw = {k: (v.to("vk") if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    with on_gpu():
        got = torch._scaled_mm(a.to("vk"), b.to("vk"), sa.to("vk"), sb.to("vk"), **vkw)
        out = torch.empty(0, dtype=want.dtype, device="vk")
        torch._scaled_mm(a.to("vk"), b.to("vk"), sa.to("vk"), sb.to("vk"), **vkw, out=out)
    assert got.dtype == want.dtype and got.shape == want.shape
    for res in (got, out):
        assert ((res.cpu().float() - want.float()).abs() <= tol).all()


def test_scaled_mm_errors():
    a = torch.randn(4, 8).to(C.FLOAT8[0]).to("vk")
    b = torch.randn(6, 8).to(C.FLOAT8[0]).to("vk").t()
    one = torch.tensor(1.0, device="vk")
    with pytest.raises(ValueError, match="Invalid scaling configuration"):
        torch._scaled_mm(a, b, torch.ones(3, device="vk"), one)
    with pytest.raises(ValueError, match="out_dtype must match output matrix type"):
        torch._scaled_mm(a, b, one, one, out_dtype=torch.float32, out=torch.empty(0, device="vk", dtype=torch.half))
    with pytest.raises(RuntimeError, match="Bias must be size 6"):
        torch._scaled_mm(a, b, one, one, bias=torch.ones(5, device="vk"), out_dtype=torch.float32)


@pytest.mark.parametrize("m", [1, 7, 16, 17, 32, 33])
def test_dyn_quant_matmul_4bit_decode_sizes_match_cpu(m):
    # up to 32 rows go through the decode kernel (one or two passes of 16 rows), more through the tensor-core kernel: all
    # bit for bit the CPU's result
    k, n, bs = 1024, 264, 64
    x, w, sc, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
    packed_cpu = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
    want = torch._dyn_quant_matmul_4bit(x, packed_cpu, bs, k, n)
    packed = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), bvec.to("vk"), bs, k, n)
    got = torch._dyn_quant_matmul_4bit(x.to("vk"), packed, bs, k, n)
    again = torch._dyn_quant_matmul_4bit(x.to("vk"), packed, bs, k, n)  # (the prepared weights come from the cache now)
    assert torch.equal(got.cpu(), want) and torch.equal(again.cpu(), want)


def test_weight_int8pack_mm_prefill_reuses_widened_weights():
    # 512 rows and more: a 16-bit GEMM over a widened copy of the weights that is kept between calls; writing into the
    # weights or the scales must invalidate it
    m, k, n = 640, 1024, 776
    a, b, s = C.config_int8(m, k, n, torch.bfloat16, seed=3)
    av, bv, sv = a.to("vk"), b.to("vk"), s.to("vk")
    want, tol = C.int8_want(a, b, s)
    first = torch._weight_int8pack_mm(av, bv, sv).cpu()
    again = torch._weight_int8pack_mm(av, bv, sv).cpu()  # (from the cache)
    assert ((first.float() - want.float()).abs() <= tol).all()
    assert torch.equal(first.view(torch.int16), again.view(torch.int16))
    b2 = torch.roll(b, 5, 0)
    bv.copy_(b2.to("vk"))  # in place: the version counter moves
    want2, tol2 = C.int8_want(a, b2, s)
    got2 = torch._weight_int8pack_mm(av, bv, sv).cpu()
    assert ((got2.float() - want2.float()).abs() <= tol2).all()
    s2 = (s.float() * 2).to(torch.bfloat16)
    sv.copy_(s2.to("vk"))
    got3 = torch._weight_int8pack_mm(av, bv, sv).cpu()
    assert torch.equal(got3.float(), got2.float() * 2)  # scales doubled exactly


def test_unimplemented_ops_raise_instead_of_falling_back():
    x = torch.ones(4, device="vk")
    with pytest.raises(NotImplementedError, match="no B200 kernel"):
        torch.sin(x)


def test_device_round_trips_and_casts():
    # the boundary itself: copies, views, casts, fills (the slice of tests/python/test_core.py the ops rely on)
    for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int32, torch.int64,
                  torch.float8_e4m3fn, torch.float8_e5m2):
        x = (torch.randn(7, 9, generator=C.gen(3)) * 20).to(dtype)
        assert torch.equal(x.to("vk").cpu().view(torch.uint8), x.view(torch.uint8))
    x = torch.randn(6, 10, generator=C.gen(4))
    v = x.to("vk")
    assert torch.equal(v[::2, 1:7].cpu(), x[::2, 1:7])
    assert torch.equal(v.t().contiguous().cpu(), x.t().contiguous())
    assert torch.equal(v.bfloat16().cpu(), x.bfloat16())
    assert torch.equal(v.half().float().cpu(), x.half().float())
    big = x * 300
    for f8 in C.FLOAT8:
        got, want = big.to("vk").to(f8).cpu(), big.to(f8)
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(torch.zeros(3, 5, dtype=torch.int8, device="vk").cpu(), torch.zeros(3, 5, dtype=torch.int8))
    assert torch.equal(torch.full((4,), 2.5, device="vk").cpu(), torch.full((4,), 2.5))
    assert torch.tensor(3.25, device="vk").item() == 3.25
    import torch_vulkan_b200 as tv
    stats = tv.memory_stats()
    assert stats["reserved_bytes"] >= stats["allocated_bytes"] > 0


FNUZ = [torch.float8_e4m3fnuz, torch.float8_e5m2fnuz]


def test_fnuz_float8_casts_match_c10():
    """The fnuz formats the reference tabulates as well (crates/pyvk/csrc/backend.cpp:471-477): every code decodes, and a
    spread of values encodes, exactly as c10 does (no infinities, no negative zero, the one NaN 0x80, overflow to NaN)."""
    for f8 in FNUZ:
        codes = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(f8)
        got, want = codes.to("vk").float().cpu(), codes.float()
        assert torch.equal(got.isnan(), want.isnan()) and torch.equal(got[~want.isnan()], want[~want.isnan()])
        vals = want[~want.isnan()].sort().values
        mid = (vals[1:] + vals[:-1]) / 2  # halfway cases: ties to even
        probes = torch.cat([vals, mid, torch.nextafter(mid, torch.tensor(float("inf"))), torch.nextafter(mid, torch.tensor(-float("inf"))),
                            torch.randn(4000, generator=C.gen(8)) * 300, torch.randn(4000, generator=C.gen(9)) * 1e-3,
                            torch.tensor([0.0, -0.0, float("inf"), -float("inf"), float("nan"), 1e-12, -1e-12, 1e9, -1e9])])
        got, want = probes.to("vk").to(f8).cpu().view(torch.uint8), probes.to(f8).view(torch.uint8)
        assert torch.equal(got, want)


@pytest.mark.parametrize("fa,fb", [(FNUZ[0], FNUZ[0]), (FNUZ[1], FNUZ[0]), (FNUZ[0], C.FLOAT8[0])])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float8_e4m3fnuz])
@pytest.mark.parametrize("rowwise", [False, True])
def test_scaled_mm_fnuz(fa, fb, out_dtype, rowwise):
    """_scaled_mm with fnuz operands and outputs against the reference's emulated formula (crates/pyvk/csrc/quant.cpp:283-299)."""
    a, b, sa, sb, bias, _ = C.scaled_case(fa, fb, out_dtype, rowwise, m=40, k=96, n=72)
    scale_result = torch.tensor(2.0) if out_dtype in FNUZ else None
    want, tol = C.scaled_want(a, b, sa, sb, bias, scale_result, out_dtype)
    if out_dtype in FNUZ:  # (scaled_want's formula, with the division the fnuz output takes as well)
        af, bf = a.float() * sa, b.float() * sb
        want = ((af @ bf) * 0.5).to(out_dtype)
        tol = torch.finfo(out_dtype).eps * want.float().abs() + 2**-20 * (af.abs() @ bf.abs()) * 0.5
    kw = dict(bias=bias.to("vk") if bias is not None else None, out_dtype=out_dtype,
              scale_result=scale_result.to("vk") if scale_result is not None else None)
    with on_gpu():
        got = torch._scaled_mm(a.to("vk"), b.to("vk"), sa.to("vk"), sb.to("vk"), **kw)
    assert got.dtype == want.dtype and ((got.cpu().float() - want.float()).abs() <= tol).all()

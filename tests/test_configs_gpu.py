"""The benchmark configurations at their full sizes on device "vk": direct comparison with the CPU where the CPU
finishes in seconds, size-independent properties (row independence, column-slice consistency, linearity in the
scales) where it does not."""

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


def test_config1_fp32_int8_weight_only():
    a, b, s = C.config_int8(32, 4096, 4096, torch.float32)
    want, tol = C.int8_want(a, b, s)
    got = torch._weight_int8pack_mm(a.to("vk"), b.to("vk"), s.to("vk")).cpu()
    assert ((got - want).abs() <= tol).all()
    # the stated bound: rtol 1e-5 with a magnitude floor (outputs near zero carry the sum's absolute error)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5 * float(want.abs().max()))


@pytest.mark.parametrize("m", [1, 4, 16])
def test_config2_decode_full_size(m):
    a, b, s = C.config_int8(m, 8192, 28672, torch.bfloat16)
    want, tol = C.int8_want(a, b, s)
    bv, sv = b.to("vk"), s.to("vk")
    got = torch._weight_int8pack_mm(a.to("vk"), bv, sv).cpu()
    assert ((got.float() - want.float()).abs() <= tol).all()
    assert torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-2 * float(want.float().abs().max()))
    # a column slice of the weights gives the same columns (what sharding relies on), within the same bound
    part = torch._weight_int8pack_mm(a.to("vk"), b[7168:10752].contiguous().to("vk"), s[7168:10752].contiguous().to("vk")).cpu()
    assert ((part.float() - want[:, 7168:10752].float()).abs() <= tol[:, 7168:10752]).all()


def test_config3_dyn_int4_m128_bit_exact():
    x, w, sc, bias = C.config_dyn4(128)
    packed = torch._dyn_quant_pack_4bit_weight(w, sc, bias, 32, 4096, 14336)
    want = torch._dyn_quant_matmul_4bit(x, packed, 32, 4096, 14336)  # ~15 s of CPU
    packed_vk = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), bias.to("vk"), 32, 4096, 14336)
    assert torch.equal(packed_vk.cpu(), packed)
    got = torch._dyn_quant_matmul_4bit(x.to("vk"), packed_vk, 32, 4096, 14336).cpu()
    assert torch.equal(got, want)


@pytest.mark.parametrize("m", [512, 2048])
def test_config3_dyn_int4_large_m_properties(m):
    # rows are independent (qmm4.slang:134): any 16 rows of the large product equal the product of those rows alone,
    # bit for bit, and that small product is checked against the CPU
    x, w, sc, bias = C.config_dyn4(m)
    packed_vk = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), bias.to("vk"), 32, 4096, 14336)
    got = torch._dyn_quant_matmul_4bit(x.to("vk"), packed_vk, 32, 4096, 14336).cpu()
    rows = torch.tensor([0, 1, 127, 128, 129, 255, 256, 300, 333, 400, 401, 450, 500, 509, 510, 511]) * (m // 512)
    small = torch._dyn_quant_matmul_4bit(x[rows].contiguous().to("vk"), packed_vk, 32, 4096, 14336).cpu()
    assert torch.equal(got[rows], small)
    sub = slice(0, 256)  # and 256 output columns of those rows against the CPU's kernel
    packed_sub = torch._dyn_quant_pack_4bit_weight(w[sub], sc[sub], bias[sub], 32, 4096, 256)
    want = torch._dyn_quant_matmul_4bit(x[rows].contiguous(), packed_sub, 32, 4096, 256)
    assert torch.equal(small[:, sub], want)


@pytest.mark.parametrize("rowwise", [False, True])
def test_config4_fp8_full_size(rowwise):
    a, b, sa, sb = C.config_fp8(8192, 8192, 8192, rowwise)
    got = torch._scaled_mm(a.to("vk"), b.t().to("vk").t(), sa.to("vk"), sb.to("vk"), out_dtype=torch.bfloat16).cpu()
    # 1024 rows against the CPU's float32 product (the whole 8192^3 takes the CPU too long for a test)
    rows = slice(3072, 4096)
    af = a[rows].float() * (sa[rows] if rowwise else sa)
    bf = b.float() * sb
    ref = af @ bf
    mag = af.abs() @ bf.abs()
    tol = torch.finfo(torch.bfloat16).eps * ref.abs() + 2**-20 * mag
    assert ((got[rows].float() - ref).abs() <= tol).all()
    # within 2 bfloat16 ulp, with a magnitude floor for outputs near zero
    ulp = torch.finfo(torch.bfloat16).eps * ref.abs().clamp_min(2.0**-8 * float(ref.abs().max()))
    assert ((got[rows].float() - ref).abs() <= 2 * ulp).all()
    # the other rows: scaling A's rows by 2 scales the outputs by exactly 2 (power-of-two linearity, any size)
    sa2 = sa * 2
    got2 = torch._scaled_mm(a.to("vk"), b.t().to("vk").t(), sa2.to("vk"), sb.to("vk"), out_dtype=torch.bfloat16).cpu()
    assert torch.equal(got2.float(), got.float() * 2)


@pytest.mark.parametrize("m", [1, 8, 64])
def test_config5_layer_shapes(m):
    # one decoder layer's four int8 Linears (qkv, o, gate_up, down) with the stack's glue: slice / first half
    shapes = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}
    x = torch.randn(m, 4096, generator=C.gen(1)).to(torch.bfloat16)
    for idx, (name, (n, k)) in enumerate(shapes.items()):
        _, b, s = C.config_int8(1, k, n, torch.bfloat16, seed=1000 + idx)
        inp = x if k == 4096 else torch.randn(m, k, generator=C.gen(2)).to(torch.bfloat16)
        want, tol = C.int8_want(inp, b, s)
        got = torch._weight_int8pack_mm(inp.to("vk"), b.to("vk"), s.to("vk")).cpu()
        assert got.shape == (m, n)
        assert ((got.float() - want.float()).abs() <= tol).all(), name


def test_results_copied_out_beside_the_next_products(tv):
    """copy_to_host_overlapped: each product's result leaves on the second stream while the next product runs; eager and
    as a recorded step replayed with new inputs. Every result is compared with the CPU product."""
    from torch_vulkan_b200 import shard

    ms = [16, 4, 1]
    a_cpu = {m: C.config_int8(m, 1024, 4096, torch.bfloat16)[0] for m in ms}
    _, b, s = C.config_int8(1, 1024, 4096, torch.bfloat16)
    bv, sv = b.to("vk"), s.to("vk")
    a_pin = {m: a_cpu[m].clone().pin_memory() for m in ms}
    a_dev = {m: torch.empty_like(a_cpu[m], device="vk") for m in ms}
    out_pin = {m: torch.zeros(m, 4096, dtype=torch.bfloat16).pin_memory() for m in ms}

    def step():
        outs = []
        for m in ms:
            a_dev[m].copy_(a_pin[m], non_blocking=True)
        for m in ms:
            c = torch._weight_int8pack_mm(a_dev[m], bv, sv)
            tv.copy_to_host_overlapped(out_pin[m], c)
            outs.append(c)
        return outs

    def check(scale):
        for m in ms:
            want, tol = C.int8_want(a_cpu[m] * scale, b, s)
            assert ((out_pin[m].float() - want.float()).abs() <= tol).all()

    step()
    tv.synchronize()
    check(1.0)
    graph = shard.StepGraph(step, 0, warm=False)
    for scale in (2.0, -0.5):
        for m in ms:
            a_pin[m].copy_(a_cpu[m] * scale)
            out_pin[m].zero_()
        graph.replay()
        tv.synchronize()
        check(scale)
    with pytest.raises(ValueError):
        tv.copy_to_host_overlapped(torch.zeros(1, 4096, dtype=torch.bfloat16), graph.outputs[-1])

"""aten::mm / aten::addmm / nn.Linear on device "vk" (tvb_mm): the unquantised products either side of the quantised
ones. Reference: the float64 product of the same operands; bound: one rounding of the output type plus float32
accumulation noise, the bound the reference's tests use for its products (tests/python/test_quant.py:36-40)."""

import ctypes

import pytest
import torch

import torch_vulkan_b200 as tv
from torch_vulkan_b200 import cabi

pytestmark = pytest.mark.gpu

EPS = {torch.float32: 2.0 ** -23, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


def gen(seed):
    return torch.Generator().manual_seed(seed)


def bound(a, b, dtype):
    want = a.double() @ b.double()
    return want, EPS[dtype] * want.abs() + 2.0 ** -20 * (a.double().abs() @ b.double().abs()) + 1e-30


def raw_mm(a, b, bias, variant):
    m, k = a.shape
    n = b.shape[1]
    out = torch.empty(m, n, dtype=a.dtype, device="vk")
    code = cabi._dtype_code(a.dtype)
    cabi.check(cabi.lib().tvb_mm(0, a.data_ptr(), code, a.stride(0), a.stride(1), b.data_ptr(), b.stride(0), b.stride(1),
                                 bias.data_ptr() if bias is not None else None, code, out.data_ptr(), code, m, n, k, variant))
    cabi.synchronize()
    return out.cpu()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(128, 64, 256), (300, 520, 1000), (2048, 4096, 512), (129, 72, 264)])
def test_tvb_mm_tensor_core_kernel(dtype, m, k, n):
    a = torch.randn(m, k, generator=gen(1)).to(dtype)
    w = torch.randn(n, k, generator=gen(2)).to(dtype)  # B = w.t(): K-major, the way a Linear's weight arrives
    bias = torch.randn(n, generator=gen(3)).to(dtype)
    want, tol = bound(a, w.t(), dtype)
    got = raw_mm(a.to("vk"), w.to("vk").t(), None, 2)
    assert ((got.double() - want).abs() <= tol).all()
    got_b = raw_mm(a.to("vk"), w.to("vk").t(), bias.to("vk"), 2)
    assert ((got_b.double() - (want + bias.double())).abs() <= tol + EPS[dtype] * bias.double().abs()).all()
    plain = raw_mm(a.to("vk"), w.to("vk").t(), None, 1)
    assert ((plain.double() - want).abs() <= tol).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(256, 64, 256), (300, 520, 1000), (1100, 256, 1300)])
def test_tvb_mm_cta_pairs(dtype, m, k, n):
    """Variant 3: a pair of CTAs on each 256 x 256 tile (tcgen05 cta_group::2), bias and residual included."""
    a = torch.randn(m, k, generator=gen(1)).to(dtype)
    w = torch.randn(n, k, generator=gen(2)).to(dtype)
    bias = torch.randn(n, generator=gen(3)).to(dtype)
    res = torch.randn(m, n, generator=gen(4)).to(dtype)
    want, tol = bound(a, w.t(), dtype)
    got = raw_mm(a.to("vk"), w.to("vk").t(), bias.to("vk"), 3)
    assert ((got.double() - (want + bias.double())).abs() <= tol + EPS[dtype] * bias.double().abs()).all()
    got_r = raw_addmm(a.to("vk"), w.to("vk").t(), res.to("vk"), 3)
    assert ((got_r.double() - (want + res.double())).abs() <= tol + EPS[dtype] * (want + res.double()).abs()).all()


def raw_addmm(a, b, residual, variant, out=None):
    m, k = a.shape
    n = b.shape[1]
    out = torch.empty(m, n, dtype=a.dtype, device="vk") if out is None else out
    code = cabi._dtype_code(a.dtype)
    cabi.check(cabi.lib().tvb_addmm(0, a.data_ptr(), code, a.stride(0), a.stride(1), b.data_ptr(), b.stride(0), b.stride(1),
                                    None, code, residual.data_ptr(), cabi._dtype_code(residual.dtype), residual.stride(0),
                                    out.data_ptr(), code, m, n, k, variant))
    cabi.synchronize()
    return out.cpu()


@pytest.mark.parametrize("dtype,res_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                             (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("m,k,n", [(128, 64, 256), (300, 520, 1000), (129, 72, 264), (260, 128, 77)])
def test_tvb_addmm_residual_in_the_epilogue(dtype, res_dtype, m, k, n):
    a = torch.randn(m, k, generator=gen(11)).to(dtype)
    w = torch.randn(n, k, generator=gen(12)).to(dtype)
    res = (torch.randn(m, n, generator=gen(13)) * 4).to(res_dtype)
    want, tol = bound(a, w.t(), dtype)
    want = want + res.double()
    tol = tol + EPS[dtype] * res.double().abs()
    for variant in (2, 1):
        got = raw_addmm(a.to("vk"), w.to("vk").t(), res.to("vk"), variant)
        assert ((got.double() - want).abs() <= tol).all(), variant
    # rows of the residual further apart than n (a slice of a wider matrix), and the output written over the residual
    wide = torch.zeros(m, n + 24, dtype=res_dtype)
    wide[:, 8:8 + n] = res
    got = raw_addmm(a.to("vk"), w.to("vk").t(), wide.to("vk")[:, 8:8 + n], 2)
    assert ((got.double() - want).abs() <= tol).all()
    if res_dtype == dtype:
        inplace = res.to("vk")
        got = raw_addmm(a.to("vk"), w.to("vk").t(), inplace, 2, out=inplace)
        assert ((got.double() - want).abs() <= tol).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_aten_addmm_with_a_matrix(dtype):
    for m, k, n in ((5, 7, 3), (256, 512, 1024), (1, 64, 48)):
        a = torch.randn(m, k, generator=gen(14)).to(dtype)
        b = torch.randn(k, n, generator=gen(15)).to(dtype)
        res = torch.randn(m, n, generator=gen(16)).to(dtype)
        want, tol = bound(a, b, dtype)
        want = want + res.double()
        tol = tol + EPS[dtype] * res.double().abs()
        got = torch.addmm(res.to("vk"), a.to("vk"), b.to("vk")).cpu()
        assert got.shape == (m, n) and ((got.double() - want).abs() <= tol).all()
        res_t = res.t().contiguous().to("vk").t()  # a column-major residual is copied to rows first
        got = torch.addmm(res_t, a.to("vk"), b.to("vk")).cpu()
        assert ((got.double() - want).abs() <= tol).all()
        stream = res.to("vk")  # x = x + a @ b, written over x
        torch.addmm(stream, a.to("vk"), b.to("vk"), out=stream)
        assert ((stream.cpu().double() - want).abs() <= tol).all()


def test_tvb_mm_rejects_what_it_cannot_take():
    a = torch.randn(16, 32).to("vk")
    b = torch.randn(32, 8).to("vk")
    out = torch.empty(16, 8, device="vk")
    lib = cabi.lib()
    rc = lib.tvb_mm(0, a.data_ptr(), cabi.F32, 32, 1, b.data_ptr(), 8, 1, None, cabi.F32, out.data_ptr(), cabi.F32, 16, 8, 32, 2)
    assert rc != 0 and b"tcgen05" in lib.tvb_last_error()
    rc = lib.tvb_mm(0, a.data_ptr(), cabi.I8, 32, 1, b.data_ptr(), 8, 1, None, cabi.F32, out.data_ptr(), cabi.F32, 16, 8, 32, 0)
    assert rc != 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_aten_mm_layouts(dtype):
    for m, k, n in ((5, 7, 3), (256, 512, 1024), (1100, 264, 520)):
        a = torch.randn(m, k, generator=gen(4)).to(dtype)
        b = torch.randn(k, n, generator=gen(5)).to(dtype)
        want, tol = bound(a, b, dtype)
        av, bv = a.to("vk"), b.to("vk")
        assert ((torch.mm(av, bv).cpu().double() - want).abs() <= tol).all()  # row-major B
        bt = b.t().contiguous().to("vk").t()  # column-major B
        assert ((torch.mm(av, bt).cpu().double() - want).abs() <= tol).all()
        at_ = a.t().contiguous().to("vk").t()  # column-major A
        assert ((torch.mm(at_, bv).cpu().double() - want).abs() <= tol).all()
        out = torch.empty(0, dtype=dtype, device="vk")
        torch.mm(av, bv, out=out)
        assert out.shape == (m, n) and ((out.cpu().double() - want).abs() <= tol).all()
    assert torch.mm(torch.empty(0, 4, dtype=dtype, device="vk"), torch.empty(4, 3, dtype=dtype, device="vk")).shape == (0, 3)
    zero_k = torch.mm(torch.empty(3, 0, dtype=dtype, device="vk"), torch.empty(0, 2, dtype=dtype, device="vk")).cpu()
    assert torch.equal(zero_k, torch.zeros(3, 2, dtype=dtype))


def test_aten_mm_errors():
    a = torch.randn(4, 5).to("vk")
    with pytest.raises(RuntimeError, match="cannot be multiplied"):
        torch.mm(a, torch.randn(4, 5).to("vk"))
    with pytest.raises(RuntimeError, match="same dtype"):
        torch.mm(a, torch.randn(5, 2).to(torch.bfloat16).to("vk"))
    with pytest.raises(NotImplementedError):
        torch.mm(a.to(torch.int32), a.t().contiguous().to(torch.int32))
    with pytest.raises(NotImplementedError):
        torch.addmm(torch.randn(4, 1).to("vk"), a, torch.randn(5, 3).to("vk"))  # neither a bias vector nor a full matrix
    with pytest.raises(NotImplementedError):
        torch.addmm(torch.randn(3).to("vk"), a, torch.randn(5, 3).to("vk"), beta=0.5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_linear_module_on_vk(dtype):
    torch.manual_seed(6)
    lin = torch.nn.Linear(512, 768).to(dtype).requires_grad_(False)
    dev = torch.nn.Linear(512, 768).to(dtype).requires_grad_(False)
    dev.load_state_dict(lin.state_dict())
    dev = dev.to("vk")
    for shape in ((3, 512), (2, 130, 512), (1, 1, 512)):
        x = torch.randn(*shape, generator=gen(7)).to(dtype)
        want, tol = bound(x.reshape(-1, 512), lin.weight.t(), dtype)
        want = want + lin.bias.double()
        got = dev(x.to("vk")).cpu()
        assert got.shape == (*shape[:-1], 768)
        assert ((got.reshape(-1, 768).double() - want).abs() <= tol + EPS[dtype] * (lin.bias.double().abs() + want.abs())).all()
    tv.synchronize()

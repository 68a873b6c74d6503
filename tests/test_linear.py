"""The Linear modules over the quantised products (torch_vulkan_b200/linear.py): quantisation helpers, forward against
the dequantised float Linear, swapping the layers of a model, the on-disk form, sharding over two CPU ranks (gloo), and,
on a GPU, the same modules on device "vk" against their CPU twins."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

import torch_vulkan_b200 as tv
from torch_vulkan_b200 import linear as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_linear(k, n, bias=True, seed=0):
    torch.manual_seed(seed)
    lin = nn.Linear(k, n, bias=bias)
    return lin.requires_grad_(False)


def dequant_int4(nibbles, scales, block_size):
    n, k = nibbles.shape[0], nibbles.shape[1] * 2
    q = torch.stack([(nibbles & 15).to(torch.int16) - 8, (nibbles >> 4).to(torch.int16) - 8], dim=2).reshape(n, k).float()
    return (q.reshape(n, k // block_size, block_size) * scales.float()[:, :, None]).reshape(n, k)


def test_int8_quantisation_round_trip():
    w = torch.randn(48, 160, generator=torch.Generator().manual_seed(1))
    q, s = L.quantize_int8_per_channel(w)
    assert q.dtype == torch.int8 and s.shape == (48,) and int(q.abs().max()) <= 127
    assert ((q.float() * s[:, None] - w).abs() <= s[:, None] * 0.5 + 1e-7).all()  # half a step per element
    assert (q.abs().amax(dim=1) == 127).all()  # every row uses the full range


def test_int4_quantisation_layout():
    w = torch.randn(16, 128, generator=torch.Generator().manual_seed(2))
    nib, s = L.quantize_int4_groupwise(w, 32)
    assert nib.shape == (16, 64) and s.shape == (16, 4)
    assert ((dequant_int4(nib, s, 32) - w).abs() <= s.repeat_interleave(32, dim=1) * 0.5 + 1e-7).all()
    with pytest.raises(ValueError):
        L.quantize_int4_groupwise(torch.randn(4, 30), 32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_int8_linear_cpu_forward(dtype):
    lin = make_linear(256, 96)
    x = torch.randn(2, 5, 256, generator=torch.Generator().manual_seed(3))
    mod = L.Int8Linear.from_float(lin, dtype=dtype)
    y = mod(x.to(dtype))
    assert y.shape == (2, 5, 96) and y.dtype == dtype
    q, s = L.quantize_int8_per_channel(lin.weight)
    want = x @ (q.float() * s.to(dtype).float()[:, None]).t() + lin.bias.to(dtype).float()
    tol = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 4e-3}[dtype]
    assert ((y.float() - want).abs() <= tol * want.abs().max()).all()
    res = torch.randn(2, 5, 96, generator=torch.Generator().manual_seed(5)).to(dtype)
    assert torch.equal(mod(x.to(dtype), residual=res), y + res)
    with pytest.raises(ValueError):
        mod(x.to(dtype), residual=res[0])
    with pytest.raises(TypeError):
        mod(x.to(torch.float64))


@pytest.mark.parametrize("block_size", [32, 256])
def test_dyn_int4_linear_cpu_forward(block_size):
    lin = make_linear(256, 64)
    x = torch.randn(7, 256, generator=torch.Generator().manual_seed(4))
    mod = L.DynInt4Linear.from_float(lin, block_size=block_size)
    y = mod(x)
    nib, s = L.quantize_int4_groupwise(lin.weight, block_size)
    s = s.to(torch.bfloat16) if block_size < 256 else s
    want = x @ dequant_int4(nib, s, block_size).t() + lin.bias
    assert ((y - want).abs() <= 0.02 * want.abs().max()).all()  # the activations are quantised to 8 bits per row


def test_swap_linears_and_save_load(tmp_path):
    torch.manual_seed(5)
    model = nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Sequential(nn.Linear(128, 32, bias=False))).requires_grad_(False)
    x = torch.randn(3, 64)
    want = model(x)
    names = L.swap_linears(model, kind="int8", dtype=torch.float32, skip=lambda name, mod: name == "2.0")
    assert names == ["0"] and isinstance(model[0], L.Int8Linear) and isinstance(model[2][0], nn.Linear)
    names = L.swap_linears(model, kind="dyn4", block_size=32)
    assert names == ["2.0"] and isinstance(model[2][0], L.DynInt4Linear)
    got = model(x)
    assert ((got - want).abs() <= 0.15 * want.abs().max()).all()  # int4 weights: a few percent per layer
    for i, mod in enumerate((model[0], model[2][0])):
        path = str(tmp_path / f"layer{i}.pt")
        L.save(mod, path)
        back = L.load(path)
        assert type(back) is type(mod)
        inp = x if i == 0 else torch.relu(model[0](x))
        assert torch.equal(back(inp), mod(inp))
    with pytest.raises(ValueError):
        L.swap_linears(model, kind="fp4")


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch_vulkan_b200 import linear as LL

        lin = make_linear(128, 64)
        x = torch.randn(6, 128, generator=torch.Generator().manual_seed(6))
        ok = {}
        full8 = LL.Int8Linear.from_float(lin, dtype=torch.float32)
        ok["int8"] = torch.equal(full8.shard(rank, world)(x), full8(x))
        full4 = LL.DynInt4Linear.from_float(lin, block_size=32)
        ok["dyn4"] = torch.equal(full4.shard(rank, world)(x), full4(x))
        ok["repr"] = f"rows {rank}/{world}" in repr(full8.shard(rank, world))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_sharded_linears_match_unsharded_on_two_cpu_ranks():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert len(results) == 2
    for rank in range(2):
        assert all(results[rank].values()), (rank, dict(results[rank]))


# ---------------------------------------------------------------- on the GPU

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("bias", [True, False])
def test_int8_linear_vk_matches_cpu(dtype, bias):
    lin = make_linear(512, 384, bias=bias)
    mod = L.Int8Linear.from_float(lin, dtype=dtype)
    dev = L.Int8Linear.from_float(lin, dtype=dtype).to("vk")
    for shape in ((1, 512), (4, 3, 512), (70, 512)):
        x = torch.randn(*shape, generator=torch.Generator().manual_seed(7)).to(dtype)
        want = mod(x).float()
        got = dev(x.to("vk")).cpu().float()
        assert got.shape == want.shape
        eps = {torch.float32: 1e-5, torch.bfloat16: 2 ** -7, torch.float16: 2 ** -10}[dtype]
        # product and bias are rounded one after the other on both sides; the products may differ by one rounding step
        bmax = float(lin.bias.abs().max()) if bias else 0.0
        assert ((got - want).abs() <= 2 * eps * (want.abs() + bmax) + 1e-6).all()


@pytest.mark.gpu
def test_add_bias_on_vk_and_its_limits():
    y = torch.randn(5, 12, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    b = torch.randn(12, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    got = y.to("vk")
    got += b.to("vk")
    assert torch.equal(got.cpu(), y + b)
    assert torch.equal((y.to("vk") + b.to("vk")).cpu(), y + b)
    v = y.to("vk")[:, :8]  # a strided view: rows are 12 apart
    v += b[:8].to("vk")
    assert torch.equal(v.cpu(), y[:, :8] + b[:8])
    r = torch.randn(5, 12, generator=torch.Generator().manual_seed(10)).to(torch.bfloat16)
    assert torch.equal((y.to("vk") + r.to("vk")).cpu(), y + r)  # a tensor of the same shape: the residual stream
    y3 = torch.randn(2, 3, 8, generator=torch.Generator().manual_seed(11))
    got3 = y3.to("vk")
    got3 += (y3 * 2).to("vk")
    assert torch.equal(got3.cpu(), y3 + y3 * 2)
    with pytest.raises(NotImplementedError):
        y.to("vk") + y[:, :1].to("vk")  # no broadcasting other than a bias vector
    with pytest.raises(NotImplementedError):
        y.to("vk")[:, :8] + r.to("vk")[:, :8]  # same shape, but not contiguous
    with pytest.raises(NotImplementedError):
        torch.add(y.to("vk"), b.to("vk"), alpha=2)


@pytest.mark.gpu
def test_linears_add_the_residual_on_vk():
    lin = make_linear(512, 384)
    x = torch.randn(2, 5, 512, generator=torch.Generator().manual_seed(21))
    res = torch.randn(2, 5, 384, generator=torch.Generator().manual_seed(22))
    i8 = L.Int8Linear.from_float(lin, dtype=torch.bfloat16).to("vk")
    xb, rb = x.to(torch.bfloat16).to("vk"), res.to(torch.bfloat16)
    assert torch.equal(i8(xb, residual=rb.to("vk")).cpu(), i8(xb).cpu() + rb)  # the same two roundings as the two steps
    many = torch.randn(3, 40, 512, generator=torch.Generator().manual_seed(23)).to(torch.bfloat16)  # more rows than are decoded
    rmany = torch.randn(3, 40, 384, generator=torch.Generator().manual_seed(24)).to(torch.bfloat16)
    assert torch.equal(i8(many.to("vk"), residual=rmany.to("vk")).cpu(), i8(many.to("vk")).cpu() + rmany)
    with pytest.raises(ValueError):
        i8(xb, residual=rb[:1].to("vk"))
    i4 = L.DynInt4Linear.from_float(lin, block_size=32, device="vk")
    i4_cpu = L.DynInt4Linear.from_float(lin, block_size=32)
    assert torch.equal(i4(x.to("vk"), residual=res.to("vk")).cpu(), i4_cpu(x, residual=res.clone()))
    with pytest.raises(ValueError):
        i4(x.to("vk"), residual=res[:1].to("vk"))


@pytest.mark.gpu
@pytest.mark.parametrize("block_size,k", [(32, 512), (512, 512), (64, 448)])
def test_dyn_int4_linear_vk_is_bit_exact(block_size, k):
    lin = make_linear(k, 320)
    mod = L.DynInt4Linear.from_float(lin, block_size=block_size)
    dev = L.DynInt4Linear.from_float(lin, block_size=block_size, device="vk")
    assert torch.equal(dev.packed.cpu(), mod.packed)  # packed on the device = packed on the CPU
    for m in (1, 33, 160):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(10)) * 2
        assert torch.equal(dev(x.to("vk")).cpu(), mod(x))
    moved = mod.to("vk")  # a module packed on the CPU and moved over
    x = torch.randn(9, k, generator=torch.Generator().manual_seed(11))
    assert torch.equal(moved(x.to("vk")).cpu(), L.DynInt4Linear.from_float(lin, block_size=block_size)(x))


@pytest.mark.gpu
def test_swapped_model_and_saved_layer_on_vk(tmp_path):
    torch.manual_seed(12)
    model = nn.Sequential(nn.Linear(256, 512), nn.Linear(512, 128)).requires_grad_(False)
    ref = nn.Sequential(*[L.Int8Linear.from_float(m, dtype=torch.bfloat16) for m in model])
    L.swap_linears(model, kind="int8", dtype=torch.bfloat16, device="vk")
    x = torch.randn(4, 256).to(torch.bfloat16)
    got, want = model(x.to("vk")).cpu().float(), ref(x).float()
    assert ((got - want).abs() <= 2 ** -6 * want.abs().max()).all()
    path = str(tmp_path / "l0.pt")
    L.save(model[0], path)
    back = L.load(path, device="vk")
    assert torch.equal(back(x.to("vk")).cpu(), model[0](x.to("vk")).cpu())
    tv.synchronize()

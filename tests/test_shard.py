"""Multi-rank host logic of the column-sharded products, on CPU ranks with gloo (world size 2): slicing of weights,
scales, bias and of the packed int4 vector, and the all-gather assembly. The compute on CPU tensors is PyTorch's own
CPU kernels, standing in for the GPU kernels (which the -m gpu tests check); what is under test here is that the
sharded result equals the unsharded one bit for bit."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import _cases as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch_vulkan_b200 import shard

        ok = {}
        # int8 weight-only
        a, b, s = C.config_int8(5, 256, 96, torch.float32)
        full = torch._weight_int8pack_mm(a, b, s)
        got = shard.weight_int8pack_mm(a, shard.shard_rows(b, rank, world), shard.shard_rows(s, rank, world))
        ok["int8"] = torch.equal(got, full)
        a1 = a[:1]
        ok["int8_m1"] = torch.equal(shard.weight_int8pack_mm(a1, shard.shard_rows(b, rank, world), shard.shard_rows(s, rank, world)),
                                    torch._weight_int8pack_mm(a1, b, s))
        # dyn-int4: the packed vector is re-sliced section by section
        m, k, n, bs = 4, 256, 64, 64
        x, w, sc, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
        packed = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
        full4 = torch._dyn_quant_matmul_4bit(x, packed, bs, k, n)
        mine = shard.shard_packed_4bit(packed, bs, k, n, rank, world)
        lo, hi = shard.shard_bounds(n, rank, world)
        repacked = torch._dyn_quant_pack_4bit_weight(w[lo:hi], sc[lo:hi], bvec[lo:hi], bs, k, n // world)
        ok["pack_slice"] = torch.equal(mine, repacked)
        ok["dyn4"] = torch.equal(shard.dyn_quant_matmul_4bit(x, mine, bs, k, n // world), full4)
        # float8: the reference's emulated formula per shard
        fa, fb, sa, sb = C.config_fp8(8, 64, 32, True)
        bsh, sbsh = shard.shard_scaled_mm_b(fb, sb, rank, world)
        part = ((fa.float() * sa) @ (bsh.float() * sbsh)).to(torch.bfloat16)
        whole = ((fa.float() * sa) @ (fb.float() * sb)).to(torch.bfloat16)
        ok["fp8"] = torch.equal(shard.all_gather_columns(part), whole)
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_sharded_products_match_unsharded_on_two_cpu_ranks():
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert len(results) == 2
    for rank in range(2):
        assert all(results[rank].values()), (rank, dict(results[rank]))


def test_shard_bounds():
    from torch_vulkan_b200 import shard

    assert shard.shard_bounds(28672, 3, 8) == (10752, 14336)
    with pytest.raises(ValueError):
        shard.shard_bounds(10, 0, 4)

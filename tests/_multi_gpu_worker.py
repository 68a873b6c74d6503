"""One rank of the multi-GPU test (launched by torch.distributed.run from tests/test_multi_gpu.py): column-sharded
products on device "vk" with the NCCL all-gather, compared with the single-GPU product and the reference's bound."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import _cases as C  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    import torch_vulkan_b200 as tv
    from torch_vulkan_b200 import shard

    torch.cuda.set_device(local)
    tv.set_device(local)
    dist.init_process_group("nccl")  # (no device_id: with "vk" registered, torch takes that for the accelerator)
    dev = f"vk:{local}"
    objects = dist.new_group(backend="gloo")
    try:
        # the fused product: every rank's kernel stores its columns into every rank's buffer, flags tell arrival
        for m in (1, 4, 16):
            a, b, s = C.config_int8(m, 2048, 1024 * world, torch.bfloat16)
            want, tol = C.int8_want(a, b, s)
            outs = shard.GatheredOutputs(m, 1024 * world, torch.bfloat16, local, objects)
            av, bv, sv = a.to(dev), shard.shard_rows(b, rank, world).to(dev), shard.shard_rows(s, rank, world).to(dev)
            for rep in range(5):  # both buffers, several sequence numbers
                got = outs.weight_int8pack_mm(av, bv, sv).cpu()
                assert ((got.float() - want.float()).abs() <= tol).all(), f"rank {rank}: fused sharded product wrong (m={m}, rep={rep})"
            # the same product captured in a CUDA graph and replayed (the sequence number lives on the device)
            graph = shard.StepGraph(lambda: outs.weight_int8pack_mm(av, bv, sv), local)
            for rep in range(3):
                got = graph.replay().cpu()
                assert ((got.float() - want.float()).abs() <= tol).all(), f"rank {rank}: graph replay wrong (m={m}, rep={rep})"
            shard.barrier(objects)
        for m in (1, 4, 16):
            a, b, s = C.config_int8(m, 2048, 1024 * world, torch.bfloat16)
            want, tol = C.int8_want(a, b, s)
            full = torch._weight_int8pack_mm(a.to(dev), b.to(dev), s.to(dev)).cpu()
            got = shard.weight_int8pack_mm(a.to(dev), shard.shard_rows(b, rank, world).to(dev),
                                           shard.shard_rows(s, rank, world).to(dev)).cpu()
            assert got.shape == want.shape
            assert ((got.float() - want.float()).abs() <= tol).all(), f"rank {rank}: sharded int8 product outside the bound (m={m})"
            assert ((got.float() - full.float()).abs() <= tol).all()
        # dyn-int4: bit for bit, sharded or not
        m, k, n, bs = 40, 512, 256 * world, 32
        x, w, sc, bvec = C.dyn4_case(m, k, n, bs, True, torch.float32)
        packed = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
        want4 = torch._dyn_quant_matmul_4bit(x, packed, bs, k, n)
        mine = shard.shard_packed_4bit(packed, bs, k, n, rank, world).to(dev)
        got4 = shard.dyn_quant_matmul_4bit(x.to(dev), mine, bs, k, n // world).cpu()
        assert torch.equal(got4, want4), f"rank {rank}: sharded dyn-int4 product differs"
        # float8
        fa, fb, sa, sb = C.config_fp8(256, 1024, 512 * world, True)
        want8, tol8 = C.scaled_want(fa, fb, sa, sb, None, None, torch.bfloat16)
        bsh, sbsh = shard.shard_scaled_mm_b(fb, sb, rank, world)
        got8 = shard.scaled_mm(fa.to(dev), bsh.t().contiguous().to(dev).t(), sa.to(dev), sbsh.to(dev), out_dtype=torch.bfloat16).cpu()
        assert ((got8.float() - want8.float()).abs() <= tol8).all(), f"rank {rank}: sharded float8 product outside the bound"
        tv.synchronize(local)
        shard.barrier()
        if rank == 0:
            print("multi-gpu ok", world)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

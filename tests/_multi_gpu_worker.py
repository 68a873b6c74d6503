"""One rank of the multi-GPU test (launched by torch.distributed.run from tests/test_multi_gpu.py): column-sharded
products on device "vk", with the fused peer-store gather and with the NCCL all-gather, compared with the single-GPU
product and the reference's bound."""

import datetime
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
    # (no device_id: with "vk" registered, torch takes that for the accelerator; a short timeout: a rank that fell out must
    # not hold the others for ten minutes)
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=180))
    dev = f"vk:{local}"
    objects = dist.new_group(backend="gloo")
    try:
        # the fused product: every rank's kernel stores its columns into every rank's buffer; arrival is counted per
        # source rank, and every product kernel waits for the previous product of the channel by itself
        channel = shard.PeerChannel(local, objects)
        for m in (1, 4, 16):
            n = 1024 * world
            _, b, s = C.config_int8(m, 2048, n, torch.bfloat16)
            bv, sv = shard.shard_rows(b, rank, world).to(dev), shard.shard_rows(s, rank, world).to(dev)
            reps = 6
            a_host = [torch.randn(m, 2048, generator=C.gen(100 + r)).to(torch.bfloat16) for r in range(reps)]
            wants = [C.int8_want(a, b, s) for a in a_host]
            outs = shard.GatheredOutputs(m, n, torch.bfloat16, channel)
            av = a_host[0].to(dev)
            for rep in range(reps):  # both buffers in turn, A rewritten in place: every product has its own expected value
                av.copy_(a_host[rep].to(dev))
                got = outs.weight_int8pack_mm(av, bv, sv)
                channel.wait()
                want, tol = wants[rep]
                assert ((got.cpu().float() - want.float()).abs() <= tol).all(), f"rank {rank}: fused sharded product wrong (m={m}, rep={rep})"
            # the same product recorded twice (one graph per output buffer) and replayed in turn
            def body():
                out = outs.weight_int8pack_mm(av, bv, sv)
                channel.wait()
                return out

            graphs = [shard.StepGraph(body, local, warm=False) for _ in range(2)]
            for rep in range(reps):
                av.copy_(a_host[reps - 1 - rep].to(dev))
                got = graphs[rep % 2].replay().cpu()
                want, tol = wants[reps - 1 - rep]
                assert ((got.float() - want.float()).abs() <= tol).all(), f"rank {rank}: graph replay wrong (m={m}, rep={rep})"
            shard.barrier(objects)

        # a chain: each product takes the gathered output of the one before as its A, no call in between
        m, k0, widths = 4, 2048, (1024 * world, 512 * world, 1024 * world)
        layers, k = [], k0
        for i, n in enumerate(widths):
            _, b, s = C.config_int8(m, k, n, torch.bfloat16, seed=10 * i)
            s = (s.float() / 30).to(torch.bfloat16)  # (keeps the chain's values near one)
            layers.append((b, s, shard.shard_rows(b, rank, world).to(dev), shard.shard_rows(s, rank, world).to(dev),
                           shard.GatheredOutputs(m, n, torch.bfloat16, channel, depth=1)))
            k = n // 2  # the next product reads the first half of this one's columns
        x_host = [torch.randn(m, k0, generator=C.gen(200 + r)).to(torch.bfloat16) for r in range(4)]
        xv = x_host[0].to(dev)

        def chain():
            h, hs = xv, []
            for b, s, bv, sv, outs in layers:
                full = outs.weight_int8pack_mm(h, bv, sv)
                hs.append(full)
                h = full[:, : full.shape[1] // 2]
            channel.wait()
            return hs

        def check_chain(hs, x, what):
            h = x
            for (b, s, _, _, _), got in zip(layers, hs):
                got = got.cpu()
                want, tol = C.int8_want(h, b, s)  # (from this device's own previous output: one product's bound per step)
                assert ((got.float() - want.float()).abs() <= tol).all(), f"rank {rank}: chained sharded product wrong ({what})"
                h = got[:, : got.shape[1] // 2]

        check_chain(chain(), x_host[0], "eager")
        graph = shard.StepGraph(chain, local, warm=False)
        for rep in range(4):
            xv.copy_(x_host[rep].to(dev))
            check_chain(graph.replay(), x_host[rep], f"replay {rep}")
        shard.barrier(objects)
        # the same chain as one launch of the persistent kernel (every product waits, inside the kernel, for the columns of the
        # one before from all ranks; the launch ends when the last product has arrived from everywhere)
        prods, h = [], xv
        for b, s, bv, sv, outs in layers:
            prods.append((h, bv, sv, outs))
            h = outs.bufs[0][:, : outs.n_total // 2]
        persistent = shard.ProductChain(prods, local, channel)
        for rep in range(4):
            xv.copy_(x_host[3 - rep].to(dev))
            check_chain(persistent.run(), x_host[3 - rep], f"persistent kernel, run {rep}")
        # and a step of products that have nothing to do with each other, m = 1, 4 and 16, in one launch
        ind = []
        for i, m_ in enumerate((1, 4, 16)):
            a_, b_, s_ = C.config_int8(m_, 2048, 1024 * world, torch.bfloat16, seed=50 + i)
            ind.append((a_, b_, s_, a_.to(dev), shard.shard_rows(b_, rank, world).to(dev), shard.shard_rows(s_, rank, world).to(dev),
                        shard.GatheredOutputs(m_, 1024 * world, torch.bfloat16, channel, depth=1)))
        step = shard.ProductChain([(av_, bv_, sv_, g_, i) for i, (_, _, _, av_, bv_, sv_, g_) in enumerate(ind)], local, channel)
        for rep in range(3):
            for (a_, b_, s_, *_), got in zip(ind, step.run()):
                want, tol = C.int8_want(a_, b_, s_)
                assert ((got.cpu().float() - want.float()).abs() <= tol).all(), f"rank {rank}: independent products in one launch wrong (run {rep})"
        shard.barrier(objects)
        # the same three products as one launch of the decode kernel (tvb_qmm8_group_gather), eager and replayed with A
        # rewritten; a sharded product queued right behind the group takes the m = 4 output as its A
        _, b_n, s_n = C.config_int8(4, 1024 * world, 512 * world, torch.bfloat16, seed=77)
        s_n = (s_n.float() / 30).to(torch.bfloat16)
        bv_n, sv_n = shard.shard_rows(b_n, rank, world).to(dev), shard.shard_rows(s_n, rank, world).to(dev)
        after = shard.GatheredOutputs(4, 512 * world, torch.bfloat16, channel, depth=1)
        acts = [x[3] for x in ind]

        def grouped():
            outs = shard.weight_int8pack_mm_group(acts, [x[4] for x in ind], [x[5] for x in ind], outs=[x[6] for x in ind], bufs=[0, 0, 0])
            nxt = after.weight_int8pack_mm(outs[1], bv_n, sv_n, buf=0)
            channel.wait()
            return outs + [nxt]

        hosts = [shard.HostGathered(x[6].m, x[6].n_total, torch.bfloat16, channel, depth=1) for x in ind]

        def grouped_to_host():
            outs = shard.weight_int8pack_mm_group(acts, [x[4] for x in ind], [x[5] for x in ind], outs=[x[6] for x in ind], bufs=[0, 0, 0],
                                                  host_outs=hosts)
            channel.wait()
            return outs

        for rep in range(3):  # the same launch also storing every rank's columns into host memory that all ranks map
            scale = (1.0, -2.0, 0.5)[rep]
            for (a_, *_), av_ in zip(ind, acts):
                av_.copy_((a_ * scale).to(dev))
            for h in hosts:
                h.tensors[0].zero_()
            shard.barrier(objects)
            grouped_to_host()
            tv.synchronize()
            for (a_, b_, s_, *_), h in zip(ind, hosts):
                want, tol = C.int8_want(a_ * scale, b_, s_)
                assert ((h.tensors[0].float() - want.float()).abs() <= tol).all(), f"rank {rank}: results delivered to the host wrong (rep {rep})"
            shard.barrier(objects)
        grouped_graph = None
        for rep in range(5):
            scale = (1.0, -2.0, 0.5, 4.0, -1.0)[rep]
            for (a_, *_), av_ in zip(ind, acts):
                av_.copy_((a_ * scale).to(dev))
            if rep == 2:
                grouped_graph = shard.StepGraph(grouped, local, warm=False)
            res = grouped() if grouped_graph is None else grouped_graph.replay()
            for (a_, b_, s_, *_), got in zip(ind, res):
                want, tol = C.int8_want(a_ * scale, b_, s_)
                assert ((got.cpu().float() - want.float()).abs() <= tol).all(), f"rank {rank}: grouped sharded products wrong (rep {rep})"
            want, tol = C.int8_want(res[1].cpu(), b_n, s_n)
            assert ((res[3].cpu().float() - want.float()).abs() <= tol).all(), f"rank {rank}: product behind the group wrong (rep {rep})"
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
        # float8 with the gather fused into the tcgen05 epilogue: a shape the tensor-core kernel takes, ragged in m, both scale modes
        for rowwise in (True, False):
            fa, fb, sa, sb = C.config_fp8(300, 1024, 512 * world, rowwise)
            want8, tol8 = C.scaled_want(fa, fb, sa, sb, None, None, torch.bfloat16)
            bsh, sbsh = shard.shard_scaled_mm_b(fb, sb, rank, world)
            fav, bshv, sav, sbv = fa.to(dev), bsh.t().contiguous().to(dev).t(), sa.to(dev), sbsh.to(dev)
            outs8 = shard.GatheredOutputs(300, 512 * world, torch.bfloat16, channel)
            for rep in range(3):
                got8 = outs8.scaled_mm(fav, bshv, sav, sbv)
                channel.wait()
                assert ((got8.cpu().float() - want8.float()).abs() <= tol8).all(), f"rank {rank}: fused sharded float8 product wrong (rep {rep})"
        # the C ABI's own communicator: the slices of the dyn-int4 and float8 products assembled without torch.distributed
        comm = shard.AbiComm(local, objects)
        part4 = torch._dyn_quant_matmul_4bit(x.to(dev), mine, bs, k, n // world)
        full4 = comm.all_gather_columns(part4)
        comm.wait()
        assert torch.equal(full4.cpu(), want4), f"rank {rank}: tvb_all_gather_columns (dyn-int4) differs"
        fa, fb, sa, sb = C.config_fp8(256, 1024, 512 * world, True)
        want8, tol8 = C.scaled_want(fa, fb, sa, sb, None, None, torch.bfloat16)
        bsh, sbsh = shard.shard_scaled_mm_b(fb, sb, rank, world)
        part8 = torch._scaled_mm(fa.to(dev), bsh.t().contiguous().to(dev).t(), sa.to(dev), sbsh.to(dev), out_dtype=torch.bfloat16)
        full8 = comm.all_gather_columns(part8)
        one_row = comm.all_gather_columns(part8[:1])
        comm.wait()
        assert ((full8.cpu().float() - want8.float()).abs() <= tol8).all(), f"rank {rank}: tvb_all_gather_columns (float8) differs"
        assert torch.equal(one_row.cpu(), full8[:1].cpu())
        comm.destroy()
        tv.synchronize(local)
        shard.barrier()
        if rank == 0:
            print("multi-gpu ok", world)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

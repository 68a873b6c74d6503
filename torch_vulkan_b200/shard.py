"""Column-sharded quantised products across the GPUs of one node.

The path shards along N: every output column depends on one weight row, its scale(s) and bias, and on all of A.
Rank g of G owns rows [g*N/G, (g+1)*N/G) of the weights (and the matching scales / bias); A is replicated; the
only exchange is the all-gather of the [M, N/G] partial outputs. The reference has no multi-device mode
(crates/pyvk/csrc/backend.cpp:296: one device): this module is new functionality whose contract is "the columns
each rank computes are the columns the single-GPU op computes".

The helpers work on whatever device the tensors live on: on "vk" the products run the CUDA kernels and the gather
runs over NCCL on zero-copy CUDA views of the "vk" tensors, queued on the backend's stream; on CPU tensors with a
gloo group they run PyTorch's CPU ops, which is how the host logic is tested without GPUs.
"""

import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """[lo, hi) of the N dimension owned by `rank`; N must divide evenly (every benchmark N does)."""
    if n % world != 0:
        raise ValueError(f"N={n} is not divisible by the {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(t, rank, world):
    """Rows of a [N, ...] tensor (int8 weights, per-channel scales, bias) owned by `rank`."""
    lo, hi = shard_bounds(t.shape[0], rank, world)
    return t[lo:hi].contiguous()


def shard_scaled_mm_b(b, scale_b, rank, world):
    """Columns of the float8 B [K, N] (column-major) and of a row-wise scale_b [1, N] owned by `rank`."""
    lo, hi = shard_bounds(b.shape[1], rank, world)
    sb = scale_b if scale_b.numel() == 1 else scale_b[:, lo:hi].contiguous()
    return b[:, lo:hi], sb


def shard_packed_4bit(packed, block_size, in_features, out_features, rank, world):
    """The slice of a _dyn_quant_pack_4bit_weight vector that holds `rank`'s output features: the vector is three
    sections (weights' bytes, scales, optional bias; crates/vkcore/shaders/qmm4.slang:8-12), each sliced by rows."""
    n, k = out_features, in_features
    lo, hi = shard_bounds(n, rank, world)
    nblocks = k // block_size
    nw, ns = n * k // 2, n * nblocks
    parts = [packed[:nw].reshape(n, k // 2)[lo:hi].reshape(-1), packed[nw:nw + ns].reshape(n, nblocks)[lo:hi].reshape(-1)]
    if packed.numel() > nw + ns:
        parts.append(packed[nw + ns:nw + ns + n][lo:hi])
    return torch.cat([p.cpu() for p in parts]).to(packed.device) if packed.device.type == "vk" else torch.cat(parts)


def all_gather_columns(c_local, group=None):
    """[M, N/G] on every rank -> [M, N] on every rank (rank g's columns at [g*N/G, (g+1)*N/G))."""
    world = dist.get_world_size(group)
    if world == 1:
        return c_local
    m, n_local = c_local.shape
    c_local = c_local.contiguous()
    gathered = torch.empty((world * m, n_local), dtype=c_local.dtype, device=c_local.device)  # rank-major
    if c_local.device.type == "vk":
        import torch_vulkan_b200 as tv

        # NCCL sees CUDA views of the same memory; the collective is queued behind the product on the backend's stream
        with torch.cuda.stream(tv.cuda_stream(c_local.device.index)):
            dist.all_gather_into_tensor(tv.as_cuda(gathered), tv.as_cuda(c_local), group=group)
    else:
        dist.all_gather_into_tensor(gathered, c_local, group=group)
    if m == 1:
        return gathered.reshape(1, world * n_local)
    return gathered.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)


def weight_int8pack_mm(a, w_shard, scales_shard, group=None):
    """aten::_weight_int8pack_mm with the weight rows sharded: returns the full [M, N] on every rank."""
    return all_gather_columns(torch._weight_int8pack_mm(a, w_shard, scales_shard), group)


def dyn_quant_matmul_4bit(x, packed_shard, block_size, in_features, out_features_local, group=None):
    """aten::_dyn_quant_matmul_4bit with the output features sharded (activations are quantised on every rank:
    cheap, deterministic, identical)."""
    return all_gather_columns(torch._dyn_quant_matmul_4bit(x, packed_shard, block_size, in_features, out_features_local), group)


def scaled_mm(a, b_shard, scale_a, scale_b_shard, bias_shard=None, out_dtype=None, group=None):
    """aten::_scaled_mm with B's columns sharded."""
    c = torch._scaled_mm(a, b_shard, scale_a, scale_b_shard, bias=bias_shard, out_dtype=out_dtype)
    return all_gather_columns(c, group)


def barrier(group=None):
    """dist.barrier() for processes that registered device "vk": torch would pick "vk" (which has no collective backend)
    as the barrier's device, so the barrier is an all-reduce of one element on the group's own device."""
    if dist.get_backend(group) == "nccl":
        t = torch.zeros(1, device=torch.device("cuda", torch.cuda.current_device()))
        dist.all_reduce(t, group=group)
        torch.cuda.synchronize()
    else:
        t = torch.zeros(1)
        dist.all_reduce(t, group=group)


class AbiComm:
    """The C ABI's own communicator (tvb_comm_*: NCCL behind the library, for hosts that bind it without PyTorch): rank 0
    makes the id, the object group carries it, every rank joins. all_gather_columns assembles [m, N/G] slices into [m, N]
    on the backend's stream; wait() bounds the wait on the host and aborts the communicator instead of hanging."""

    def __init__(self, device_index, object_group, timeout_ms=30000):
        import ctypes

        from . import cabi

        self._c, self._ct, self.dev = cabi, ctypes, device_index
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        ident = ctypes.create_string_buffer(128)
        if self.rank == 0:
            cabi.check(cabi.lib().tvb_comm_unique_id(ident))
        box = [ident.raw]
        dist.broadcast_object_list(box, src=0, group=object_group)
        handle = ctypes.c_void_p(0)
        cabi.check(cabi.lib().tvb_comm_init_rank(device_index, box[0], self.world, self.rank, timeout_ms, ctypes.byref(handle)))
        self.handle = handle

    def all_gather_columns(self, c_local):
        m, n_local = c_local.shape
        c_local = c_local.contiguous()
        out = torch.empty((m, n_local * self.world), dtype=c_local.dtype, device=c_local.device)
        self._c.check(self._c.lib().tvb_all_gather_columns(self.handle, c_local.data_ptr(), out.data_ptr(), self._c._dtype_code(c_local.dtype),
                                                           m, n_local))
        self._keep = c_local  # (alive until the next call: the collective reads it on the stream)
        return out

    def wait(self, timeout_ms=30000):
        self._c.check(self._c.lib().tvb_comm_wait(self.handle, timeout_ms))

    def destroy(self):
        if self.handle:
            self._c.lib().tvb_comm_destroy(self.handle)
            self.handle = None


class PeerChannel:
    """What the ranks of one node share for the fused sharded products: every rank's array of arrival counters (one
    entry per source rank, added to by the product kernels of all ranks over NVLink) and, per rank, the device-resident
    count of products queued so far. All sharded products of a process go through one channel and are totally ordered
    on it: each product kernel waits for the previous one to have arrived from every rank before it reads its A or
    stores a column (see tvb_qmm8_gather in include/tvb200.h).

    `object_group` is a gloo group, used to exchange IPC handles. Construction is collective.
    """

    def __init__(self, device_index, object_group):
        import ctypes

        from . import cabi

        self._c, self._ct = cabi, ctypes
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.dev, self.group = device_index, object_group
        vk = torch.device("vk", device_index)
        self.state = torch.zeros(64, dtype=torch.int32, device=vk)  # [0, 32): arrival counters [slot][rank]; [32]: product count
        self.flags, self.seq = self.state[:32], self.state[32:33]
        cabi.check(cabi.lib().tvb_synchronize(device_index))  # the counters are zero before any peer may add to them
        self.flag_ptrs = self.share(self.flags)
        barrier(object_group)

    def share(self, tensor):
        """Maps `tensor` (this rank's) and every peer's counterpart into this process: a ctypes array of `world`
        device pointers, entry r being rank r's tensor. Collective; the tensor must stay alive."""
        ctypes, cabi, lib = self._ct, self._c, self._c.lib()
        handle, off = ctypes.create_string_buffer(64), ctypes.c_uint64(0)
        cabi.check(lib.tvb_ipc_export(self.dev, tensor.data_ptr(), handle, ctypes.byref(off)))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (handle.raw, off.value), group=self.group)
        ptrs = []
        for r, (h, o) in enumerate(everyone):
            if r == self.rank:
                ptrs.append(tensor.data_ptr())
            else:
                out = ctypes.c_void_p(0)
                cabi.check(lib.tvb_ipc_import(self.dev, h, o, ctypes.byref(out)))
                ptrs.append(out.value)
        return (ctypes.c_void_p * self.world)(*ptrs)

    def wait(self):
        """Queues the kernel that waits until every rank's slices of all products queued so far have arrived: what is
        queued after it on the backend's stream (copies, any other kernel) may read the gathered outputs."""
        self._c.check(self._c.lib().tvb_wait_flags(self.dev, self.flags.data_ptr(), self.world, self.seq.data_ptr()))


class GatheredOutputs:
    """Output buffers for the fused sharded decode product (tvb_qmm8_gather): every rank holds full [m, N] buffers
    (`depth` of them, written in turn) that all ranks' kernels store their column slices into directly, over NVLink
    for the peers. No collective call, no copy: the product kernel's epilogue is the gather.

    A buffer returned by weight_int8pack_mm may be handed to the next sharded product of the channel as its A at once
    (that kernel waits for the columns itself); anything else must be queued after channel.wait(). With two buffers a
    buffer is rewritten by the second product after the one that filled it, which is safe as long as its other readers
    on this rank were queued before this rank's next product. A CUDA graph freezes the buffer its products use: record
    `depth` graphs in turn (or `depth` steps per graph) when the outputs of a step are read after the step.
    """

    def __init__(self, m, n_total, dtype, channel, depth=2):
        self._c = channel._c
        self.channel, self.m, self.n_total, self.depth = channel, m, n_total, depth
        vk = torch.device("vk", channel.dev)
        self.bufs = [torch.empty((m, n_total), dtype=dtype, device=vk) for _ in range(depth)]
        self.c_ptrs = [channel.share(b) for b in self.bufs]
        self.calls = 0
        barrier(channel.group)

    def weight_int8pack_mm(self, a, w_shard, scales_shard, buf=None, independent=0):
        """Queues the product; returns the [m, N] buffer every rank's columns are stored into (`buf`: which of the
        `depth` buffers, the same on every rank; default: in turn). `independent`: how many of the channel's latest
        products this one has nothing to do with (it reads none of their outputs and writes no buffer a rank may still
        be reading while they run): it then does not wait for them."""
        cabi, lib, ch = self._c, self._c.lib(), self.channel
        m, k = a.shape
        n_local = w_shard.shape[0]
        assert m == self.m and n_local * ch.world == self.n_total and scales_shard.dtype == a.dtype
        d = self.calls % self.depth if buf is None else buf
        self.calls += 1
        cabi.check(lib.tvb_qmm8_gather(ch.dev, a.data_ptr(), cabi._dtype_code(a.dtype), a.stride(0), w_shard.data_ptr(),
                                       scales_shard.data_ptr(), self.c_ptrs[d], ch.flag_ptrs, ch.world, ch.rank,
                                       ch.seq.data_ptr(), independent, m, n_local, k))
        return self.bufs[d]


    def scaled_mm(self, a, b_shard, scale_a, scale_b_shard, bias_shard=None, buf=None, independent=0):
        """aten::_scaled_mm with B's columns sharded, the gather fused into the tcgen05 kernel's epilogue
        (tvb_scaled_mm_gather): float8 a [m, k] row-major, b_shard [k, n_local] column-major, float32 scales (one value
        each, or [m, 1] and this rank's [1, n_local]); returns the [m, N] buffer (of this object's dtype) that every
        rank's columns are stored into. Valid for the channel's next sharded product at once, for anything else after
        channel.wait()."""
        cabi, lib, ch = self._c, self._c.lib(), self.channel
        m, k = a.shape
        n_local = b_shard.shape[1]
        assert m == self.m and n_local * ch.world == self.n_total
        rowwise = 0 if (scale_a.numel() == 1 and scale_b_shard.numel() == 1) else 1
        sa, sb = scale_a.contiguous().reshape(-1), scale_b_shard.contiguous().reshape(-1)
        d = self.calls % self.depth if buf is None else buf
        self.calls += 1
        self._keep = (sa, sb)  # (alive until the next call: the kernel reads them)
        cabi.check(lib.tvb_scaled_mm_gather(ch.dev, a.data_ptr(), cabi._dtype_code(a.dtype), a.stride(0), a.stride(1), b_shard.data_ptr(),
                                            cabi._dtype_code(b_shard.dtype), b_shard.stride(0), b_shard.stride(1), sa.data_ptr(),
                                            sb.data_ptr(), rowwise, bias_shard.data_ptr() if bias_shard is not None else None,
                                            cabi._dtype_code(bias_shard.dtype) if bias_shard is not None else cabi.F32, None,
                                            self.c_ptrs[d], cabi._dtype_code(self.bufs[d].dtype), ch.flag_ptrs, ch.world, ch.rank,
                                            ch.seq.data_ptr(), independent, m, n_local, k))
        return self.bufs[d]


class HostGathered:
    """[m, n_total] result buffers (`depth` of them, used in turn) in page-locked host memory that every rank of the node
    maps: one shared-memory segment, registered with CUDA in every process. A grouped sharded launch given such buffers
    (`weight_int8pack_mm_group(..., host_outs=...)`) stores each rank's columns straight into them, so after channel.wait()
    and synchronize() every process reads the whole result from `tensors[buf]` with no copy down: a node delivers a result
    to its host once, not once per rank. Collective: every rank of the channel constructs it."""

    def __init__(self, m, n_total, dtype, channel, depth=2):
        import ctypes
        import os

        from . import cabi

        self._c, self.channel, self.m, self.n_total, self.depth = cabi, channel, m, n_total, depth
        esize = torch.empty((), dtype=dtype).element_size()
        each = (m * n_total * esize + 4095) // 4096 * 4096
        # Every step that can fail is tried locally and the ranks agree on the outcome afterwards, so that a node without
        # usable shared memory makes every rank raise the same error instead of leaving some of them in a collective.
        self._file, self._registered, ok, why = None, None, True, ""
        names = [None]
        if channel.rank == 0:
            try:
                path = f"/dev/shm/tvb200_{os.getpid()}_{id(self):x}"
                self._file = torch.from_file(path, shared=True, size=each * depth, dtype=torch.uint8)
                names[0] = path
            except Exception as exc:  # noqa: BLE001
                why = str(exc)
        src = dist.get_global_rank(channel.group, 0) if channel.group is not None else 0
        dist.broadcast_object_list(names, src=src, group=channel.group)
        self.path = names[0]
        if self.path is None:
            raise RuntimeError("HostGathered: rank 0 could not create a shared-memory file " + why)
        if channel.rank != 0:
            try:
                self._file = torch.from_file(self.path, shared=True, size=each * depth, dtype=torch.uint8)
            except Exception as exc:  # noqa: BLE001
                ok, why = False, str(exc)
        barrier(channel.group)
        if channel.rank == 0:
            os.unlink(self.path)  # (the mappings keep the memory)
        dev = ctypes.c_void_p(0)
        if ok:
            if cabi.lib().tvb_host_register(self._file.data_ptr(), each * depth, ctypes.byref(dev)) == 0:
                self._registered = self._file.data_ptr()
            else:
                ok, why = False, cabi.lib().tvb_last_error().decode("utf-8", "replace")
        flags = [None] * channel.world
        dist.all_gather_object(flags, (ok, why), group=channel.group)
        if not all(f[0] for f in flags):
            self.close()
            raise RuntimeError("HostGathered: " + "; ".join(f[1] for f in flags if not f[0]))
        self.tensors = [self._file[i * each:i * each + m * n_total * esize].view(dtype).view(m, n_total) for i in range(depth)]
        self.dev_ptrs = [dev.value + i * each for i in range(depth)]
        self.calls = 0

    def close(self):
        if getattr(self, "_registered", None) is not None:
            self._c.lib().tvb_host_unregister(self._registered)
            self._registered = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def weight_int8pack_mm_group(activations, weights, scales, outs=None, device_index=None, bufs=None, independent=0, host_outs=None):
    """Up to four int8 weight-only decode products of one shape in ONE launch (tvb_qmm8_group / tvb_qmm8_group_gather):
    products that do not depend on each other, such as one decoding step's requests against different weights. Product i is
    activations[i] [m_i, k] (m_i <= 16) times weights[i] [n, k] int8 with scales[i] [n]; n, k and the dtype are shared.

    One GPU: `outs` are the [m_i, n] output tensors (made when None); returns them. An output may also be a page-locked
    CPU tensor (`pin_memory()`): the kernel then stores that product's columns straight into host memory as they are
    finished, and no copy is needed to bring the result down (it is there after synchronize()). Sharded: `outs` are GatheredOutputs
    of one channel, one per product (weights[i] being this rank's rows), `bufs` which buffer of each to write (default: in
    turn); returns the [m_i, N] buffers, valid for the channel's next sharded product at once and for anything else after
    channel.wait(). `independent`: as for GatheredOutputs.weight_int8pack_mm, counted before the launch's first product.
    `host_outs` (sharded): one HostGathered per product; the launch also stores every product's columns into its buffer
    `bufs[i]` in host memory (see HostGathered)."""
    import ctypes

    from . import cabi

    lib, count = cabi.lib(), len(activations)
    assert 1 <= count <= 4 and len(weights) == count and len(scales) == count
    n, k = weights[0].shape
    dtype = activations[0].dtype
    items = (cabi.TvbGroupItem * count)()
    sharded = outs is not None and isinstance(outs[0], GatheredOutputs)
    keep, results = [], []
    if outs is None:
        outs = [torch.empty((a.shape[0], n), dtype=dtype, device=a.device) for a in activations]
    for i, (a, w, s, out) in enumerate(zip(activations, weights, scales, outs)):
        assert tuple(w.shape) == (n, k) and w.dtype == torch.int8 and w.is_contiguous() and a.shape[1] == k and a.stride(1) == 1
        assert a.dtype == dtype and s.dtype == dtype and s.numel() == n
        if sharded:
            assert out.m == a.shape[0] and out.n_total == n * out.channel.world and out.channel is outs[0].channel
            d = (out.calls % out.depth) if bufs is None else bufs[i]
            out.calls += 1
            ptrs, buf = out.c_ptrs[d], out.bufs[d]
        else:
            assert tuple(out.shape) == (a.shape[0], n) and out.is_contiguous() and out.dtype == dtype
            assert out.device.type != "cpu" or out.is_pinned(), "a host output must be page-locked"
            ptrs, buf = (ctypes.c_void_p * 1)(out.data_ptr()), out
        keep.append(ptrs)
        items[i].a, items[i].a_sm, items[i].b, items[i].scales = a.data_ptr(), a.stride(0), w.data_ptr(), s.data_ptr()
        items[i].c_ranks, items[i].m = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p)), a.shape[0]
        if host_outs is not None:
            h = host_outs[i]
            assert sharded and h.m == a.shape[0] and h.n_total == out.n_total
            hd = (h.calls % h.depth) if bufs is None else bufs[i]
            h.calls += 1
            items[i].c_host = h.dev_ptrs[hd]
        results.append(buf)
    if sharded:
        ch = outs[0].channel
        cabi.check(lib.tvb_qmm8_group_gather(ch.dev, cabi._dtype_code(dtype), items, count, ch.flag_ptrs, ch.world, ch.rank,
                                             ch.seq.data_ptr(), independent, n, k))
    else:
        dev = device_index if device_index is not None else (activations[0].device.index or 0)
        cabi.check(lib.tvb_qmm8_group(dev, cabi._dtype_code(dtype), items, count, n, k))
    return results


class ProductChain:
    """A fixed sequence of int8 weight-only decode products run by one persistent kernel (tvb_qmm8_chain_*): the weights
    of the next products stream in while the current one is finished, and a product may take the output of the one
    before it as its A. `products`: a list of (a, w, scales, out[, independent]) with a [m, k] (m <= 64; its buffer is
    read at every run, so the caller rewrites it in place), w int8 [n_local, k], scales [n_local], and `out` either a
    [m, n_local] tensor (one GPU) or a GatheredOutputs, alone or with the index of one of its buffers (sharded: every
    rank's columns land in every rank's buffer; outputs[i] is then that buffer). `independent` (0 to 3): how many of the products just before it this one has nothing
    to do with. With a channel the run ends only when the last product has arrived from every rank."""

    def __init__(self, products, device_index=0, channel=None):
        import ctypes

        from . import cabi

        self._c, self.dev, self.channel = cabi, device_index, channel
        world = 1 if channel is None else channel.world
        items = (cabi.TvbChainItem * len(products))()
        self._keep, self.outputs = [], []
        for i, prod in enumerate(products):
            a, w, s, out = prod[:4]
            m, k = a.shape
            n_local = w.shape[0]
            assert w.dtype == torch.int8 and w.is_contiguous() and s.dtype == a.dtype and a.stride(1) == 1
            if isinstance(out, tuple) or isinstance(out, GatheredOutputs):
                out, d = out if isinstance(out, tuple) else (out, None)  # (gathered outputs, which of its buffers)
                assert channel is not None and out.m == m and out.n_total == n_local * world
                if d is None:
                    d = out.calls % out.depth
                    out.calls += 1
                ptrs, buf = out.c_ptrs[d], out.bufs[d]
            else:
                assert world == 1 and tuple(out.shape) == (m, n_local) and out.is_contiguous() and out.dtype == a.dtype
                ptrs, buf = (ctypes.c_void_p * 1)(out.data_ptr()), out
            self._keep += [a, w, s, buf, ptrs]
            self.outputs.append(buf)
            items[i] = cabi.TvbChainItem(a.data_ptr(), a.stride(0), w.data_ptr(), s.data_ptr(), ptrs, m, n_local, k,
                                         prod[4] if len(prod) > 4 else 0, 0)
        handle = ctypes.c_void_p(0)
        dtype = cabi._dtype_code(products[0][0].dtype)
        if channel is None:
            cabi.check(cabi.lib().tvb_qmm8_chain_create(device_index, dtype, items, len(products), None, 1, 0, None, 0, ctypes.byref(handle)))
        else:
            cabi.check(cabi.lib().tvb_qmm8_chain_create(device_index, dtype, items, len(products), channel.flag_ptrs, channel.world,
                                                        channel.rank, channel.seq.data_ptr(), 1, ctypes.byref(handle)))
        self.handle = handle

    def run(self):
        self._c.check(self._c.lib().tvb_qmm8_chain_run(self.dev, self.handle))
        return self.outputs

    def __del__(self):
        try:
            self._c.lib().tvb_qmm8_chain_destroy(self.handle)
        except Exception:
            pass


class StepGraph:
    """A CUDA graph of whatever `fn` queues on the backend's stream (a decoding step: a handful of short kernels whose
    launch cost would otherwise bound the step). `fn` is run once to warm up (`warm=False`: not at all, for a step
    whose shapes have run before), then once under capture; replay() queues the recording. Tensors `fn` returns stay
    alive with the graph and are overwritten by every replay. What `fn` decides on the host is frozen: a step that
    alternates output buffers (GatheredOutputs) always replays into the buffers of the recorded call."""

    def __init__(self, fn, device_index=0, warm=True):
        import ctypes

        from . import cabi

        self._c, self.dev = cabi, device_index
        lib = cabi.lib()
        if warm:
            fn()
        cabi.check(lib.tvb_synchronize(device_index))
        cabi.check(lib.tvb_graph_begin(device_index))
        try:
            self.outputs = fn()
        finally:
            exec_ = ctypes.c_void_p(0)
            cabi.check(lib.tvb_graph_end(device_index, ctypes.byref(exec_)))
        self.exec = exec_

    def replay(self):
        self._c.check(self._c.lib().tvb_graph_launch(self.dev, self.exec))
        return self.outputs

    def __del__(self):
        try:
            self._c.lib().tvb_graph_destroy(self.exec)
        except Exception:
            pass

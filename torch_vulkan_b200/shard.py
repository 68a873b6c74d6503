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


class GatheredOutputs:
    """Output buffers for the fused sharded decode product (tvb_qmm8_gather): every rank holds a full [m, N] buffer
    (two of them, used alternately) that all ranks' kernels write their column slices into directly, over NVLink for
    the peers, plus per-buffer arrival flags. No collective call, no copy: the product kernel's epilogue is the gather.

    `object_group` is a gloo group used once, to exchange the buffers' IPC handles.
    """

    def __init__(self, m, n_total, dtype, device_index, object_group, depth=2):
        import ctypes

        from . import cabi

        self._c, self._ct = cabi, ctypes
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.dev, self.m, self.n_total, self.depth = device_index, m, n_total, depth
        vk = torch.device("vk", device_index)
        self.bufs = [torch.empty((m, n_total), dtype=dtype, device=vk) for _ in range(depth)]
        self.flags = [torch.zeros(self.world, dtype=torch.int32, device=vk) for _ in range(depth)]
        lib = cabi.lib()

        def export(t):
            handle, off = ctypes.create_string_buffer(64), ctypes.c_uint64(0)
            cabi.check(lib.tvb_ipc_export(device_index, t.data_ptr(), handle, ctypes.byref(off)))
            return handle.raw, off.value

        mine = [(export(b), export(f)) for b, f in zip(self.bufs, self.flags)]
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=object_group)

        def import_(entry):
            handle, off = entry
            out = ctypes.c_void_p(0)
            cabi.check(lib.tvb_ipc_import(device_index, handle, off, ctypes.byref(out)))
            return out.value

        self.c_ptrs, self.flag_ptrs = [], []
        for d in range(depth):
            cs, fs = [], []
            for r in range(self.world):
                if r == self.rank:
                    cs.append(self.bufs[d].data_ptr())
                    fs.append(self.flags[d].data_ptr())
                else:
                    cs.append(import_(everyone[r][d][0]))
                    fs.append(import_(everyone[r][d][1]))
            self.c_ptrs.append((ctypes.c_void_p * self.world)(*cs))
            self.flag_ptrs.append((ctypes.c_void_p * self.world)(*fs))
        self.calls = 0
        self.seq_counter = torch.ones(1, dtype=torch.int32, device=vk)  # the sequence number lives on the device
        cabi.check(lib.tvb_synchronize(device_index))  # the flags are zero before any peer may write them
        barrier(object_group)

    def weight_int8pack_mm(self, a, w_shard, scales_shard):
        """The full [m, N] product on every rank; valid for work queued after this call on the backend's stream."""
        cabi, lib = self._c, self._c.lib()
        m, k = a.shape
        n_local = w_shard.shape[0]
        assert m == self.m and n_local * self.world == self.n_total and scales_shard.dtype == a.dtype
        d = self.calls % self.depth
        self.calls += 1
        cabi.check(lib.tvb_qmm8_gather(self.dev, a.data_ptr(), cabi._dtype_code(a.dtype), a.stride(0), w_shard.data_ptr(),
                                       scales_shard.data_ptr(), self.c_ptrs[d], self.flag_ptrs[d], self.world, self.rank,
                                       self.seq_counter.data_ptr(), m, n_local, k))
        cabi.check(lib.tvb_wait_flags(self.dev, self.flags[d].data_ptr(), self.world, self.seq_counter.data_ptr()))
        return self.bufs[d]


class StepGraph:
    """A CUDA graph of whatever `fn` queues on the backend's stream (a decoding step: a handful of short kernels whose
    launch cost would otherwise bound the step). `fn` is run once to warm up, once under capture; replay() queues the
    recording. Tensors `fn` returns stay alive with the graph and are overwritten by every replay."""

    def __init__(self, fn, device_index=0):
        import ctypes

        from . import cabi

        self._c, self.dev = cabi, device_index
        lib = cabi.lib()
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

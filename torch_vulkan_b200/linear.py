"""Linear layers over the quantised matrix products: the caller's side of the path.

The reference stops at the three aten ops (crates/pyvk/csrc/quant.cpp:315-322); what calls them in a model is a
Linear whose weight was quantised ahead of time ("as LLaMA's LM head passes it", tests/python/test_quant.py:34).
These modules hold the weights in the form the ops take, so that a forward is one product (plus the bias):

* Int8Linear      aten::_weight_int8pack_mm: int8 weights [N, K], one scale per output feature.
* DynInt4Linear   aten::_dyn_quant_pack_4bit_weight once, aten::_dyn_quant_matmul_4bit per forward: int4 weights in
                  blocks of `block_size` along K (or one block per row), activations quantised per row on the fly.

Both work on whatever device their tensors live on ("vk": the B200 kernels; CPU: PyTorch's own kernels for the same ops,
which is how the logic is tested without a GPU) and both can hold one rank's slice of the output features of a Linear
sharded over the GPUs of a node (`shard(rank, world)`): the forward then assembles the full output on every rank.
`swap_linears` replaces the nn.Linear modules of a model in place; `save` / `load` keep the quantised form on disk so
that a restart skips the quantisation.
"""

import torch
from torch import nn

from . import shard as _shard


def quantize_int8_per_channel(weight):
    """float [N, K] -> (int8 [N, K], float32 scales [N]) with weight ~= q * scale: symmetric, absmax / 127 per row."""
    w = weight.detach().to(torch.float32).cpu()
    scales = w.abs().amax(dim=1).clamp_min(1e-12) / 127.0
    q = torch.round(w / scales[:, None]).clamp_(-127, 127).to(torch.int8)
    return q, scales


def quantize_int4_groupwise(weight, block_size):
    """float [N, K] -> (uint8 [N, K/2] nibble pairs, float32 scales [N, K/block_size]) in the layout
    aten::_dyn_quant_pack_4bit_weight takes: value = (nibble - 8) * scale, the even k in the low nibble, the odd k in
    the high one (as ATen/native/cpu/int4mm_kernel.cpp's ref_dyn_quant_matmul_4bit_* and the reference's shader read them)."""
    w = weight.detach().to(torch.float32).cpu()
    n, k = w.shape
    if k % 2 or k % block_size:
        raise ValueError(f"in_features={k} must be even and a multiple of block_size={block_size}")
    blocks = w.reshape(n, k // block_size, block_size)
    scales = blocks.abs().amax(dim=2).clamp_min(1e-12) / 7.0
    q = torch.round(blocks / scales[:, :, None]).clamp_(-8, 7).to(torch.int16).reshape(n, k) + 8
    packed = ((q[:, 1::2] << 4) | q[:, 0::2]).to(torch.uint8)
    return packed, scales


class _ShardedMixin:
    rank, world = 0, 1
    _group = None

    def _gather(self, y_local):
        if self.world == 1:
            return y_local
        return _shard.all_gather_columns(y_local, self._group)

    def _finish(self, y_local, lead, residual):
        """The full output in the caller's shape, with the residual stream (a tensor of that shape) added in place."""
        y = self._gather(y_local).reshape(*lead, self.full_out_features)
        if residual is not None:
            if residual.shape != y.shape:
                raise ValueError(f"residual of shape {tuple(residual.shape)} for an output of shape {tuple(y.shape)}")
            y += residual.contiguous()
        return y


class Int8Linear(nn.Module, _ShardedMixin):
    """y = x @ (weight_int8 * scales[:, None]).T + bias through aten::_weight_int8pack_mm.

    `scales` are kept in the activations' dtype (the op requires it); pass `dtype` to choose it."""

    def __init__(self, weight_int8, scales, bias=None, dtype=torch.bfloat16):
        super().__init__()
        if weight_int8.dtype != torch.int8 or weight_int8.dim() != 2:
            raise ValueError("weight_int8 must be an int8 matrix [out_features, in_features]")
        if scales.shape != (weight_int8.shape[0],):
            raise ValueError("scales must have one entry per output feature")
        self.out_features, self.in_features = weight_int8.shape
        self.register_buffer("weight", weight_int8.contiguous())
        self.register_buffer("scales", scales.to(dtype).contiguous())
        self.register_buffer("bias", None if bias is None else bias.detach().to(dtype).contiguous())
        self.full_out_features = self.out_features

    @classmethod
    def from_float(cls, linear, dtype=torch.bfloat16):
        q, s = quantize_int8_per_channel(linear.weight)
        return cls(q, s, None if linear.bias is None else linear.bias.detach().cpu(), dtype=dtype)

    def shard(self, rank, world, group=None):
        """Keeps only `rank`'s rows (output features); the forward gathers the full output (NCCL on "vk", gloo on CPU)."""
        out = Int8Linear(_shard.shard_rows(self.weight, rank, world), _shard.shard_rows(self.scales, rank, world),
                         None if self.bias is None else _shard.shard_rows(self.bias, rank, world), dtype=self.scales.dtype)
        out.rank, out.world, out._group, out.full_out_features = rank, world, group, self.out_features
        return out

    def forward(self, x, residual=None):
        """`residual`: a tensor of the output's shape added to it (x + proj(h) of a decoder block in one call)."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != self.scales.dtype:
            raise TypeError(f"Int8Linear holds {self.scales.dtype} scales; got {x2.dtype} activations")
        if x2.device.type == "vk" and self.world == 1 and (self.bias is not None or residual is not None):
            # one call for product, bias and residual (one launch when at most 32 rows are decoded); same roundings
            if residual is not None and residual.shape != (*lead, self.out_features):
                raise ValueError(f"residual of shape {tuple(residual.shape)} for an output of shape {(*lead, self.out_features)}")
            from . import _native
            r2 = None if residual is None else residual.reshape(-1, self.out_features)
            return _native.int8_linear(x2, self.weight, self.scales, self.bias, r2).reshape(*lead, self.out_features)
        y = torch._weight_int8pack_mm(x2, self.weight, self.scales)
        if self.bias is not None:
            y += self.bias
        return self._finish(y, lead, residual)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.full_out_features}, bias={self.bias is not None}, "
                f"dtype={self.scales.dtype}" + (f", rows {self.rank}/{self.world}" if self.world > 1 else ""))


class DynInt4Linear(nn.Module, _ShardedMixin):
    """y = dynamically quantised x @ int4 weights + bias through aten::_dyn_quant_matmul_4bit (float32 or bfloat16 x).

    Holds the tensor aten::_dyn_quant_pack_4bit_weight returns; on "vk" the tensor-core form of the weights is derived
    from it once and cached by the backend for as long as this tensor lives."""

    def __init__(self, packed, block_size, in_features, out_features):
        super().__init__()
        self.block_size, self.in_features, self.out_features = block_size, in_features, out_features
        self.full_out_features = out_features
        self.register_buffer("packed", packed)

    @classmethod
    def from_quantized(cls, nibbles, scales, bias, block_size, device=None):
        """nibbles uint8 [N, K/2], scales [N, K/block_size] (bfloat16 for blocks, float32 for one block per row),
        bias float32 [N] or None: the arguments of aten::_dyn_quant_pack_4bit_weight."""
        n, k = nibbles.shape[0], nibbles.shape[1] * 2
        if device is not None:
            nibbles, scales = nibbles.to(device), scales.to(device)
            bias = None if bias is None else bias.to(device)
        packed = torch._dyn_quant_pack_4bit_weight(nibbles, scales, bias, block_size, k, n)
        return cls(packed, block_size, k, n)

    @classmethod
    def from_float(cls, linear, block_size=32, device=None):
        k = linear.in_features
        nibbles, scales = quantize_int4_groupwise(linear.weight, block_size)
        scales = scales.to(torch.bfloat16) if block_size < k else scales.to(torch.float32)
        bias = None if linear.bias is None else linear.bias.detach().to(torch.float32).cpu()
        return cls.from_quantized(nibbles, scales, bias, block_size, device)

    def shard(self, rank, world, group=None):
        lo, hi = _shard.shard_bounds(self.out_features, rank, world)
        part = _shard.shard_packed_4bit(self.packed, self.block_size, self.in_features, self.out_features, rank, world)
        out = DynInt4Linear(part, self.block_size, self.in_features, hi - lo)
        out.rank, out.world, out._group, out.full_out_features = rank, world, group, self.out_features
        return out

    def forward(self, x, residual=None):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        y = torch._dyn_quant_matmul_4bit(x2, self.packed, self.block_size, self.in_features, self.out_features)
        return self._finish(y, lead, residual)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.full_out_features}, block_size={self.block_size}"
                + (f", rows {self.rank}/{self.world}" if self.world > 1 else ""))


def swap_linears(model, kind="int8", dtype=torch.bfloat16, block_size=32, device=None, skip=None):
    """Replaces every nn.Linear under `model` (in place) with its quantised counterpart, quantising on the CPU and moving
    the result to `device`. kind: "int8" (Int8Linear) or "dyn4" (DynInt4Linear). `skip(name, module)` keeps a layer as is.
    Returns the names of the layers it replaced."""
    if kind not in ("int8", "dyn4"):
        raise ValueError("kind must be 'int8' or 'dyn4'")
    replaced = []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if not isinstance(child, nn.Linear) or (skip is not None and skip(full, child)):
                continue
            if kind == "int8":
                new = Int8Linear.from_float(child, dtype=dtype)
                if device is not None:
                    new = new.to(device)
            else:
                new = DynInt4Linear.from_float(child, block_size=block_size, device=device)
            setattr(module, child_name, new)
            replaced.append(full)
    return replaced


def save(module, path):
    """Writes the quantised form of an Int8Linear / DynInt4Linear (CPU copies of its tensors and its geometry)."""
    if isinstance(module, Int8Linear):
        blob = {"kind": "int8", "weight": module.weight.cpu(), "scales": module.scales.cpu(),
                "bias": None if module.bias is None else module.bias.cpu()}
    elif isinstance(module, DynInt4Linear):
        blob = {"kind": "dyn4", "packed": module.packed.cpu(), "block_size": module.block_size,
                "in_features": module.in_features, "out_features": module.out_features}
    else:
        raise TypeError("save() takes an Int8Linear or a DynInt4Linear")
    torch.save(blob, path)


def load(path, device=None):
    """The module `save` wrote, on `device` (no quantisation and, for int4, no packing is repeated)."""
    blob = torch.load(path, map_location="cpu", weights_only=True)
    if blob["kind"] == "int8":
        out = Int8Linear(blob["weight"], blob["scales"], blob["bias"], dtype=blob["scales"].dtype)
    else:
        out = DynInt4Linear(blob["packed"], blob["block_size"], blob["in_features"], blob["out_features"])
    return out if device is None else out.to(device)

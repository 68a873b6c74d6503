"""torch_vulkan_b200: torch-vulkan's quantised matrix products on a B200, as device "vk".

    import torch, torch_vulkan_b200
    a = torch.randn(4, 8192).bfloat16().to("vk")
    y = torch._weight_int8pack_mm(a, w_int8.to("vk"), scales.to("vk"))
    print(y.cpu())

Importing this module registers a PyTorch backend on the PrivateUse1 key (C++, see
csrc/aten) and names it "vk", exactly as the reference's package does
(python/torch_vulkan/__init__.py:29-33), so code written for torch_vulkan's
`_weight_int8pack_mm`, `_dyn_quant_pack_4bit_weight`, `_dyn_quant_matmul_4bit` and
`_scaled_mm` runs unchanged. The kernels are hand-written CUDA for sm_100a behind the
C ABI of include/tvb200.h. Nothing else of PyTorch is implemented on this device and
nothing ever runs on the CPU instead: an op without a kernel raises NotImplementedError
(the reference's TORCH_VK_STRICT behaviour is the only mode).

The public functions mirror python/torch_vulkan/__init__.py:54-148.
"""

import atexit
import os
import sys
import types

import torch

__version__ = "0.1.0"

torch.utils.rename_privateuse1_backend("vk")

# `python -m torch_vulkan_b200._build` has to get past this file on a tree where nothing is built yet: that one command
# runs without the extension (and does nothing but build it).
_building = any(arg == "torch_vulkan_b200._build" for arg in getattr(sys, "orig_argv", []))
if _building:
    _native = None
else:
    try:
        from . import _native  # registers the C++ backend
    except ImportError as exc:  # no silent fallback: without the extension nothing works
        raise ImportError(
            "torch_vulkan_b200._native is not built (or libtvb200.so is missing): run "
            "`python -m torch_vulkan_b200._build`. There is no pure-Python or CPU path.") from exc

torch.utils.generate_methods_for_privateuse1_backend()

__all__ = ["device_count", "device_name", "empty_cache", "fallback_counts", "is_available", "memory_stats", "synchronize",
           "as_cuda", "from_cuda", "cuda_stream"]


def device_count():
    """Number of B200s the backend can use (the reference has one device)."""
    return _native.device_count()


def is_available():
    return device_count() > 0


def device_name(device=0):
    return _native.device_name(_index(device))


def _index(device):
    if device is None:
        return _current[0]  # (as the CUDA module: no device named means the current one)
    if isinstance(device, int):
        return device
    d = torch.device(device)
    return d.index or 0


def synchronize(device=None):
    """Waits for all queued GPU work on the device (the copy-out lane of copy_to_host_overlapped included)."""
    try:
        _native.synchronize(_index(device))
    finally:
        _copied_out.clear()


_copied_out = []  # sources of overlapped copies: kept alive (and out of the allocator's pool) until the next synchronize


def copy_to_host_overlapped(dst, src):
    """Copies the "vk" tensor `src` into the page-locked CPU tensor `dst` on the runtime's second stream: the copy starts
    when everything queued so far has run, and kernels queued afterwards run beside it (a step's results travel to the host
    under the step's remaining products). The bytes are in `dst` after synchronize(). Do not write to `src` before that.
    Inside a recorded step (shard.StepGraph) the recording holds the copy; return `src` from the step so that it lives
    as long as the recording. The reference has one queue per device (crates/vkcore/src/stream.rs): no counterpart."""
    from . import cabi

    if src.device.type != "vk" or dst.device.type != "cpu" or not dst.is_pinned():
        raise ValueError("copy_to_host_overlapped: from a \"vk\" tensor into a page-locked CPU tensor")
    if src.dtype != dst.dtype or src.shape != dst.shape or not src.is_contiguous() or not dst.is_contiguous():
        raise ValueError("copy_to_host_overlapped: contiguous tensors of one dtype and shape")
    idx = src.device.index or 0
    cabi.check(cabi.lib().tvb_memcpy_d2h_overlapped(idx, dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size()))
    _copied_out.append(src)
    return dst


def memory_stats(device=None):
    allocated, reserved, blocks = _native.memory_stats(_index(device))
    return {"allocated_bytes": allocated, "reserved_bytes": reserved, "blocks": blocks}


def empty_cache(device=None):
    """Returns cached, unused device memory to the driver."""
    _native.empty_cache(_index(device))


def fallback_counts():
    """{op: count} of aten ops that ran on the CPU instead of the GPU: always empty here."""
    return dict(_native.fallback_counts())


def dispatch_count():
    """Kernels launched so far."""
    return _native.dispatch_count()


def as_cuda(tensor):
    """A torch.cuda tensor sharing the memory of a "vk" tensor (for torch.distributed / NCCL)."""
    return _native.as_cuda(tensor)


def from_cuda(tensor):
    """A "vk" tensor sharing the memory of a torch.cuda tensor."""
    return _native.from_cuda(tensor)


def cuda_stream(device=None):
    """The stream the backend's kernels are queued on, as a torch.cuda stream (for events and NCCL ordering)."""
    idx = _index(device)
    return torch.cuda.ExternalStream(_native.stream(idx), device=torch.device("cuda", idx))


class _DeviceContext:
    """torch.vk.device(d): a context manager selecting device d."""

    def __init__(self, device):
        self.device = _index(device)
        self.prev = 0

    def __enter__(self):
        self.prev = _current[0]
        set_device(self.device)
        return self

    def __exit__(self, *exc):
        set_device(self.prev)
        return False


_current = [0]


def set_device(device):
    idx = _index(device)
    _native.set_device(idx)
    _current[0] = idx


def current_device():
    return _current[0]


def _device_module():
    # torch.vk: what PyTorch expects of a backend's device module (python/torch_vulkan/__init__.py:164-187).
    mod = types.ModuleType("torch.vk")
    mod.is_available = is_available
    mod.device_count = device_count
    mod.current_device = current_device
    mod.device = _DeviceContext
    mod.set_device = set_device
    mod.synchronize = synchronize
    mod.is_initialized = lambda: True
    mod._is_in_bad_fork = lambda: False
    mod.get_amp_supported_dtype = lambda: [torch.float32]
    mod._lazy_init = lambda: None
    mod.memory_stats = memory_stats
    mod.empty_cache = empty_cache
    mod.manual_seed_all = lambda seed: None  # (no random kernels on this device)
    mod.manual_seed = lambda seed: None
    return mod


torch._register_device_module("vk", _device_module())
sys.modules["torch.vk"] = torch.vk


@atexit.register
def _shutdown():
    # Finish queued work and release the pools before interpreter teardown.
    if _native is not None:
        _native.shutdown()

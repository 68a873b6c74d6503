"""CPU-side checks (no GPU): the C-ABI library loads and exports every symbol that
include/tvb200.h declares, fails loudly without a device, and the host logic of the
decode kernel's work split is consistent."""

import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tvb200.h")).read()
    return sorted(set(re.findall(r"TVB_API[^;]*?\b(tvb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from torch_vulkan_b200 import cabi

    lib = cabi.lib()
    names = declared_symbols()
    assert len(names) >= 27
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(cabi.SIGNATURES) == names  # the ctypes table covers the header, no more, no less


def test_no_device_means_errors_not_fallbacks():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from torch_vulkan_b200 import cabi

    lib = cabi.lib()
    assert lib.tvb_device_count() <= 0
    assert lib.tvb_synchronize(0) == -1 and lib.tvb_last_error()
    import torch_vulkan_b200 as tv

    assert not tv.is_available() and tv.fallback_counts() == {}
    with pytest.raises(RuntimeError):
        torch.zeros(3, device="vk")
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch._weight_int8pack_mm(torch.zeros(2, 16), torch.zeros(3, 16, dtype=torch.int8), torch.ones(3).to("vk"))


def test_argument_checks_match_the_cpu_kernels_messages():
    # the checks run before any device work, so they can be exercised here through the meta-free path:
    # tensors on the CPU reach the "vk" kernels only when one operand is on "vk", which needs a device;
    # what can be checked on the CPU is that PyTorch's own kernels raise the messages the tests expect.
    import torch

    with pytest.raises(RuntimeError, match="expect B to be int8 tensor"):
        torch._weight_int8pack_mm(torch.zeros(4, 16), torch.zeros(3, 16), torch.ones(3))
    with pytest.raises(RuntimeError, match="Group size should be multiple of 32"):
        torch._dyn_quant_pack_4bit_weight(torch.zeros(8, 32, dtype=torch.uint8), torch.ones(8, 2), None, 48, 64, 8)


def range_start(c, units, grid):
    return c * units // grid


def range_owner(x, units, grid):
    return ((x + 1) * grid + units - 1) // units - 1


@pytest.mark.parametrize("tiles,chunks,grid", [(112, 64, 148), (2, 32, 64), (14, 64, 148), (1, 1, 1), (3, 7, 5), (28, 64, 148),
                                               (17, 112, 148), (1, 8, 8)])
def test_decode_kernel_work_split(tiles, chunks, grid):
    """The (tile, chunk) units of qmm8_skinny_kernel are cut into `grid` contiguous ranges; the CTA that finishes a tile
    must find every contributor and its scratch slot from the same formulas the kernel uses (csrc/kernels/qmm8.cu)."""
    units = tiles * chunks
    grid = min(grid, units)
    starts = [range_start(c, units, grid) for c in range(grid + 1)]
    assert starts[0] == 0 and starts[-1] == units and all(b > a for a, b in zip(starts, starts[1:]))
    for x in range(units):
        c = range_owner(x, units, grid)
        assert starts[c] <= x < starts[c + 1]
    sizes = [b - a for a, b in zip(starts, starts[1:])]
    assert max(sizes) - min(sizes) <= 1  # every SM streams the same number of bytes, give or take one chunk
    for t in range(tiles):
        first, last = range_owner(t * chunks, units, grid), range_owner(t * chunks + chunks - 1, units, grid)
        slots = set()
        for c in range(first, last + 1):
            lo, hi = max(starts[c], t * chunks), min(starts[c + 1], (t + 1) * chunks)
            assert lo < hi  # every CTA in [first, last] contributes
            slot = 0 if starts[c] // chunks == t else 1
            # slot 0 is the CTA's first segment, slot 1 its last: a CTA never needs a third partial segment
            if slot == 1:
                assert (starts[c + 1] - 1) // chunks == t
            assert (c, slot) not in slots
            slots.add((c, slot))


def test_comm_entry_points_fail_cleanly_without_a_gpu():
    """The collective entry points: an id can be made wherever NCCL can be loaded; joining a communicator without a usable
    GPU returns -1 with a message instead of crashing (the multi-rank path itself is covered on GPUs and, for the host
    logic of assembling column slices, by the gloo ranks of test_shard.py)."""
    import ctypes

    import torch

    from torch_vulkan_b200 import cabi

    lib = cabi.lib()
    ident = ctypes.create_string_buffer(128)
    rc = lib.tvb_comm_unique_id(ident)
    assert rc in (0, -1)
    if rc == -1:
        assert b"NCCL" in lib.tvb_last_error()
    if not torch.cuda.is_available():
        handle = ctypes.c_void_p(0)
        assert lib.tvb_comm_init_rank(0, ident.raw, 1, 0, 100, ctypes.byref(handle)) == -1
        assert len(lib.tvb_last_error()) > 0
    assert lib.tvb_comm_abort(None) == 0 and lib.tvb_comm_destroy(None) == 0


def test_grouped_launch_and_host_registration_check_their_arguments():
    """What tvb_qmm8_group / tvb_qmm8_group_gather / tvb_host_register refuse before they touch a device."""
    import ctypes

    from torch_vulkan_b200 import cabi

    lib = cabi.lib()
    items = (cabi.TvbGroupItem * 5)()
    assert lib.tvb_qmm8_group(0, cabi.BF16, items, 0, 128, 128) == -1 and b"1 to 4 products" in lib.tvb_last_error()
    assert lib.tvb_qmm8_group(0, cabi.BF16, items, 5, 128, 128) == -1 and b"1 to 4 products" in lib.tvb_last_error()
    assert lib.tvb_qmm8_group(0, cabi.F32, items, 2, 128, 128) == -1 and b"float16 or bfloat16" in lib.tvb_last_error()
    assert lib.tvb_qmm8_group(0, cabi.BF16, None, 2, 128, 128) == -1
    flags = (ctypes.c_void_p * 2)(0, 0)
    assert lib.tvb_qmm8_group_gather(0, cabi.BF16, items, 2, flags, 9, 0, None, 0, 128, 128) == -1
    assert b"1 to 8 ranks" in lib.tvb_last_error()
    assert lib.tvb_qmm8_group_gather(0, cabi.BF16, items, 2, flags, 2, 0, None, 0, 128, 128) == -1
    assert b"NULL pointer" in lib.tvb_last_error()
    out = ctypes.c_void_p(0)
    assert lib.tvb_host_register(None, 4096, ctypes.byref(out)) == -1 and b"tvb_host_register" in lib.tvb_last_error()
    assert lib.tvb_host_unregister(None) == -1

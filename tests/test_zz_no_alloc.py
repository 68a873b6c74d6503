"""tvb_qmm8_static_scratch: the decode kernel for callers that must not allocate.

A host that gave all device memory to its own pool, or that bans driver allocations on its request path, cannot use
tvb_qmm8, whose scratch is allocated on first use. This entry point keeps that scratch in an array inside the library.
The test calls it through the C ABI twice in a row (the array is shared and keeps the previous call's contents, so the
second call proves the clearing) and compares with tvb_qmm8 on the same inputs, within the bound the other int8 tests
use. It is collected last, so a run that stops at the first failure has already run everything else, and it does not
depend on state left by other tests: it passes alone in a fresh process too."""

import ctypes

import pytest
import torch

import _cases as C

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(1, 1024, 3000), (16, 2048, 4099), (5, 8192, 777), (40, 512, 1000)])
def test_static_scratch_matches_allocating_entry_point(dtype, m, k, n):
    from torch_vulkan_b200 import cabi

    lib = cabi.lib()
    assert lib.tvb_device_count() >= 1
    a, b, s = C.config_int8(m, k, n, dtype, seed=m + n)
    want, tol = C.int8_want(a, b, s)
    da, db, ds = a.cuda(), b.cuda(), s.cuda()
    torch.cuda.synchronize()
    ref = cabi.qmm8(da, db, ds)
    cabi.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        torch.cuda.synchronize()
        rc = lib.tvb_qmm8_static_scratch(0, da.data_ptr(), cabi._dtype_code(dtype), da.stride(0), db.data_ptr(), ds.data_ptr(),
                                         out.data_ptr(), m, n, k, ctypes.c_void_p(stream))
        assert rc == 0, lib.tvb_last_error()
        torch.cuda.synchronize()
        assert ((out.cpu().float() - ref.cpu().float()).abs() <= tol).all(), f"call {call}: differs from tvb_qmm8"
        assert ((out.cpu().float() - want.float()).abs() <= tol).all(), f"call {call}: differs from the expected product"
        # how a bounded wait that ran out would surface: the call's status word, read back without any allocation
        word = ctypes.c_int(-1)
        assert lib.tvb_qmm8_static_scratch_status(0, ctypes.c_void_p(stream), ctypes.byref(word)) == 0, lib.tvb_last_error()
        assert word.value == 0


def test_static_scratch_rejects_what_it_cannot_hold():
    from torch_vulkan_b200 import cabi

    lib = cabi.lib()
    a, b, s = C.config_int8(2, 256, 64, torch.bfloat16)
    da, db, ds = a.cuda(), b.cuda(), s.cuda()
    out = torch.empty(2, 64, dtype=torch.bfloat16, device="cuda")
    args = (da.data_ptr(), cabi.BF16, da.stride(0), db.data_ptr(), ds.data_ptr(), out.data_ptr())
    # more output columns than the built-in scratch covers (nothing is launched: the sizes alone are checked)
    assert lib.tvb_qmm8_static_scratch(0, *args, 2, 4096 * 256 + 1, 256, None) == -1
    assert b"built-in scratch" in lib.tvb_last_error()
    assert lib.tvb_qmm8_static_scratch(0, *args, 65, 64, 256, None) == -1
    assert b"at most 64 rows" in lib.tvb_last_error()
    assert lib.tvb_qmm8_static_scratch(0, *args, 2, 64, 200, None) == -1  # k not a multiple of 128
    fa = a.float().cuda()
    assert lib.tvb_qmm8_static_scratch(0, fa.data_ptr(), cabi.F32, fa.stride(0), db.data_ptr(), ds.data_ptr(), out.data_ptr(),
                                       2, 64, 256, None) == -1

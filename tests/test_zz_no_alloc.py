"""The allocation-free batch-statistics entry point, called through its exported C
symbol, must agree with the regular entry points (which take caller-allocated
scratch) -- on two calls in a row, because every call reuses the same built-in
scratch array and has to clear it itself.

Callers that cannot allocate device memory (threads that must never trigger a
device-wide synchronisation, plugins living inside someone else's memory budget)
use this entry point; everything it needs beyond inputs and outputs is inside the
library.  The file name sorts last so a run that stops at the first failure has
already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from catch_b200.ops import capi

    lib = capi.lib()
    lib.b200_bn_batch_stats_noalloc.argtypes = [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_float, C.c_void_p,
                                                C.c_void_p, C.c_void_p]
    lib.b200_bn_batch_stats_noalloc.restype = C.c_int
    lib.b200_bn_stats.argtypes = [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p]
    lib.b200_bn_stats.restype = C.c_int
    lib.b200_bn_finalize.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.b200_bn_finalize.restype = C.c_int
    return lib, capi


def _existing(lib, capi, x, eps):
    rows, ch = x.shape
    sums = torch.zeros(2 * ch, dtype=torch.float64, device="cuda")  # caller-allocated scratch
    mean = torch.empty(ch, dtype=torch.float32, device="cuda")
    invstd = torch.empty(ch, dtype=torch.float32, device="cuda")
    capi.check(lib.b200_bn_stats(x.data_ptr(), capi.DT[x.dtype], rows, ch, sums.data_ptr(), None))
    capi.check(lib.b200_bn_finalize(sums.data_ptr(), rows, ch, eps, 0.0, mean.data_ptr(), invstd.data_ptr(), None, None,
                                    capi.DT[torch.float32], None))
    return mean, invstd


def test_noalloc_matches_existing_entry_point_twice():
    lib, capi = _lib()
    eps = 1e-5
    torch.manual_seed(0)
    # two different problems back to back: the second must not see the first one's sums
    for shape, dtype in (((70001, 256), torch.bfloat16), ((4099, 64), torch.float32)):
        x = (torch.randn(*shape, device="cuda") * 3 + 1.5).to(dtype)
        mean = torch.empty(shape[1], dtype=torch.float32, device="cuda")
        invstd = torch.empty(shape[1], dtype=torch.float32, device="cuda")
        rc = lib.b200_bn_batch_stats_noalloc(x.data_ptr(), capi.DT[dtype], shape[0], shape[1], eps, mean.data_ptr(),
                                             invstd.data_ptr(), None)
        assert rc == 0, capi.lib().b200_error_string(rc)
        ref_mean, ref_invstd = _existing(lib, capi, x, eps)
        torch.cuda.synchronize()
        assert torch.allclose(mean, ref_mean, rtol=1e-6, atol=1e-6)
        assert torch.allclose(invstd, ref_invstd, rtol=1e-6, atol=1e-6)
        # and both agree with plain PyTorch in fp32
        xf = x.float()
        assert torch.allclose(mean, xf.mean(0), rtol=3e-3, atol=3e-3)
        assert torch.allclose(invstd, (xf.var(0, unbiased=False) + eps).rsqrt(), rtol=3e-3, atol=3e-3)


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    lib, capi = _lib()
    ch = 4096 + 8
    x = torch.zeros(4, ch, device="cuda")
    out = torch.empty(ch, device="cuda")
    rc = lib.b200_bn_batch_stats_noalloc(x.data_ptr(), capi.DT[torch.float32], 4, ch, 1e-5, out.data_ptr(), out.data_ptr(), None)
    assert rc != 0
    torch.cuda.synchronize()

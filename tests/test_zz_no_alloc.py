"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory at the point where they need the kernel
(a recorded-and-replayed region, a callback of an application that owns the memory pool, a latency
path where the allocator would synchronise).  ``mm_rmsnorm_bwd_noalloc`` serves them by keeping the
kernel's fp32 workspace in a fixed array inside the library.  This test checks that it returns the
same dx / dw as the ordinary entry point (which takes the workspace from the caller) on two calls in a
row with different data - the second call reuses the array with the first call's contents still in it -
and that shapes beyond the fixed workspace are refused without launching anything.

Collected last on purpose (file name), so that a run stopping at the first failure has already run
every other test.  It passes alone in a fresh process as well as after the other tests.
"""
import ctypes as C

import pytest
import torch

from mindspeed_mm_b200.ops import build

pytestmark = pytest.mark.gpu


def _lib():
    lib = C.CDLL(build.lib_path())
    p, i = C.c_void_p, C.c_int
    lib.mm_rmsnorm_fwd.argtypes = [p, p, p, p, i, i, C.c_float, p]
    lib.mm_rmsnorm_bwd.argtypes = [p, p, p, p, p, p, p, i, i, p]
    lib.mm_rmsnorm_bwd_grid.argtypes = [i]
    lib.mm_rmsnorm_bwd_noalloc.argtypes = [p, p, p, p, p, p, i, i, p]
    lib.mm_noalloc_strerror.argtypes = [i]
    lib.mm_noalloc_strerror.restype = C.c_char_p
    return lib


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= atol + rtol * (b.abs().max().item() + 1e-6), err


def test_rmsnorm_bwd_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    st = torch.cuda.current_stream().cuda_stream
    for call, (T, H) in enumerate([(1000, 3584), (4097, 1280)]):
        torch.manual_seed(call)
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
        dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        y = torch.empty_like(x)
        rstd = torch.empty(T, device="cuda", dtype=torch.float32)
        assert lib.mm_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), T, H, 1e-6, st) == 0
        dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
        scratch = torch.empty(lib.mm_rmsnorm_bwd_grid(T) * H, device="cuda", dtype=torch.float32)
        assert lib.mm_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(),
                                  dw_ref.data_ptr(), scratch.data_ptr(), T, H, st) == 0
        dx, dw = torch.full_like(x, float("nan")), torch.full_like(w, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = lib.mm_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                        dw.data_ptr(), T, H, st)
        assert rc == 0, lib.mm_noalloc_strerror(rc)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        _close(dx, dx_ref, rtol=1e-3, atol=1e-3)      # same arithmetic per row
        _close(dw, dw_ref)                            # different number of partials -> fp32 order differs


def test_rmsnorm_bwd_noalloc_refuses_oversize():
    lib = _lib()
    z = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8, device="cuda", dtype=torch.float32)
    st = torch.cuda.current_stream().cuda_stream
    for T, H in [(4, 8192), (4, 4100), (0, 512)]:
        rc = lib.mm_rmsnorm_bwd_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), f.data_ptr(), z.data_ptr(),
                                        z.data_ptr(), T, H, st)
        assert rc == -20
        assert b"4096" in lib.mm_noalloc_strerror(rc)
    torch.cuda.synchronize()

"""The allocation-free RMSNorm backward (ulm_rmsnorm_bwd_static).

Some users of the library cannot hand it scratch memory: their allocator is
frozen after warm-up, or they are inside a stream capture, or they call from a
binding that has no device allocator.  For them the library carries its own
fixed scratch array.  This test calls that entry point through the C ABI twice in
a row and checks both results against the ordinary entry point, which gets its
scratch from the caller, and against the CPU oracle; it also checks the property
the entry point exists for -- the amount of free device memory and the framework
allocator's counters are the same after the call as before.  It lives in its own
file, collected last, and must pass both alone in a fresh process and after the
rest of the suite.
"""
import ctypes as C

import pytest
import torch

import _native as N
from oracle import ops

pytestmark = pytest.mark.gpu

DT = {torch.float16: N.ULM_F16, torch.bfloat16: N.ULM_BF16, torch.float32: N.ULM_F32}


def _args(x, w, dy, rstd, dx, dw, partial):
    return N.RmsBwdArgs(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr() if rstd is not None else None,
                        dx.data_ptr(), dw.data_ptr(), partial.data_ptr() if partial is not None else None,
                        x.stride(0), dy.stride(0), dx.stride(0), x.shape[0], x.shape[1],
                        DT[x.dtype], DT[w.dtype], 1e-6, C.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize('dtype,rows,d', [(torch.bfloat16, 4096, 768), (torch.float32, 333, 1024),
                                          (torch.float16, 5, 64)])
def test_static_scratch_matches_caller_scratch_twice(dtype, rows, d):
    lib = N.lib()
    assert torch.cuda.is_available()
    g = torch.Generator().manual_seed(rows + d)
    for call in range(2):                                 # second call reuses the array the first one dirtied
        x = torch.randn((rows, d), generator=g).to(dtype).cuda()
        dy = torch.randn((rows, d), generator=g).to(dtype).cuda()
        w = (1 + 0.02 * torch.randn((d,), generator=g)).cuda()
        ref_dx, ref_dw = torch.empty_like(x), torch.empty(d, device='cuda')
        parts = int(lib.ulm_rmsnorm_bwd_partial_rows(rows))
        partial = torch.empty((parts, d), device='cuda')
        N.check(lib.ulm_rmsnorm_bwd(C.byref(_args(x, w, dy, None, ref_dx, ref_dw, partial))), 'rmsnorm_bwd')
        got_dx, got_dw = torch.empty_like(x), torch.empty(d, device='cuda')
        args = _args(x, w, dy, None, got_dx, got_dw, None)
        if call == 0:
            # the very first call on a device looks up the array's address; do it before measuring
            N.check(lib.ulm_rmsnorm_bwd_static(C.byref(args)), 'rmsnorm_bwd_static')
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
        N.check(lib.ulm_rmsnorm_bwd_static(C.byref(args)), 'rmsnorm_bwd_static')
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        # nothing was allocated or freed by the call, by the library or through the framework
        assert free1 == free0
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (alloc0, reserved0)
        # same kernels, same reduction order: the tolerance of the RMSNorm tests, in practice equal
        torch.testing.assert_close(got_dx.float(), ref_dx.float(), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(got_dw, ref_dw, rtol=1e-5, atol=1e-5)
        # and against the CPU oracle, at the RMSNorm tests' tolerances
        edx, edw = ops.rms_norm_backward(x.cpu(), w.cpu(), dy.cpu())
        tol = 1e-5 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1e-2)
        torch.testing.assert_close(got_dx.cpu().float(), edx.float(), rtol=tol, atol=tol)
        assert float((got_dw.cpu().double() - edw.double()).norm() / edw.double().norm()) < 1e-5


def test_static_scratch_rejects_rows_wider_than_its_array():
    lib = N.lib()
    x = torch.zeros((4, 2048), dtype=torch.bfloat16, device='cuda')
    w = torch.ones(2048, device='cuda')
    dw = torch.empty(2048, device='cuda')
    rc = lib.ulm_rmsnorm_bwd_static(C.byref(_args(x, w, x, None, torch.empty_like(x), dw, None)))
    assert rc == -4
    assert b'exceeds the built-in scratch' in lib.ulm_last_error()


def test_static_scratch_refuses_tensors_of_another_device_than_the_current_one():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    lib = N.lib()
    with torch.cuda.device(1):
        x = torch.zeros((4, 64), dtype=torch.bfloat16, device='cuda:1')
        w = torch.ones(64, device='cuda:1')
        dw = torch.empty(64, device='cuda:1')
        args = _args(x, w, x, None, torch.empty_like(x), dw, None)
    with torch.cuda.device(0):
        assert lib.ulm_rmsnorm_bwd_static(C.byref(args)) == -1
        assert b'is current' in lib.ulm_last_error()

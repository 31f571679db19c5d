"""The allocation-free RMSNorm backward (`rb_rmsnorm_bwd_static`).

Some users of the library cannot allocate device memory at the point where they
need this gradient - their host framework owns the allocator, or allocation is
forbidden in the phase they run in - so they cannot hand the regular entry point
the scratch buffer it wants.  The static variant keeps that scratch inside the
library.  Here it is called the way such a user would: through the exported C
symbol, with raw pointers, and compared with the regular entry point on two
consecutive calls (the second call reuses whatever the first left in the
built-in scratch).  This file sorts last so that a run that stops at the first
failure has already run everything else.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "relax_b200", "_C.so")


def _lib():
    lib = ctypes.CDLL(SO)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.rb_rmsnorm_bwd_static.argtypes = [vp, vp, vp, vp, vp, i, i, f, i, vp]
    lib.rb_rmsnorm_bwd_static.restype = i
    lib.rb_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, i, i, f, i, vp]
    lib.rb_rmsnorm_bwd.restype = i
    lib.rb_rmsnorm_bwd_parts.argtypes = [i, i]
    lib.rb_rmsnorm_bwd_parts.restype = i
    return lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_static_entry_point_matches_regular_one_twice_in_a_row():
    lib = _lib()
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(123)
    for call, (rows, cols, dtype, code) in enumerate([(3000, 4096, torch.bfloat16, 0), (777, 1024, torch.float32, 2)]):
        x = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
        dy = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(dtype)
        # regular entry point: the caller supplies scratch
        dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
        scratch = torch.empty(lib.rb_rmsnorm_bwd_parts(rows, cols) * cols, dtype=torch.float32, device="cuda")
        rc = lib.rb_rmsnorm_bwd(_ptr(x), _ptr(w), _ptr(dy), _ptr(dx_ref), _ptr(dw_ref), _ptr(scratch), rows, cols, 1e-6,
                                code, stream)
        assert rc == 0
        # static entry point: inputs and outputs only
        dx, dw = torch.full_like(x, float("nan")), torch.full_like(w, float("nan"))
        rc = lib.rb_rmsnorm_bwd_static(_ptr(x), _ptr(w), _ptr(dy), _ptr(dx), _ptr(dw), rows, cols, 1e-6, code, stream)
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        assert torch.allclose(dx.float(), dx_ref.float(), atol=0.03, rtol=2e-2)
        assert torch.allclose(dw.float(), dw_ref.float(), atol=0.02 * rows ** 0.5, rtol=2e-2)
        # and both agree with a plain PyTorch fp32 statement of the op
        xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
        y.backward(dy.float())
        assert torch.allclose(dx.float(), xf.grad, atol=0.03, rtol=2e-2)
        assert torch.allclose(dw.float(), wf.grad, atol=0.02 * rows ** 0.5, rtol=2e-2)


def test_static_entry_point_refuses_oversized_problems():
    lib = _lib()
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.zeros(4, 16384, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(16384, device="cuda", dtype=torch.bfloat16)
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rc = lib.rb_rmsnorm_bwd_static(_ptr(x), _ptr(w), _ptr(x), _ptr(dx), _ptr(dw), 4, 16384, 1e-6, 0, stream)
    assert rc == -20          # RB_ERR_NOALLOC_TOO_LARGE: nothing launched
    torch.cuda.synchronize()

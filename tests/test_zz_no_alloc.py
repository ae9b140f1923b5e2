"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some hosts of the kernel library may not allocate device memory at call time (stream capture, fixed memory
budgets, allocator-free serving loops).  ``lmoe_rms_norm_bwd_noalloc`` keeps its scratch in a fixed array
inside the library; this test checks it against the regular entry point (scratch allocated by torch) on two
calls in a row, and checks that oversize problems are refused.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, fn_noalloc, rows, N, dtype, seed, with_w=True, with_dres=True):
    dev = torch.device("cuda", 0)
    torch.manual_seed(seed)
    x = torch.randn(rows, N, device=dev).to(dtype)
    dy = torch.randn(rows, N, device=dev).to(dtype)
    dres = torch.randn(rows, N, device=dev).to(dtype) if with_dres else None
    w = (1 + 0.1 * torch.randn(N, device=dev)).to(dtype) if with_w else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    code = 1 if dtype == torch.bfloat16 else 0
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    # regular entry point: caller-provided partials
    P = min(rows, 296)
    partial = torch.empty(P, N, dtype=torch.float32, device=dev) if with_w else None
    dx_ref = torch.empty_like(x)
    dw_ref = torch.empty(N, dtype=dtype, device=dev) if with_w else None
    rc = lib.lmoe_rms_norm_bwd(p(dy), p(x), p(w), p(rstd), p(dres), p(dx_ref), p(partial), p(dw_ref),
                               ctypes.c_int64(rows), ctypes.c_int(N), ctypes.c_int(P), ctypes.c_int(code), st)
    assert rc == 0
    # allocation-free entry point: inputs and outputs only
    dx = torch.empty_like(x)
    dw = torch.empty(N, dtype=dtype, device=dev) if with_w else None
    rc = fn_noalloc(p(dy), p(x), p(w), p(rstd), p(dres), p(dx), p(dw), ctypes.c_int64(rows), ctypes.c_int(N),
                    ctypes.c_int(code), st)
    assert rc == 0, lib.lmoe_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert torch.allclose(dx.float(), dx_ref.float(), rtol=3e-2, atol=3e-2)
    if with_w:
        assert torch.allclose(dw.float(), dw_ref.float(), rtol=3e-2, atol=3e-2 * max(1.0, rows ** 0.5))
    # and against the definition in fp32 PyTorch (relative Frobenius error), not only against the sibling entry point
    xf = x.float().requires_grad_(True)
    wf = None if w is None else w.float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    if wf is not None:
        y = y * wf
    y.backward(dy.float())
    dx_def = xf.grad + (dres.float() if with_dres else 0.0)
    rel = lambda a, b: ((a.float() - b).norm() / b.norm().clamp_min(1e-6)).item()
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-4
    assert rel(dx, dx_def) < tol, rel(dx, dx_def)
    if with_w:
        assert rel(dw, wf.grad) < tol, rel(dw, wf.grad)


def test_no_alloc_entry_point_matches_regular_one():
    from linear_moe_b200.ops import cuda as K
    lib = K.lib()
    fn = lib.lmoe_rms_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    lib.lmoe_noalloc_strerror.restype = ctypes.c_char_p
    # two calls in a row share the built-in scratch; the second must not see leftovers of the first
    _run(lib, fn, rows=1000, N=2048, dtype=torch.bfloat16, seed=0)
    _run(lib, fn, rows=77, N=1024, dtype=torch.float32, seed=1)
    # optional operands: no weight (no dw, the scratch is not touched) and no residual gradient
    _run(lib, fn, rows=300, N=512, dtype=torch.bfloat16, seed=2, with_w=False)
    _run(lib, fn, rows=300, N=512, dtype=torch.float32, seed=3, with_dres=False)
    # beyond the stated maximum: refused with a clear error, nothing launched
    z = ctypes.c_void_p(0)
    rc = fn(z, z, z, z, z, z, z, ctypes.c_int64(4), ctypes.c_int(8192), ctypes.c_int(1), z)
    assert rc == -100
    assert b"exceeds" in lib.lmoe_noalloc_strerror(rc)
    rc = fn(z, z, z, z, z, z, z, ctypes.c_int64(1 << 31), ctypes.c_int(1024), ctypes.c_int(1), z)
    assert rc == -100                                     # more rows than the kernels can index

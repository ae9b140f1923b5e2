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


def _run(lib, fn_noalloc, rows, N, dtype, seed):
    dev = torch.device("cuda", 0)
    torch.manual_seed(seed)
    x = torch.randn(rows, N, device=dev).to(dtype)
    dy = torch.randn(rows, N, device=dev).to(dtype)
    dres = torch.randn(rows, N, device=dev).to(dtype)
    w = (1 + 0.1 * torch.randn(N, device=dev)).to(dtype)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    code = 1 if dtype == torch.bfloat16 else 0
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    # regular entry point: caller-provided partials
    P = min(rows, 296)
    partial = torch.empty(P, N, dtype=torch.float32, device=dev)
    dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
    rc = lib.lmoe_rms_norm_bwd(p(dy), p(x), p(w), p(rstd), p(dres), p(dx_ref), p(partial), p(dw_ref),
                               ctypes.c_int64(rows), ctypes.c_int(N), ctypes.c_int(P), ctypes.c_int(code), st)
    assert rc == 0
    # allocation-free entry point: inputs and outputs only
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rc = fn_noalloc(p(dy), p(x), p(w), p(rstd), p(dres), p(dx), p(dw), ctypes.c_int64(rows), ctypes.c_int(N),
                    ctypes.c_int(code), st)
    assert rc == 0, lib.lmoe_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert torch.allclose(dx.float(), dx_ref.float(), rtol=3e-2, atol=3e-2)
    assert torch.allclose(dw.float(), dw_ref.float(), rtol=3e-2, atol=3e-2 * max(1.0, rows ** 0.5))


def test_no_alloc_entry_point_matches_regular_one():
    from linear_moe_b200.ops import cuda as K
    lib = K.lib()
    fn = lib.lmoe_rms_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    lib.lmoe_noalloc_strerror.restype = ctypes.c_char_p
    # two calls in a row share the built-in scratch; the second must not see leftovers of the first
    _run(lib, fn, rows=1000, N=2048, dtype=torch.bfloat16, seed=0)
    _run(lib, fn, rows=77, N=1024, dtype=torch.float32, seed=1)
    # beyond the stated maximum: refused with a clear error, nothing launched
    z = ctypes.c_void_p(0)
    rc = fn(z, z, z, z, z, z, z, ctypes.c_int64(4), ctypes.c_int(8192), ctypes.c_int(1), z)
    assert rc == -100
    assert b"exceeds" in lib.lmoe_noalloc_strerror(rc)

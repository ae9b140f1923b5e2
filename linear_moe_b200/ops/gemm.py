"""Binding of the tcgen05 / TMA / TMEM GEMM family (``csrc/gemm_tcgen05.cu``).

``gemm_nt(a, b)`` computes ``a @ b.T`` for bf16 ``a [M,K]``, ``b [N,K]`` with fp32 accumulation in tensor memory.
``gemm_nt_swiglu(a, w_tiled)`` fuses the SwiGLU activation into the epilogue; it expects the fc1 weight in the
*tiled* layout produced by :func:`tile_swiglu_weight` (per 256 rows: 128 gate rows then the matching 128 up rows).

The kernels report a bounded-wait expiry through an error word; :func:`check_error` raises if it is set.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_ENABLED = os.environ.get("LMOE_TCGEN05_GEMM", "1") != "0"
_ERR: Optional[torch.Tensor] = None


def available() -> bool:
    return _ENABLED and torch.cuda.is_available()


def enable(flag: bool):
    global _ENABLED
    _ENABLED = bool(flag)


def _err(device) -> torch.Tensor:
    global _ERR
    if _ERR is None or _ERR.device != device:
        _ERR = torch.zeros(1, dtype=torch.int32, device=device)
    return _ERR


def check_error():
    if _ERR is not None:
        v = int(_ERR.item())
        if v != 0:
            _ERR.zero_()
            raise RuntimeError(f"tcgen05 GEMM: bounded wait expired (code {v:#x})")


def _ok(t: torch.Tensor) -> bool:
    return (t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.shape[1] % 8 == 0 and t.data_ptr() % 16 == 0)


def supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    return available() and _ok(a) and _ok(b) and a.shape[1] == b.shape[1] and b.shape[0] % 8 == 0


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
    from . import cuda as K
    M, Kd = a.shape
    N = b.shape[0]
    No = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, No, dtype=torch.bfloat16, device=a.device)
    rc = K.lib().lmoe_gemm_bf16_nt(K._p(a), K._p(b), K._p(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(Kd),
                                   ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(out.stride(0)),
                                   ctypes.c_int(1 if swiglu else 0), K._p(_err(a.device)), ctypes.c_int(K.NUM_SMS), K._st())
    K._check(rc, "gemm_bf16_nt")
    return out


def tile_swiglu_weight(w: torch.Tensor) -> torch.Tensor:
    """``[2f, h]`` = [gate; up]  ->  per 128 output columns: 128 gate rows followed by the 128 up rows."""
    f = w.shape[0] // 2
    assert f % 128 == 0
    g, u = w[:f].reshape(f // 128, 128, -1), w[f:].reshape(f // 128, 128, -1)
    return torch.cat([g, u], dim=1).reshape(2 * f, -1).contiguous()


def supports_swiglu(x, w) -> bool:
    return False          # the model keeps fc1 in [gate; up] order; the tiled layout is opt-in


def supports_grouped(x, w1, w2) -> bool:
    return False

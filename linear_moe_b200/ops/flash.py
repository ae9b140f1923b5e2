"""Binding of the causal GQA flash-attention kernels (``csrc/flash_attn.cu``).

``FlashAttention.apply(q, k, v, scale, q_offset, window)`` takes ``q [B,Tq,Hq,D]`` and ``k/v [B,Tk,Hkv,D]`` in bf16
(unit stride along ``D``, token/head strides free so views into a fused QKV projection need no copy) and returns
``o [B,Tq,Hq,D]``.  Key ``j`` is visible to query ``i`` iff ``j <= q_offset + i`` (and ``j > q_offset + i - window``).
"""
from __future__ import annotations

import ctypes
import os

import torch

_ENABLED = os.environ.get("LMOE_FLASH_ATTN", "1") != "0"
_TCGEN05_FWD = os.environ.get("LMOE_FLASH_TCGEN05", "1") != "0"      # forward on tcgen05/TMEM (csrc/flash_attn_tc.cu)
_TCGEN05_BWD = os.environ.get("LMOE_FLASH_TCGEN05_BWD", "1") != "0"  # backward on tcgen05/TMEM (two kernels: dQ, dK/dV)


class _FaTcBwdArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("lse", "delta", "dq", "dk", "dv")] +
                [(n, ctypes.c_int) for n in ("B", "Tq", "Tk", "Hq", "Hkv", "q_offset", "window")] +
                [("scale", ctypes.c_float), ("err", ctypes.c_void_p)])


def _backward_tcgen05(q, k, v, out, d_out, lse, scale, q_offset, window):
    from . import cuda as K
    from . import gemm
    B, Tq, Hq, D = q.shape
    dq = torch.empty(B, Tq, Hq, D, dtype=q.dtype, device=q.device)
    dk = torch.empty(B, k.shape[1], k.shape[2], D, dtype=q.dtype, device=q.device)
    dv = torch.empty_like(dk)
    delta = torch.empty_like(lse)
    a = _FaTcBwdArgs()
    a.lse, a.delta, a.dq, a.dk, a.dv = lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.B, a.Tq, a.Hq, a.Tk, a.Hkv = B, Tq, Hq, k.shape[1], k.shape[2]
    a.q_offset, a.window, a.scale = int(q_offset), int(window or 0), float(scale)
    a.err = gemm._err(q.device).data_ptr()
    st = lambda t: (ctypes.c_longlong * 3)(t.stride(0), t.stride(1), t.stride(2))
    K._check(K.lib().lmoe_flash_attn_bwd_tc(K._p(q), st(q), K._p(k), st(k), K._p(v), st(v), K._p(out), K._p(d_out), K._p(delta),
                                            ctypes.byref(a), ctypes.c_int(D), K._st()), "flash_attn_bwd_tc", 3)
    return dq, dk, dv


class _FaTcArgs(ctypes.Structure):
    _fields_ = ([("out", ctypes.c_void_p), ("lse", ctypes.c_void_p)] +
                [(n, ctypes.c_int) for n in ("B", "Tq", "Tk", "Hq", "Hkv", "q_offset", "window")] +
                [("scale", ctypes.c_float), ("err", ctypes.c_void_p)])


def _forward_tcgen05(q, k, v, out, lse, scale, q_offset, window):
    from . import cuda as K
    from . import gemm
    a = _FaTcArgs()
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.B, a.Tq, a.Hq = q.shape[0], q.shape[1], q.shape[2]
    a.Tk, a.Hkv = k.shape[1], k.shape[2]
    a.q_offset, a.window, a.scale = int(q_offset), int(window or 0), float(scale)
    a.err = gemm._err(q.device).data_ptr()
    st = lambda t: (ctypes.c_longlong * 3)(t.stride(0), t.stride(1), t.stride(2))
    K._check(K.lib().lmoe_flash_attn_fwd_tc(K._p(q), st(q), K._p(k), st(k), K._p(v), st(v), ctypes.byref(a),
                                            ctypes.c_int(q.shape[-1]), K._st()), "flash_attn_fwd_tc")


class _FaArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("q", "k", "v", "o", "d_o")] +
                [(n, ctypes.c_int64) for n in ("qs_b", "qs_t", "qs_h", "ks_b", "ks_t", "ks_h", "vs_b", "vs_t", "vs_h")] +
                [(n, ctypes.c_void_p) for n in ("out", "lse", "delta", "dq_acc", "dk", "dv")] +
                [(n, ctypes.c_int) for n in ("B", "Tq", "Tk", "Hq", "Hkv", "q_offset", "window")] +
                [("scale", ctypes.c_float)])


def _view_ok(t: torch.Tensor) -> bool:
    return (t.dim() == 4 and t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0)


def supported(q, k, v, causal, window) -> bool:
    if not (_ENABLED and q.is_cuda and causal):
        return False
    D = q.shape[-1]
    return (q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and D in (64, 128) and k.shape[-1] == D and v.shape[-1] == D
            and q.shape[2] % k.shape[2] == 0 and k.shape[2] == v.shape[2] and k.shape[1] == v.shape[1])


def _args(q, k, v, scale, q_offset, window) -> _FaArgs:
    a = _FaArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.qs_b, a.qs_t, a.qs_h = q.stride(0), q.stride(1), q.stride(2)
    a.ks_b, a.ks_t, a.ks_h = k.stride(0), k.stride(1), k.stride(2)
    a.vs_b, a.vs_t, a.vs_h = v.stride(0), v.stride(1), v.stride(2)
    a.B, a.Tq, a.Hq = q.shape[0], q.shape[1], q.shape[2]
    a.Tk, a.Hkv = k.shape[1], k.shape[2]
    a.q_offset, a.window, a.scale = int(q_offset), int(window or 0), float(scale)
    return a


def _fix(t: torch.Tensor) -> torch.Tensor:
    return t if _view_ok(t) else t.contiguous()


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, q_offset, window=None):
        from . import cuda as K
        q, k, v = _fix(q), _fix(k), _fix(v)
        B, Tq, Hq, D = q.shape
        out = torch.empty(B, Tq, Hq, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(B, Hq, Tq, dtype=torch.float32, device=q.device)
        if _TCGEN05_FWD:
            _forward_tcgen05(q, k, v, out, lse, scale, q_offset, window)
        else:
            a = _args(q, k, v, scale, q_offset, window)
            a.out, a.lse = out.data_ptr(), lse.data_ptr()
            K._check(K.lib().lmoe_flash_attn_fwd(ctypes.byref(a), ctypes.c_int(D), K._st()), "flash_attn_fwd")
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (scale, q_offset, window)
        return out

    @staticmethod
    def backward(ctx, d_out):
        from . import cuda as K
        q, k, v, out, lse = ctx.saved_tensors
        scale, q_offset, window = ctx.cfg
        B, Tq, Hq, D = q.shape
        d_out = d_out.contiguous()
        if _TCGEN05_BWD:
            dq, dk, dv = _backward_tcgen05(q, k, v, out, d_out, lse, scale, q_offset, window)
            return dq, dk, dv, None, None, None
        delta = torch.empty_like(lse)
        dq_acc = torch.zeros(B, Tq, Hq, D, dtype=torch.float32, device=q.device)
        dk = torch.empty(B, k.shape[1], k.shape[2], D, dtype=q.dtype, device=q.device)
        dv = torch.empty_like(dk)
        a = _args(q, k, v, scale, q_offset, window)
        a.o, a.d_o, a.lse, a.delta = out.data_ptr(), d_out.data_ptr(), lse.data_ptr(), delta.data_ptr()
        a.dq_acc, a.dk, a.dv = dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr()
        K._check(K.lib().lmoe_flash_attn_bwd(ctypes.byref(a), ctypes.c_int(D), K._st()), "flash_attn_bwd", 2)
        return dq_acc.to(q.dtype), dk, dv, None, None, None

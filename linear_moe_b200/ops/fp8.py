"""fp8 (e4m3) linear layers on the tcgen05 fp8 GEMM (``csrc/gemm_fp8.cu``).

Every GEMM of a linear layer is brought to the form ``diag(sa) (A8 B8^T) diag(sb)`` by quantising both operands along
the contracted dimension with one fp32 scale per row (token, output channel, ...), from the current tensor's amax:

    forward  y  = x W^T      A = rows(x)       B = rows(W)
    dgrad    dx = dy W       A = rows(dy)      B = rows(W^T)
    wgrad    dW = dy^T x     A = rows(dy^T)    B = rows(x^T)

``set_enabled(True)`` (done by the model builder when ``ModelConfig.fp8`` is set) routes ``ops.linear`` of the
projection layers through :class:`Fp8Linear`; the LM head, the router and the norms stay in bf16/fp32, as they do
under the reference's TransformerEngine fp8 autocast (hybrid_transformer_block.py:355-377).
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

_ENABLED = False


def set_enabled(flag: bool):
    global _ENABLED
    _ENABLED = bool(flag)


def enabled() -> bool:
    return _ENABLED


def supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    M = x.numel() // x.shape[-1]
    N, Kd = weight.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2
            and M % 16 == 0 and N % 16 == 0 and Kd % 16 == 0 and M >= 128)


def quant_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[R, C]`` (unit stride along C) -> (e4m3 bytes ``[R, C]``, fp32 scale ``[R]``)."""
    from . import cuda as K
    R, C = x.shape
    assert x.stride(1) == 1
    q = torch.empty(R, C, dtype=torch.uint8, device=x.device)
    s = torch.empty(R, dtype=torch.float32, device=x.device)
    K._check(K.lib().lmoe_fp8_quant_rows(K._p(x), ctypes.c_longlong(x.stride(0)), K._p(q), K._p(s), ctypes.c_int(R),
                                         ctypes.c_int(C), K._st()), "fp8_quant_rows")
    return q, s


def quant_cols_t(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[R, C]`` -> (e4m3 bytes of the transpose ``[C, R]``, fp32 scale ``[C]``): rows of ``x^T``."""
    from . import cuda as K
    R, C = x.shape
    assert x.stride(1) == 1
    q = torch.empty(C, R, dtype=torch.uint8, device=x.device)
    s = torch.empty(C, dtype=torch.float32, device=x.device)
    scratch = torch.empty(C, dtype=torch.int32, device=x.device)
    K._check(K.lib().lmoe_fp8_quant_cols_t(K._p(x), ctypes.c_longlong(x.stride(0)), K._p(q), K._p(s), K._p(scratch),
                                           ctypes.c_int(R), ctypes.c_int(C), K._st()), "fp8_quant_cols_t", 2)
    return q, s


def gemm_nt(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor, pairs: bool = True) -> torch.Tensor:
    """``diag(sa) (a8 [M,K] @ b8 [N,K]^T) diag(sb)`` -> bf16 ``[M, N]``.  ``pairs`` selects the CTA-pair kernel
    (``tcgen05.mma.cta_group::2``, ``csrc/gemm_2cta.cu``), which halves the shared-memory traffic per SM."""
    from . import cuda as K
    from . import gemm
    M, Kd = a8.shape
    N = b8.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a8.device)
    if pairs:
        K._check(K.lib().lmoe_gemm_fp8_nt_2cta(K._p(a8), K._p(b8), K._p(out), K._p(sa), K._p(sb), ctypes.c_int(M), ctypes.c_int(N),
                                               ctypes.c_int(Kd), ctypes.c_int(N), K._p(gemm._err(a8.device)),
                                               ctypes.c_int(K.NUM_SMS), K._st()), "gemm_fp8_nt_2cta")
        return out
    K._check(K.lib().lmoe_gemm_fp8_nt(K._p(a8), K._p(b8), K._p(out), K._p(sa), K._p(sb), ctypes.c_int(M), ctypes.c_int(N),
                                      ctypes.c_int(Kd), ctypes.c_int(N), K._p(gemm._err(a8.device)), ctypes.c_int(K.NUM_SMS),
                                      K._st()), "gemm_fp8_nt")
    return out


def dequant_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    return q.view(torch.float8_e4m3fn).float() * s[:, None]


class Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.stride(1) == 1 else x2.contiguous()
        xq, sx = quant_rows(x2)
        wq, sw = quant_rows(weight)
        y = gemm_nt(xq, sx, wq, sw)
        ctx.save_for_backward(x2, weight)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import cuda as K
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dq, sd = quant_rows(dy2)
            wtq, swt = quant_cols_t(weight)                         # rows of W^T [K, N]
            dx = gemm_nt(dq, sd, wtq, swt).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            dtq, sdt = quant_cols_t(dy2)                            # rows of dy^T [N, M]
            xtq, sxt = quant_cols_t(x2)                             # rows of x^T  [K, M]
            dw = gemm_nt(dtq, sdt, xtq, sxt)
            mg = getattr(weight, "main_grad", None)
            if mg is not None and mg.dtype == torch.float32 and mg.is_cuda:
                if getattr(weight, "_main_grad_fresh", False):
                    mg.copy_(dw)
                    weight._main_grad_fresh = False
                else:
                    K.accumulate_grad(mg, dw)
                dw = None
        return dx, dw

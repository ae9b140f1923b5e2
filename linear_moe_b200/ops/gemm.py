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


_CUDA_OK: Optional[bool] = None


def available() -> bool:
    global _CUDA_OK
    if _CUDA_OK is None:
        _CUDA_OK = torch.cuda.is_available()          # asked on every linear: cache the answer
    return _ENABLED and _CUDA_OK


def enable(flag: bool):
    global _ENABLED
    _ENABLED = bool(flag)


def _err(device) -> torch.Tensor:
    """Error word of the tcgen05 kernels: element 1 of the fused-communication status tensor, so the training loop
    reads both with one copy (``fused_comm.check_status``)."""
    global _ERR
    if _ERR is None or _ERR.device != device:
        from ..parallel import fused_comm
        _ERR = fused_comm.status_word(device)[1:2]
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


def gemm_nt_2cta(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a @ b.T`` on CTA pairs (``tcgen05.mma.cta_group::2``, 256 x 256 tile per pair; ``csrc/gemm_2cta.cu``)."""
    from . import cuda as K
    M, Kd = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    rc = K.lib().lmoe_gemm_bf16_nt_2cta(K._p(a), K._p(b), K._p(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(Kd),
                                        ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(out.stride(0)),
                                        K._p(_err(a.device)), ctypes.c_int(K.NUM_SMS), K._st())
    K._check(rc, "gemm_bf16_nt_2cta")
    return out


def dense_ok(*ts: torch.Tensor) -> bool:
    """Every 2-D bf16 operand fits the TMA rules of the dense kernel (unit inner stride, 16-byte pitches and base)."""
    if not available():
        return False
    for t in ts:
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
                and t.shape[1] % 8 == 0 and t.data_ptr() % 16 == 0 and t.shape[0] > 0):
            return False
    return True


BAND = int(os.environ.get("LMOE_GEMM_BAND", "0"))          # tile rows per band of the tile order (0 = kernel default)


def dense(a: torch.Tensor, b: torch.Tensor, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
          accumulate: bool = False, out_dtype=torch.bfloat16, band: Optional[int] = None,
          bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C[M,N] (+)= A B`` on the CTA-pair tcgen05 kernel of ``csrc/gemm_dense.cu`` (``bias`` ``[N]`` bf16: added in the
    epilogue of the bf16-output form).

    ``a`` is ``[M,K]`` (or ``[K,M]`` with ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]`` with ``b_mn``).  ``out`` may be a
    bf16 or fp32 matrix; ``accumulate`` (fp32 only) adds into it with TMA reduce-adds instead of overwriting.
    The three GEMMs of a linear layer are ``dense(x, w)`` (forward), ``dense(dy, w, b_mn=True)`` (data gradient) and
    ``dense(dy, x, a_mn=True, b_mn=True)`` (weight gradient)."""
    from . import cuda as K
    M, Kd = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    assert (b.shape[0] if b_mn else b.shape[1]) == Kd, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    mode = 0 if out.dtype == torch.bfloat16 else (2 if accumulate else 1)
    assert out.shape == (M, N) and out.stride(1) == 1 and (mode != 0 or not accumulate)
    if bias is not None:
        assert mode == 0 and bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
        rc = K.lib().lmoe_gemm_dense_bias(K._p(a), ctypes.c_int(a.stride(0)), ctypes.c_int(int(a_mn)), K._p(b),
                                          ctypes.c_int(b.stride(0)), ctypes.c_int(int(b_mn)), K._p(out), ctypes.c_int(out.stride(0)),
                                          K._p(bias), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(Kd),
                                          ctypes.c_int(BAND if band is None else band), K._p(_err(a.device)),
                                          ctypes.c_int(K.NUM_SMS), K._st())
        K._check(rc, "gemm_dense_bias")
        return out
    rc = K.lib().lmoe_gemm_dense(K._p(a), ctypes.c_int(a.stride(0)), ctypes.c_int(int(a_mn)), K._p(b), ctypes.c_int(b.stride(0)),
                                 ctypes.c_int(int(b_mn)), K._p(out), ctypes.c_int(out.stride(0)), ctypes.c_int(mode),
                                 ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(Kd), ctypes.c_int(BAND if band is None else band),
                                 K._p(_err(a.device)), ctypes.c_int(K.NUM_SMS), K._st())
    K._check(rc, "gemm_dense")
    return out


def dense_swiglu(x: torch.Tensor, w: torch.Tensor, want_pre: bool = True, band: Optional[int] = None, out_shape=None):
    """``silu(x Wg^T) * (x Wu^T)`` for ``w = [Wg ; Wu]`` (``[2F, K]``, the ordinary fc1 layout) with the activation in
    the GEMM epilogue.  Returns ``(act [M,F], pre [M,2F] or None)``; ``pre`` is what the backward pass needs."""
    from . import cuda as K
    M, Kd = x.shape
    F2 = w.shape[0]
    Fh = F2 // 2
    act = torch.empty(out_shape or (M, Fh), dtype=torch.bfloat16, device=x.device)
    pre = torch.empty(M, F2, dtype=torch.bfloat16, device=x.device) if want_pre else None
    rc = K.lib().lmoe_gemm_dense_swiglu(K._p(x), ctypes.c_int(x.stride(0)), K._p(w), ctypes.c_int(w.stride(0)), K._p(act),
                                        ctypes.c_int(Fh), K._p(pre), ctypes.c_int(F2), ctypes.c_int(M),
                                        ctypes.c_int(Fh), ctypes.c_int(Kd), ctypes.c_int(BAND if band is None else band),
                                        K._p(_err(x.device)), ctypes.c_int(K.NUM_SMS), K._st())
    K._check(rc, "gemm_dense_swiglu")
    return act, pre


def dense_dswiglu(dy: torch.Tensor, w2: torch.Tensor, pre: torch.Tensor, band: Optional[int] = None) -> torch.Tensor:
    """``dPre = SwiGLU'(pre) applied to (dy @ w2)`` for ``w2 [H, F]`` (the fc2 weight as stored) and ``pre [M, 2F]``: the
    data-gradient GEMM of fc2 with the activation backward in its epilogue.  ``F`` must be a multiple of 64."""
    from . import cuda as K
    M, H = dy.shape
    Fh = w2.shape[1]
    dpre = torch.empty(M, 2 * Fh, dtype=torch.bfloat16, device=dy.device)
    rc = K.lib().lmoe_gemm_dense_dswiglu(K._p(dy), ctypes.c_int(dy.stride(0)), K._p(w2), ctypes.c_int(w2.stride(0)), K._p(pre),
                                         ctypes.c_int(pre.stride(0)), K._p(dpre), ctypes.c_int(2 * Fh), ctypes.c_int(M),
                                         ctypes.c_int(Fh), ctypes.c_int(H), ctypes.c_int(BAND if band is None else band),
                                         K._p(_err(dy.device)), ctypes.c_int(K.NUM_SMS), K._st())
    K._check(rc, "gemm_dense_dswiglu")
    return dpre


def tile_swiglu_weight(w: torch.Tensor) -> torch.Tensor:
    """``[2f, h]`` = [gate; up]  ->  per 128 output columns: 128 gate rows followed by the 128 up rows."""
    f = w.shape[0] // 2
    assert f % 128 == 0
    g, u = w[:f].reshape(f // 128, 128, -1), w[f:].reshape(f // 128, 128, -1)
    return torch.cat([g, u], dim=1).reshape(2 * f, -1).contiguous()


# ---------------------------------------------------------------------------------------------
# grouped / layout-general GEMMs (csrc/gemm_grouped.cu)
# ---------------------------------------------------------------------------------------------
PAIRS = os.environ.get("LMOE_GEMM_PAIRS", "1") != "0"     # CTA-pair (cta_group::2) kernels for the grouped GEMMs
ROW_ALIGN = 256 if PAIRS else 128                          # expert segments are padded to whole pair tiles


def _gg(A, a_mn, B, b_mn, C, mode, M, N, Kd, groups, offs, c_stride, pairs=None, accumulate=False):
    from . import cuda as K
    pairs = PAIRS if pairs is None else pairs
    rc = K.lib().lmoe_gemm_grouped(
        K._p(A), ctypes.c_int(A.shape[0]), ctypes.c_int(A.shape[1]), ctypes.c_int(A.stride(0)), ctypes.c_int(int(a_mn)),
        K._p(B), ctypes.c_int(B.shape[0]), ctypes.c_int(B.shape[1]), ctypes.c_int(B.stride(0)), ctypes.c_int(int(b_mn)),
        K._p(C), ctypes.c_int(C.stride(-2)), ctypes.c_int(mode), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(Kd),
        ctypes.c_int(groups), K._p(offs), ctypes.c_longlong(c_stride), K._p(_err(A.device)), ctypes.c_int(K.NUM_SMS),
        ctypes.c_int(int(pairs)), ctypes.c_int(int(C.dtype == torch.float32)), ctypes.c_int(int(accumulate)), K._st())
    K._check(rc, "gemm_grouped")
    return C


def gemm_general(a: torch.Tensor, b: torch.Tensor, a_mn: bool = False, b_mn: bool = False, pairs=None) -> torch.Tensor:
    """Dense ``C[M,N]``.  ``a`` is ``[M,K]`` (or ``[K,M]`` if ``a_mn``); ``b`` is ``[N,K]`` (or ``[K,N]`` if ``b_mn``)."""
    M, Kd = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    C = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    return _gg(a, a_mn, b, b_mn, C, 0, M, N, Kd, 0, None, 0, pairs)


def padded_offsets(counts: torch.Tensor, align: int = 0) -> torch.Tensor:
    """Per-expert token counts -> int32 row offsets ``[E+1]`` with every segment padded to ``align`` rows (device op);
    the default is the tile height of the grouped kernels in use (:data:`ROW_ALIGN`)."""
    align = align or ROW_ALIGN
    padded = (counts + align - 1) // align * align
    offs = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    offs[1:] = torch.cumsum(padded, 0).to(torch.int32)
    return offs


class GroupedLinear(torch.autograd.Function):
    """``y[rows of expert e] = x[rows of expert e] @ w[e]`` for ``w [E, K, N]`` over a padded expert-sorted buffer.
    Forward, dgrad and wgrad are three launches of the grouped tcgen05 kernel; the expert offsets never leave the device.
    Every offset must be a multiple of :data:`ROW_ALIGN`."""

    @staticmethod
    def forward(ctx, x, w, offs, out=None, dx_out=None):
        """``out`` / ``dx_out``: holders (objects with a ``buf`` tensor ``[rows, N]`` / ``[rows, K]``, not tensors, so that
        autograd does not track the workspace) into which the result / the input gradient is written instead of a fresh
        tensor: the expert-parallel exchange lets the GEMM write straight into the buffer its peers read."""
        E, Kd, N = w.shape
        y = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device) if out is None else out.buf[: x.shape[0]]
        assert y.shape == (x.shape[0], N) and y.is_contiguous()
        _gg(x, False, w.view(E * Kd, N), True, y, 1, 0, N, Kd, E, offs, 0)
        ctx.save_for_backward(x, w, offs)
        ctx.dx_out = dx_out
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, offs = ctx.saved_tensors
        E, Kd, N = w.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x) if ctx.dx_out is None else ctx.dx_out.buf[: x.shape[0]]
        assert dx.shape == x.shape and dx.is_contiguous()
        _gg(dy, False, w.view(E * Kd, N), False, dx, 1, 0, Kd, N, E, offs, 0)              # dy @ w[e]^T
        mg = getattr(w, "main_grad", None)
        if PAIRS and mg is not None and mg.dtype == torch.float32 and mg.is_contiguous() and mg.shape == w.shape:
            # weight gradient straight into the fp32 accumulator (first write after zero_grad overwrites, later ones add)
            fresh = getattr(w, "_main_grad_fresh", False)
            _gg(x, True, dy, True, mg, 2, Kd, N, 0, E, offs, Kd * N, accumulate=not fresh)
            w._main_grad_fresh = False
            w._direct_wgrad = True
            return dx, None, None, None, None
        dw = torch.empty_like(w)
        _gg(x, True, dy, True, dw, 2, Kd, N, 0, E, offs, Kd * N)                           # x_e^T @ dy_e
        return dx, dw, None, None, None


def supports_grouped(x, w1, w2) -> bool:
    h, f2 = w1.shape[1], w1.shape[2]
    return (available() and x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16
            and h % 8 == 0 and f2 % 16 == 0 and x.is_contiguous())


def grouped_mlp(x_sorted: torch.Tensor, tokens_per_expert: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """Expert-sorted tokens ``[T, h]`` through per-expert SwiGLU MLPs (``w1 [E,h,2f]``, ``w2 [E,f,h]``).  Tokens are
    scattered into a 128-row-padded buffer (index arithmetic on the device only), run through two grouped GEMMs with the
    SwiGLU kernel in between, and gathered back."""
    from . import cuda as K
    E = w1.shape[0]
    T, h = x_sorted.shape
    counts = tokens_per_expert.to(torch.int64)
    offs = padded_offsets(counts)
    start = torch.cumsum(counts, 0) - counts                                   # unpadded start of each expert
    eid = torch.repeat_interleave(torch.arange(E, device=x_sorted.device), counts, output_size=T)
    dest = offs[:-1].to(torch.int64)[eid] + (torch.arange(T, device=x_sorted.device) - start[eid])
    Tp = (T + E * (ROW_ALIGN - 1) + ROW_ALIGN - 1) // ROW_ALIGN * ROW_ALIGN
    xp = torch.zeros(Tp, h, dtype=x_sorted.dtype, device=x_sorted.device).index_copy(0, dest, x_sorted)
    y1 = GroupedLinear.apply(xp, w1, offs)
    act = K.swiglu(y1)
    y2 = GroupedLinear.apply(act, w2, offs)
    return y2.index_select(0, dest)

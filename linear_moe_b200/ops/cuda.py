"""CUDA back end of :mod:`linear_moe_b200.ops`: ctypes bindings of ``lib/liblmoe.so`` wrapped in
``torch.autograd.Function``s.

The library is plain C ABI (no torch headers): every entry point takes raw device pointers, sizes and
the CUDA stream, so a call costs one ctypes dispatch and launches on torch's current stream.  A missing
library is an error on a machine with a GPU (no silent fallback to eager).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ..ref import ops as R
from . import lsm_torch as LT

_LIB: Optional[ctypes.CDLL] = None
_NUM_SMS = None


def num_sms() -> int:
    """SM count of the current device (148 on a B200); persistent kernels size their grids from it."""
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                    if torch.cuda.is_available() else 148)
    return _NUM_SMS


def __getattr__(name):                       # ``K.NUM_SMS`` for the callers in other modules
    if name == "NUM_SMS":
        return num_sms()
    raise AttributeError(name)
launch_count = 0          # kernels of this library launched since the last reset (bench.py reports it)


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "liblmoe.so")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        p = lib_path()
        if not os.path.exists(p):
            raise RuntimeError(f"{p} is missing: run `python -m linear_moe_b200.build` (nvcc, sm_100a) first")
        _LIB = ctypes.CDLL(p)
    return _LIB


def reset_launch_count() -> int:
    global launch_count
    n, launch_count = launch_count, 0
    return n


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _st():
    """The current CUDA stream as the launchers take it.  ``torch.cuda.current_stream()`` builds a Python stream object
    through several layers of device-index checks (~15 us, once per kernel launch); the raw query is a single C call."""
    if _RAW_STREAM is not None:
        return ctypes.c_void_p(_RAW_STREAM(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError(f"unsupported dtype {t.dtype} (bf16 and fp32 kernels only)")


def _check(rc: int, name: str, n: int = 1):
    global launch_count
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    launch_count += n


_i64, _i32, _f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_float


def _same_dtype(x, *ts):
    return [None if t is None else (t if t.dtype == x.dtype else t.to(x.dtype)) for t in ts]


# =====================================================================================
# GEMM-shaped: every dense linear runs the CTA-pair tcgen05 kernel of csrc/gemm_dense.cu
# =====================================================================================
def _rows(t: torch.Tensor) -> torch.Tensor:
    """``[..., n]`` -> a 2-D view (or copy) that satisfies the TMA rules of the dense kernel."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def wgrad_into_main_grad(weight, dy2: torch.Tensor, x2: torch.Tensor) -> bool:
    """``weight.main_grad (+)= dy2^T x2`` straight from the GEMM epilogue in fp32 (TMA store for the first write after
    ``zero_grad``, TMA reduce-add afterwards), skipping the bf16 gradient tensor and the separate accumulation pass
    (the counterpart of Megatron's gradient-accumulation fusion).  Returns False when the parameter has no fp32
    accumulator or the operands do not fit the kernel."""
    from . import gemm
    mg = getattr(weight, "main_grad", None)
    if os.environ.get("LMOE_DIRECT_WGRAD", "1") == "0":
        return False
    if mg is None or mg.dtype != torch.float32 or not mg.is_contiguous() or not gemm.dense_ok(dy2, x2):
        return False
    fresh = getattr(weight, "_main_grad_fresh", False)
    gemm.dense(dy2, x2, a_mn=True, b_mn=True, out=mg.view(dy2.shape[1], x2.shape[1]), accumulate=not fresh)
    weight._main_grad_fresh = False
    weight._direct_wgrad = True            # the optimizer may skip clearing this accumulator (first write overwrites)
    return True


def mm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a [M,K] @ b [N,K]^T`` (dense tcgen05 kernel for bf16 operands that fit it, library GEMM otherwise)."""
    from . import gemm
    if gemm.dense_ok(a, b) and b.shape[0] % 8 == 0:
        return gemm.dense(a, b)
    return torch.mm(a, b.t())


def mm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a [M,N] @ b [N,K]``."""
    from . import gemm
    if gemm.dense_ok(a, b):
        return gemm.dense(a, b, b_mn=True)
    return torch.mm(a, b)


def mm_tn(a: torch.Tensor, b: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """``a [M,N]^T @ b [M,K]`` -> ``[N,K]`` in ``out_dtype`` (bf16 or fp32 straight from the fp32 accumulators)."""
    from . import gemm
    out_dtype = out_dtype or a.dtype
    if gemm.dense_ok(a, b) and out_dtype in (torch.bfloat16, torch.float32):
        return gemm.dense(a, b, a_mn=True, b_mn=True, out_dtype=out_dtype)
    if out_dtype == torch.float32 and a.dtype == torch.bfloat16:
        return torch.mm(a.t(), b, out_dtype=torch.float32)
    return torch.mm(a.t(), b).to(out_dtype)


class _LinearTc(torch.autograd.Function):
    """``x W^T (+ bias)`` with forward, data gradient and weight gradient on the dense tcgen05 kernel; the bias is added to
    the fp32 accumulator in the GEMM epilogue; the weight gradient goes directly into ``W.main_grad`` when the parameter
    has one."""

    @staticmethod
    def forward(ctx, x, weight, bias=None):
        from . import gemm
        x2 = _rows(x)
        ctx.save_for_backward(x2, weight)
        ctx.xshape = x.shape
        ctx.bias_dtype = None if bias is None else bias.dtype
        # the result is allocated in its final shape: a view returned from forward() would have the 2-D buffer as its
        # autograd-less `_base`, which code that looks at view chains (fused q|k|v detection) must never see
        y = torch.empty(*x.shape[:-1], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        gemm.dense(x2, weight, out=y.view(-1, weight.shape[0]), bias=bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import gemm
        x2, weight = ctx.saved_tensors
        dy2 = _rows(dy)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.xshape, dtype=torch.bfloat16, device=dy.device)
            gemm.dense(dy2, weight, b_mn=True, out=dx.view(-1, dx.shape[-1]))
        dw = None
        if ctx.needs_input_grad[1] and not wgrad_into_main_grad(weight, dy2, x2):
            dw = gemm.dense(dy2, x2, a_mn=True, b_mn=True)
        db = None
        if ctx.bias_dtype is not None and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(ctx.bias_dtype)
        return dx, dw, db


def _skinny_ok(x, weight) -> bool:
    """A linear with at most 16 input rows and no gradient (one-token decode steps): bound by streaming the weight once."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and x.numel() > 0
            and x.numel() // x.shape[-1] <= 16 and x.shape[-1] % 32 == 0 and weight.stride(1) == 1
            and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0
            and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad))
            and os.environ.get("LMOE_SKINNY_GEMM", "1") != "0")


def linear_skinny(x, weight):
    """``x W^T`` for up to 16 rows on ``gemm_skinny_kernel`` (csrc/gemm_skinny.cu): every CTA streams 16 rows of W through
    mma.sync fragments loaded straight from global memory, K split over its warps."""
    x2 = _rows(x)
    M, K = x2.shape
    N = weight.shape[0]
    y = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)
    ll = ctypes.c_longlong
    _check(lib().lmoe_gemm_skinny(_p(x2), ll(x2.stride(0)), _p(weight), ll(weight.stride(0)), _p(y), ll(N), _i32(M), _i32(N),
                                  _i32(K), _st()), "gemm_skinny")
    return y


def linear(x, weight, bias=None):
    from . import fp8, gemm
    if _skinny_ok(x, weight):
        y = linear_skinny(x, weight)
        return y if bias is None else y + bias.to(y.dtype)
    if fp8.enabled() and bias is None and fp8.supported(x, weight):
        return fp8.Fp8Linear.apply(x, weight)
    if (weight.dtype == x.dtype == torch.bfloat16 and weight.dim() == 2 and x.shape[-1] % 8 == 0 and x.numel() > 0
            and gemm.dense_ok(weight) and weight.shape[0] % 8 == 0):
        if bias is not None and bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.data_ptr() % 16 == 0:
            return _LinearTc.apply(x, weight, bias)
        y = _LinearTc.apply(x, weight)
        return y if bias is None else y + bias.to(y.dtype)
    return F.linear(x, weight if weight.dtype == x.dtype else weight.to(x.dtype),
                    None if bias is None else bias.to(x.dtype))


class _LinearSwigluTc(torch.autograd.Function):
    """fc1 + SwiGLU with the activation in the GEMM epilogue (``gemm.dense_swiglu``): one kernel writes the activation
    and the pre-activations the backward pass needs; backward = dSwiGLU kernel, then data and weight gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, weight):
        from . import gemm
        x2 = _rows(x)
        act, pre = gemm.dense_swiglu(x2, weight, want_pre=True, out_shape=(*x.shape[:-1], weight.shape[0] // 2))
        ctx.save_for_backward(x2, weight, pre)
        ctx.xshape = x.shape
        return act

    @staticmethod
    def backward(ctx, dact):
        from . import gemm
        x2, weight, pre = ctx.saved_tensors
        d2 = dact.reshape(-1, dact.shape[-1]).contiguous()
        dpre = torch.empty_like(pre)
        rows, Fh = d2.shape
        _check(lib().lmoe_swiglu_bwd(_p(d2), _p(pre), _p(dpre), _i64(rows), _i32(Fh), _i32(_dt(pre)), _st()), "swiglu_bwd")
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.xshape, dtype=torch.bfloat16, device=dact.device)
            gemm.dense(dpre, weight, b_mn=True, out=dx.view(-1, dx.shape[-1]))
        dw = None
        if ctx.needs_input_grad[1] and not wgrad_into_main_grad(weight, dpre, x2):
            dw = gemm.dense(dpre, x2, a_mn=True, b_mn=True)
        return dx, dw


class _MlpSwigluTc(torch.autograd.Function):
    """``(silu(x Wg^T) * (x Wu^T)) W2^T`` as four GEMMs with both halves of the activation inside GEMM epilogues: the
    forward fc1 writes the activation and the pre-activations; in the backward pass the fc2 data gradient goes through
    the SwiGLU backward in its epilogue and is never written."""

    @staticmethod
    def forward(ctx, x, w1, w2):
        from . import gemm
        x2 = _rows(x)
        act, pre = gemm.dense_swiglu(x2, w1, want_pre=True)
        y = torch.empty(*x.shape[:-1], w2.shape[0], dtype=torch.bfloat16, device=x.device)
        gemm.dense(act, w2, out=y.view(-1, w2.shape[0]))
        ctx.save_for_backward(x2, w1, w2, pre, act)
        ctx.xshape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import gemm
        x2, w1, w2, pre, act = ctx.saved_tensors
        dy2 = _rows(dy)
        dw2 = None
        if ctx.needs_input_grad[2] and not wgrad_into_main_grad(w2, dy2, act):
            dw2 = gemm.dense(dy2, act, a_mn=True, b_mn=True)
        dpre = gemm.dense_dswiglu(dy2, w2, pre)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.xshape, dtype=torch.bfloat16, device=dy.device)
            gemm.dense(dpre, w1, b_mn=True, out=dx.view(-1, dx.shape[-1]))
        dw1 = None
        if ctx.needs_input_grad[1] and not wgrad_into_main_grad(w1, dpre, x2):
            dw1 = gemm.dense(dpre, x2, a_mn=True, b_mn=True)
        return dx, dw1, dw2


def mlp_swiglu(x, w1, w2):
    """SwiGLU MLP ``fc2(swiglu(fc1(x)))`` without biases; the fully fused form when the shapes allow it."""
    from . import fp8, gemm
    if _skinny_ok(x, w1):
        return linear(swiglu(linear(x, w1)), w2)
    if (not fp8.enabled() and x.dtype == w1.dtype == w2.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.numel() > 0
            and gemm.dense_ok(w1, w2) and w1.shape[0] % 128 == 0 and w2.shape[0] % 8 == 0 and w2.shape[1] * 2 == w1.shape[0]
            and os.environ.get("LMOE_FUSED_MLP", "1") != "0"):
        return _MlpSwigluTc.apply(x, w1, w2)
    return linear(linear_swiglu(x, w1), w2)


def linear_swiglu(x, weight):
    """fc1 + SwiGLU.  bf16 operands that fit the dense tcgen05 kernel take its fused-epilogue form; fp8 and everything
    else go through :func:`linear` followed by the SwiGLU kernel."""
    from . import fp8, gemm
    if _skinny_ok(x, weight):
        return swiglu(linear(x, weight))
    if (not (fp8.enabled() and fp8.supported(x, weight)) and weight.dtype == x.dtype == torch.bfloat16 and weight.dim() == 2
            and x.shape[-1] % 8 == 0 and x.numel() > 0 and gemm.dense_ok(weight) and weight.shape[0] % 16 == 0
            and os.environ.get("LMOE_FUSED_SWIGLU", "1") != "0"):
        return _LinearSwigluTc.apply(x, weight)
    return swiglu(linear(x, weight))


def fused_tp_available(group) -> bool:
    from ..parallel import fused_comm
    return fused_comm.tp_workspace(group) is not None


def fused_lasp_available(group, q, k, v, g) -> bool:
    from ..parallel import fused_comm
    if fused_comm.lasp_workspace(group) is None:
        return False
    ws = fused_comm.lasp_workspace(group)
    B, _, H, D = q.shape
    return (q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype and D == v.shape[-1]
            and D == k.shape[-1] and D in (64, 128) and B * H * D * D <= ws.max_elems)


def lasp2_scalar(q, k, v, g, scale, group, chunk_size):
    from ..parallel import fused_comm
    return fused_comm.lasp2_scalar(q, k, v, g, scale, group)


def lasp2_vector(q, k, v, gk, scale, group, chunk_size):
    from ..parallel import fused_comm
    return fused_comm.lasp2_vector(q, k, v, gk, scale, group)


def allgather_linear(x, weight, bias, group, dim):
    from ..parallel import fused_comm
    return fused_comm.allgather_linear(x, weight, bias, group, dim)


def linear_reducescatter(x, weight, group, dim):
    from ..parallel import fused_comm
    return fused_comm.linear_reducescatter(x, weight, group, dim)


# =====================================================================================
# RMSNorm (+ residual add)
# =====================================================================================
def _partial_blocks() -> int:
    return num_sms() * 4


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps, want_residual):
        N = x.shape[-1]
        xc = x.contiguous()
        rc = None if residual is None else residual.contiguous()
        (w,) = _same_dtype(xc, weight)
        rows = xc.numel() // N
        y = torch.empty_like(xc)
        res_out = torch.empty_like(xc) if rc is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(lib().lmoe_rms_norm_fwd(_p(xc), _p(rc), _p(w), _p(y), _p(res_out), _p(rstd), _i64(rows), _i32(N),
                                       _f32(eps), _i32(_dt(xc)), _st()), "rms_norm_fwd")
        xin = res_out if rc is not None else xc
        ctx.save_for_backward(xin, w, rstd)
        ctx.has_res, ctx.wdtype = rc is not None, None if weight is None else weight.dtype
        if want_residual:
            return y, xin
        return y

    @staticmethod
    def backward(ctx, dy, dres=None):
        xin, w, rstd = ctx.saved_tensors
        N = xin.shape[-1]
        rows = xin.numel() // N
        dy = dy.contiguous()
        dres = None if dres is None else dres.contiguous()
        dx = torch.empty_like(xin)
        P = min(rows, _partial_blocks())
        partial = torch.empty(P, N, dtype=torch.float32, device=xin.device) if w is not None else None
        dw = torch.empty(N, dtype=xin.dtype, device=xin.device) if w is not None else None
        _check(lib().lmoe_rms_norm_bwd(_p(dy), _p(xin), _p(w), _p(rstd), _p(dres), _p(dx), _p(partial), _p(dw),
                                       _i64(rows), _i32(N), _i32(P), _i32(_dt(xin)), _st()), "rms_norm_bwd", 2)
        if dw is not None and ctx.wdtype != dw.dtype:
            dw = dw.to(ctx.wdtype)
        return dx, (dx if ctx.has_res else None), dw, None, None


def _embedding_lookup(ids, weight, id_offset, sharded):
    if not sharded:
        return F.embedding(ids, weight)
    local = ids - id_offset
    oob = (local < 0) | (local >= weight.shape[0])
    return F.embedding(local.masked_fill(oob, 0), weight).masked_fill(oob[..., None], 0.0)


class _Embedding(torch.autograd.Function):
    """Embedding lookup whose backward scatters the gradient rows straight into the table's fp32 accumulator
    (``csrc/embedding.cu``), without the dense ``[vocab, hidden]`` gradient tensor and the pass that adds it."""

    @staticmethod
    def forward(ctx, ids, weight, id_offset, sharded):
        ctx.save_for_backward(ids)
        ctx.weight, ctx.id_offset = weight, int(id_offset)
        return _embedding_lookup(ids, weight, id_offset, sharded)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        V, h = w.shape
        dy2 = dy.reshape(-1, h).contiguous()
        idf = ids.reshape(-1).to(torch.int64).contiguous()
        mg = getattr(w, "main_grad", None)
        direct = mg is not None and mg.dtype == torch.float32 and mg.is_contiguous()
        dst = mg if direct else torch.zeros(V, h, dtype=torch.float32, device=dy.device)
        _check(lib().lmoe_embedding_bwd(_p(dy2), _p(idf), _p(dst), _i64(dy2.shape[0]), _i32(h), _i64(V), _i64(ctx.id_offset),
                                        _i32(_dt(dy2)), _st()), "embedding_bwd")
        if direct:
            w._main_grad_fresh = False
            return None, None, None, None
        return None, dst.to(w.dtype), None, None


def embedding(ids, weight, id_offset: int = 0, sharded: bool = False):
    """``weight[ids - id_offset]``; with ``sharded`` ids outside this vocabulary shard give zero rows.  See
    :class:`_Embedding` for the backward."""
    if (weight.dtype not in (torch.bfloat16, torch.float32) or weight.shape[1] % 8
            or not (weight.requires_grad and torch.is_grad_enabled())):
        return _embedding_lookup(ids, weight, id_offset, sharded)
    return _Embedding.apply(ids, weight, id_offset, sharded)


class _LayerNorm(torch.autograd.Function):
    """LayerNorm (+ fused residual add) on the kernels of ``csrc/layernorm.cu``."""

    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, want_residual):
        N = x.shape[-1]
        xc = x.contiguous()
        rc = None if residual is None else residual.contiguous()
        w, b = _same_dtype(xc, weight, bias)
        rows = xc.numel() // N
        y = torch.empty_like(xc)
        res_out = torch.empty_like(xc) if rc is not None else None
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(lib().lmoe_layer_norm_fwd(_p(xc), _p(rc), _p(w), _p(b), _p(y), _p(res_out), _p(mean), _p(rstd), _i64(rows),
                                         _i32(N), _f32(eps), _i32(_dt(xc)), _st()), "layer_norm_fwd")
        xin = res_out if rc is not None else xc
        ctx.save_for_backward(xin, w, mean, rstd)
        ctx.has_res = rc is not None
        ctx.wdtype = None if weight is None else weight.dtype
        ctx.bdtype = None if bias is None else bias.dtype
        if want_residual:
            return y, xin
        return y

    @staticmethod
    def backward(ctx, dy, dres=None):
        xin, w, mean, rstd = ctx.saved_tensors
        N = xin.shape[-1]
        rows = xin.numel() // N
        dy = dy.contiguous()
        dres = None if dres is None else dres.contiguous()
        dx = torch.empty_like(xin)
        P = min(rows, _partial_blocks())
        want = ctx.wdtype is not None or ctx.bdtype is not None
        partial = torch.empty(P, 2 * N, dtype=torch.float32, device=xin.device) if want else None
        dwdb = torch.empty(2 * N, dtype=torch.float32, device=xin.device) if want else None
        _check(lib().lmoe_layer_norm_bwd(_p(dy), _p(xin), _p(w), _p(mean), _p(rstd), _p(dres), _p(dx), _p(partial), _p(dwdb),
                                         _i64(rows), _i32(N), _i32(P), _i32(_dt(xin)), _st()), "layer_norm_bwd", 2)
        dw = None if ctx.wdtype is None else dwdb[:N].to(ctx.wdtype)
        db = None if ctx.bdtype is None else dwdb[N:].to(ctx.bdtype)
        return dx, (dx if ctx.has_res else None), dw, db, None, None


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    if not _rms_ok(x):
        return R.layer_norm(x, weight, bias, eps)
    return _LayerNorm.apply(x, None, weight, bias, eps, False)


def add_layer_norm(x, residual, weight, bias, eps: float = 1e-5):
    if not _rms_ok(x) or residual.dtype != x.dtype:
        r = x + residual
        return R.layer_norm(r, weight, bias, eps), r
    return _LayerNorm.apply(x, residual, weight, bias, eps, True)


def _rms_ok(x):
    N = x.shape[-1]
    vn = 8 if x.dtype == torch.bfloat16 else 4
    return x.dtype in (torch.bfloat16, torch.float32) and N % vn == 0 and N // vn <= 2048


def rms_norm(x, weight=None, eps: float = 1e-6):
    if not _rms_ok(x):
        return R.rms_norm(x, weight, eps)
    return _RMSNorm.apply(x, None, weight, eps, False)


def add_rms_norm(x, residual, weight, eps: float = 1e-6):
    if not _rms_ok(x):
        r = x + residual
        return R.rms_norm(r, weight, eps), r
    return _RMSNorm.apply(x, residual, weight, eps, True)


# =====================================================================================
# per-head norm + swish gate
# =====================================================================================
class _HeadNormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, weight, gate, eps, do_norm):
        B, T, H, D = o.shape
        oc, gc = o.contiguous(), gate.contiguous()
        (w,) = _same_dtype(oc, weight)
        rows = B * T * H
        y = torch.empty(B, T, H * D, dtype=o.dtype, device=o.device)
        rstd = torch.empty(rows if do_norm else 1, dtype=torch.float32, device=o.device)
        _check(lib().lmoe_head_norm_gate_fwd(_p(oc), _p(w), _p(gc), _p(y), _p(rstd), _i64(rows), _i32(D), _f32(eps),
                                             _i32(int(do_norm)), _i32(_dt(oc)), _st()), "head_norm_gate_fwd")
        ctx.save_for_backward(oc, w, gc, rstd)
        ctx.do_norm, ctx.wdtype = do_norm, None if weight is None else weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        oc, w, gc, rstd = ctx.saved_tensors
        B, T, H, D = oc.shape
        rows = B * T * H
        dy = dy.contiguous()
        d_o, dgate = torch.empty_like(oc), torch.empty_like(gc)
        need_dw = w is not None and ctx.do_norm
        P = min((rows + 7) // 8, num_sms() * 8)
        partial = torch.empty(P, D, dtype=torch.float32, device=oc.device) if need_dw else None
        dw = torch.empty(D, dtype=oc.dtype, device=oc.device) if need_dw else None
        _check(lib().lmoe_head_norm_gate_bwd(_p(dy), _p(oc), _p(w), _p(gc), _p(rstd), _p(d_o), _p(dgate), _p(partial),
                                             _p(dw), _i64(rows), _i32(D), _i32(int(ctx.do_norm)), _i32(P),
                                             _i32(_dt(oc)), _st()), "head_norm_gate_bwd", 2)
        if dw is not None and ctx.wdtype != dw.dtype:
            dw = dw.to(ctx.wdtype)
        return d_o, dw, dgate, None, None


def head_norm_gate(o, weight, gate, eps, do_norm: bool):
    if o.shape[-1] > 512 or o.dtype not in (torch.bfloat16, torch.float32) or gate.dtype != o.dtype:
        y = R.rms_norm(o, weight, eps) if do_norm else o
        B, T = o.shape[:2]
        return (y.reshape(B, T, -1).float() * F.silu(gate.float())).to(o.dtype)
    return _HeadNormGate.apply(o, weight if do_norm else None, gate, eps, do_norm)


# =====================================================================================
# gated RMSNorm (Mamba2)
# =====================================================================================
class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, z, weight, eps, G):
        N = x.shape[-1]
        xc, zc = x.contiguous(), z.contiguous()
        (w,) = _same_dtype(xc, weight)
        rows = xc.numel() // N
        y = torch.empty_like(xc)
        rstd = torch.empty(rows * (N // G), dtype=torch.float32, device=x.device)
        _check(lib().lmoe_gated_rms_norm_fwd(_p(xc), _p(zc), _p(w), _p(y), _p(rstd), _i64(rows), _i32(N), _i32(G),
                                             _f32(eps), _i32(_dt(xc)), _st()), "gated_rms_norm_fwd")
        ctx.save_for_backward(xc, zc, w, rstd)
        ctx.G, ctx.wdtype = G, weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, zc, w, rstd = ctx.saved_tensors
        N = xc.shape[-1]
        rows = xc.numel() // N
        dx, dz = torch.empty_like(xc), torch.empty_like(zc)
        dw = torch.zeros(N, dtype=torch.float32, device=xc.device)
        _check(lib().lmoe_gated_rms_norm_bwd(_p(dy.contiguous()), _p(xc), _p(zc), _p(w), _p(rstd), _p(dx), _p(dz),
                                             _p(dw), _i64(rows), _i32(N), _i32(ctx.G), _i32(_dt(xc)), _st()),
               "gated_rms_norm_bwd")
        return dx, dz, dw.to(ctx.wdtype), None, None


def gated_rms_norm(x, z, weight, eps=1e-5, group_size=None):
    if x.dtype not in (torch.bfloat16, torch.float32) or z.dtype != x.dtype:
        return R.gated_rms_norm(x, z, weight, eps, group_size)
    return _GatedRMSNorm.apply(x, z, weight, eps, group_size or x.shape[-1])


# =====================================================================================
# SwiGLU, l2norm, rotary
# =====================================================================================
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        F2 = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // F2
        y = torch.empty(*x.shape[:-1], F2 // 2, dtype=x.dtype, device=x.device)
        _check(lib().lmoe_swiglu_fwd(_p(xc), _p(y), _i64(rows), _i32(F2 // 2), _i32(_dt(xc)), _st()), "swiglu_fwd")
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        F2 = xc.shape[-1]
        dx = torch.empty_like(xc)
        _check(lib().lmoe_swiglu_bwd(_p(dy.contiguous()), _p(xc), _p(dx), _i64(xc.numel() // F2), _i32(F2 // 2),
                                     _i32(_dt(xc)), _st()), "swiglu_bwd")
        return dx


def swiglu(x):
    vn = 8 if x.dtype == torch.bfloat16 else 4
    if x.dtype not in (torch.bfloat16, torch.float32) or (x.shape[-1] // 2) % vn != 0:
        return R.swiglu(x)
    return _SwiGLU.apply(x)


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        D = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // D
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(lib().lmoe_l2norm_fwd(_p(xc), _p(y), _p(rstd), _i64(rows), _i32(D), _f32(eps), _i32(_dt(xc)), _st()),
               "l2norm_fwd")
        ctx.save_for_backward(xc, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, rstd = ctx.saved_tensors
        D = xc.shape[-1]
        dx = torch.empty_like(xc)
        _check(lib().lmoe_l2norm_bwd(_p(dy.contiguous()), _p(xc), _p(rstd), _p(dx), _i64(xc.numel() // D), _i32(D),
                                     _i32(_dt(xc)), _st()), "l2norm_bwd")
        return dx, None


def l2_norm(x, eps: float = 1e-6):
    if x.shape[-1] > 512 or x.dtype not in (torch.bfloat16, torch.float32):
        return R.l2_norm(x, eps)
    return _L2Norm.apply(x, eps)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved):
        B, T, H, D = x.shape
        xc = x.contiguous()
        cs, sn = cos.float().contiguous(), sin.float().contiguous()
        y = torch.empty_like(xc)
        Rr = cs.shape[-1] * 2
        _check(lib().lmoe_rope(_p(xc), _p(cs), _p(sn), _p(y), _i64(B * T), _i32(T), _i32(H), _i32(D), _i32(Rr),
                               _i32(int(interleaved)), _i32(0), _i32(_dt(xc)), _st()), "rope_fwd")
        ctx.save_for_backward(cs, sn)
        ctx.interleaved = interleaved
        return y

    @staticmethod
    def backward(ctx, dy):
        cs, sn = ctx.saved_tensors
        B, T, H, D = dy.shape
        dyc = dy.contiguous()
        dx = torch.empty_like(dyc)
        _check(lib().lmoe_rope(_p(dyc), _p(cs), _p(sn), _p(dx), _i64(B * T), _i32(T), _i32(H), _i32(D),
                               _i32(cs.shape[-1] * 2), _i32(int(ctx.interleaved)), _i32(1), _i32(_dt(dyc)), _st()),
               "rope_bwd")
        return dx, None, None, None


def apply_rope(x, cos, sin, interleaved=False):
    if x.dtype not in (torch.bfloat16, torch.float32):
        return R.apply_rope(x, cos, sin, interleaved)
    return _Rope.apply(x, cos, sin, interleaved)


# =====================================================================================
# softmax cross entropy on a chunk of logits
# =====================================================================================
def softmax_ce_fwd(logits, labels, loss_out, lse_out, ignore_index):
    rows, V = logits.shape
    logits = logits.contiguous()
    _check(lib().lmoe_softmax_ce_fwd(_p(logits), _p(labels.contiguous()), _p(loss_out), _p(lse_out), _i64(rows), _i32(V),
                                     _i64(ignore_index), _i32(_dt(logits)), _st()), "softmax_ce_fwd")


def softmax_ce_bwd(logits, labels, lse, gloss, ignore_index):
    """Overwrites ``logits`` with the gradient and returns it."""
    rows, V = logits.shape
    _check(lib().lmoe_softmax_ce_bwd(_p(logits), _p(labels.contiguous()), _p(lse), _p(gloss), _p(logits), _i64(rows),
                                     _i32(V), _i64(ignore_index), _i32(_dt(logits)), _st()), "softmax_ce_bwd")
    return logits


# =====================================================================================
# causal conv1d
# =====================================================================================
class _CausalConv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, init, act):
        B, T, D = x.shape
        K = weight.shape[-1]
        xc = x.contiguous()
        w, b, ini = _same_dtype(xc, weight.contiguous(), bias, None if init is None else init.contiguous())
        y = torch.empty_like(xc)
        _check(lib().lmoe_causal_conv1d_fwd(_p(xc), _p(w), _p(b), _p(ini), _p(y), _i32(B), _i32(T), _i32(D), _i32(K),
                                            _i32(int(act)), _i32(_dt(xc)), _st()), "causal_conv1d_fwd")
        ctx.save_for_backward(xc, w, b, ini)
        ctx.act, ctx.wdtype, ctx.bdtype = act, weight.dtype, None if bias is None else bias.dtype
        # final state: the last K-1 inputs (including the entering state when T < K-1)
        if T >= K - 1:
            tail = xc[:, T - (K - 1):].clone()
        elif ini is not None:
            tail = torch.cat([ini, xc], dim=1)[:, -(K - 1):]
        else:
            tail = F.pad(xc, (0, 0, K - 1 - T, 0))
        ctx.mark_non_differentiable(tail)
        return y, tail

    @staticmethod
    def backward(ctx, dy, _dtail):
        xc, w, b, ini = ctx.saved_tensors
        B, T, D = xc.shape
        K = w.shape[-1]
        dx = torch.empty_like(xc)
        dw = torch.zeros(D, K, dtype=torch.float32, device=xc.device)
        db = torch.zeros(D, dtype=torch.float32, device=xc.device) if b is not None else None
        dini = torch.empty_like(ini) if ini is not None else None
        _check(lib().lmoe_causal_conv1d_bwd(_p(dy.contiguous()), _p(xc), _p(w), _p(b), _p(ini), _p(dx), _p(dw), _p(db),
                                            _p(dini), _i32(B), _i32(T), _i32(D), _i32(K), _i32(int(ctx.act)),
                                            _i32(_dt(xc)), _st()), "causal_conv1d_bwd")
        return dx, dw.to(ctx.wdtype), None if db is None else db.to(ctx.bdtype), dini, None


def causal_conv1d(x, weight, bias=None, activation="silu", initial_state=None):
    K = weight.shape[-1]
    if x.dtype not in (torch.bfloat16, torch.float32) or K not in (2, 3, 4):
        return R.causal_conv1d(x, weight, bias, activation, initial_state)
    return _CausalConv1d.apply(x, weight, bias, initial_state, activation in ("silu", "swish"))


# =====================================================================================
# router
# =====================================================================================
class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, order):
        T, E = logits.shape
        lf = logits.float().contiguous()
        full = torch.empty_like(lf)
        probs = torch.empty(T, k, dtype=torch.float32, device=lf.device)
        idx = torch.empty(T, k, dtype=torch.int64, device=lf.device)
        _check(lib().lmoe_router_topk(_p(lf), _p(full), _p(probs), _p(idx), _p(None), _i64(T), _i32(E), _i32(k),
                                      _i32(1 if order == "topk_softmax" else 0), _st()), "router_topk")
        ctx.save_for_backward(full, probs, idx)
        ctx.order, ctx.dtype = order, logits.dtype
        ctx.mark_non_differentiable(idx)
        return probs, idx, full

    @staticmethod
    def backward(ctx, dprobs, _didx, dfull):
        full, probs, idx = ctx.saved_tensors
        if ctx.order == "softmax_topk":
            g = dfull.clone() if dfull is not None else torch.zeros_like(full)
            if dprobs is not None:
                g.scatter_add_(1, idx, dprobs)
            dl = full * (g - (g * full).sum(-1, keepdim=True))
        else:
            dl = torch.zeros_like(full)
            if dfull is not None:
                dl = full * (dfull - (dfull * full).sum(-1, keepdim=True))
            if dprobs is not None:
                dsel = probs * (dprobs - (dprobs * probs).sum(-1, keepdim=True))
                dl.scatter_add_(1, idx, dsel)
        return dl.to(ctx.dtype), None, None


def router_topk(logits, k, order="softmax_topk"):
    if logits.shape[-1] > 256 or k > 16:
        return R.router_topk(logits, k, order)
    return _RouterTopK.apply(logits, k, order)


class _GatedAdd(torch.autograd.Function):
    """``a + s * sigmoid(g)`` with one gate logit per row (``csrc/gated_add.cu``)."""

    @staticmethod
    def forward(ctx, a, s, g):
        N = a.shape[-1]
        a2, s2 = a.reshape(-1, N).contiguous(), s.reshape(-1, N).contiguous()
        g2 = g.reshape(-1).contiguous()
        out = torch.empty_like(a2)
        _check(lib().lmoe_gated_add_fwd(_p(a2), _p(s2), _p(g2), _p(out), _i64(a2.shape[0]), _i32(N), _i32(_dt(a2)), _st()),
               "gated_add_fwd")
        ctx.save_for_backward(s2, g2)
        ctx.shapes = (a.shape, g.shape)
        return out.view(a.shape)

    @staticmethod
    def backward(ctx, d_out):
        s2, g2 = ctx.saved_tensors
        N = s2.shape[-1]
        d2 = d_out.reshape(-1, N).contiguous()
        ds = torch.empty_like(s2)
        dg = torch.empty_like(g2)
        _check(lib().lmoe_gated_add_bwd(_p(d2), _p(s2), _p(g2), _p(ds), _p(dg), _i64(d2.shape[0]), _i32(N), _i32(_dt(d2)), _st()),
               "gated_add_bwd")
        return d_out, ds.view(ctx.shapes[0]), dg.view(ctx.shapes[1])


def gated_add(a, s, g):
    if a.dtype != s.dtype or g.dtype != a.dtype or a.dtype not in (torch.bfloat16, torch.float32) or a.shape[-1] % 8:
        return a + s * torch.sigmoid(g)
    return _GatedAdd.apply(a, s, g)


def moe_dprobs(rows, d_out, dest_rank, T, k):
    """Gradient of the routing probabilities in the MoE combine: ``d_probs[t, j] = <rows[t*k+j], d_out[t]>``, zero for
    dropped assignments (``moe_dprobs_kernel``, csrc/moe_comm.cu)."""
    h = d_out.shape[-1]
    rows, d_out = rows.contiguous(), d_out.contiguous()
    out = torch.empty(T, k, dtype=torch.float32, device=d_out.device)
    _check(lib().lmoe_moe_dprobs(_p(rows), _p(d_out), _p(dest_rank), _p(out), _i32(T), _i32(k), _i32(h), _i32(num_sms()),
                                 _st()), "moe_dprobs")
    return out


def grouped_mlp(x_sorted, tokens_per_expert, w1, w2):
    from . import gemm
    if gemm.available() and gemm.supports_grouped(x_sorted, w1, w2):
        return gemm.grouped_mlp(x_sorted, tokens_per_expert, w1, w2)
    if (hasattr(torch, "_grouped_mm") and x_sorted.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16
            and os.environ.get("LMOE_LIBRARY_GROUPED_MM", "1") != "0"):
        # library grouped GEMM (the counterpart of the grouped_gemm package the reference's --moe-grouped-gemm uses):
        # what the comparison arm of the benchmarks runs, and the fallback for shapes the tcgen05 kernel does not take
        try:
            offs = torch.cumsum(tokens_per_expert, 0).to(torch.int32)
            return torch._grouped_mm(swiglu(torch._grouped_mm(x_sorted, w1, offs=offs)), w2, offs=offs)
        except RuntimeError:
            pass
    outs, start = [], 0
    counts = tokens_per_expert.tolist()
    for e, n in enumerate(counts):
        xe = x_sorted[start:start + n]
        outs.append(swiglu(xe @ w1[e]) @ w2[e])
        start += n
    return torch.cat(outs, 0)


# =====================================================================================
# attention
# =====================================================================================
def flash_attention(q, k, v, scale, causal, q_offset, window):
    from . import attention
    return attention.flash_attention(q, k, v, scale, causal, q_offset, window)


# =====================================================================================
# fused Adam
# =====================================================================================
def fused_adam(p, master, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, gscale):
    n = p.numel()
    _check(lib().lmoe_fused_adam(_p(p), _p(master), _p(g), _p(m), _p(v), _i64(n), _f32(lr), _f32(b1), _f32(b2), _f32(eps),
                                 _f32(wd), _f32(bc1), _f32(bc2), _f32(gscale), _i32(_dt(p)), _st()), "fused_adam")


def accumulate_grad(acc, g):
    _check(lib().lmoe_accumulate_grad(_p(acc), _p(g), _i64(g.numel()), _i32(_dt(g)), _st()), "accumulate_grad")


# =====================================================================================
# linear sequence models
# =====================================================================================
class _LsmArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("q", "k", "v", "d_o")] +
                [(n, ctypes.c_int64) for n in ("qs_b", "qs_t", "qs_h", "ks_b", "ks_t", "ks_h", "vs_b", "vs_t", "vs_h")] +
                [(n, ctypes.c_void_p) for n in ("o", "dq", "dk", "dv")] +
                [(n, ctypes.c_int64) for n in ("dqs_b", "dqs_t", "dqs_h", "dks_b", "dks_t", "dks_h", "dvs_b", "dvs_t", "dvs_h")] +
                [("g", ctypes.c_void_p), ("gmode", ctypes.c_int), ("scale", ctypes.c_float)] +
                [(n, ctypes.c_int) for n in ("B", "T", "H", "G", "cpg")] +
                [("states", ctypes.c_void_p), ("gdecay", ctypes.c_void_p)])


def _inner_contig(t):
    """Kernels need unit stride in the last dim and 16-byte aligned rows; other strides are free."""
    if t.stride(-1) != 1 or any(s % 8 for s in t.stride()[:-1]) or t.data_ptr() % 16:
        return t.contiguous()
    return t


def lsm_groups(B, H, T):
    nchunks = (T + 63) // 64
    G = max(1, min(nchunks, num_sms() // max(B * H, 1)))
    cpg = (nchunks + G - 1) // G
    G = (nchunks + cpg - 1) // cpg
    return G, cpg


def _lsm_args(q, k, v, g, gmode, scale, B, T, H, G, cpg, states, gdecay, d_o=None, o=None, dq=None, dk=None, dv=None):
    a = _LsmArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.d_o = 0 if d_o is None else d_o.data_ptr()
    a.qs_b, a.qs_t, a.qs_h = q.stride(0), q.stride(1), q.stride(2)
    a.ks_b, a.ks_t, a.ks_h = k.stride(0), k.stride(1), k.stride(2)
    a.vs_b, a.vs_t, a.vs_h = v.stride(0), v.stride(1), v.stride(2)
    a.o = 0 if o is None else o.data_ptr()
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(a, name, 0 if t is None else t.data_ptr())
        if t is not None:
            setattr(a, name + "s_b", t.stride(0)), setattr(a, name + "s_t", t.stride(1)), setattr(a, name + "s_h", t.stride(2))
    a.g = 0 if g is None else g.data_ptr()
    a.gmode, a.scale = gmode, float(scale)
    a.B, a.T, a.H, a.G, a.cpg = B, T, H, G, cpg
    a.states = states.data_ptr()
    a.gdecay = 0 if gdecay is None else gdecay.data_ptr()
    return a


def _lsm_launch(which, D, args):
    _check(lib().lmoe_lsm_scalar_launch(_i32(which), _i32(D), ctypes.byref(args), _st()), f"lsm_scalar[{which}]")


def _lsm_combine(rev, states, gdecay, gconst, seed, final_out, BH, H, G, cpg, T, D):
    _check(lib().lmoe_lsm_scalar_combine(_i32(rev), _p(states), _p(gdecay), _p(gconst), _p(seed), _p(final_out), _i32(BH),
                                         _i32(H), _i32(G), _i32(cpg), _i32(T), _i32(D), _st()), "lsm_scalar_combine")


_LASP_CTX = None          # set by parallel.fused_comm.lasp2_scalar while a sequence-parallel call is running


class _LsmScalar(torch.autograd.Function):
    """o, S_T = scalar-decay linear attention.  q,k,v bf16 [B,T,H,D]; g None | [H] | [B,T,H] fp32."""

    @staticmethod
    def forward(ctx, q, k, v, g, scale, init):
        B, T, H, D = q.shape
        q, k, v = _inner_contig(q), _inner_contig(k), _inner_contig(v)
        gmode = 0 if g is None else (1 if g.dim() == 1 else 2)
        gf = None if g is None else g.float().contiguous()
        G, cpg = lsm_groups(B, H, T)
        states = torch.empty(B, H, G, D, D, dtype=torch.float32, device=q.device)
        gdecay = torch.empty(B, H, G, dtype=torch.float32, device=q.device) if gmode == 2 else None
        o = torch.empty(B, T, H, D, dtype=q.dtype, device=q.device)
        final = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
        seed = None if init is None else init.float().contiguous()
        a = _lsm_args(q, k, v, gf, gmode, scale, B, T, H, G, cpg, states, gdecay, o=o)
        _lsm_launch(0, D, a)
        lasp = _LASP_CTX if init is None else None
        if lasp is not None:       # sequence split over ranks: exchange fused into the combine kernel
            lasp.combine(0, states, gf if gmode == 1 else None, final, B * H, H, G, cpg, T, D,
                         gdecay=gdecay, dmode=1 if gmode == 2 else 0)
        else:
            _lsm_combine(0, states, gdecay, gf if gmode == 1 else None, seed, final, B * H, H, G, cpg, T, D)
        _lsm_launch(2, D, a)
        ctx.lasp = lasp
        ctx.save_for_backward(q, k, v, gf, states, gdecay, final)
        ctx.scale, ctx.gmode, ctx.grid, ctx.has_init = scale, gmode, (G, cpg), init is not None
        ctx.g_dtype = None if g is None else g.dtype
        return o, final

    @staticmethod
    def backward(ctx, d_o, dfinal):
        q, k, v, gf, states, gdecay, final = ctx.saved_tensors
        B, T, H, D = q.shape
        G, cpg = ctx.grid
        d_o = d_o.contiguous()
        if d_o.dtype != q.dtype:
            d_o = d_o.to(q.dtype)
        # dq | dk | dv are written straight into one [B,T,H,3D] buffer: when q,k,v were views of a fused
        # projection, autograd's concatenation of the three gradients becomes a no-op copy
        dqkv = torch.empty(B, T, H, 3 * D, dtype=q.dtype, device=q.device)
        dq, dk, dv = dqkv[..., :D], dqkv[..., D:2 * D], dqkv[..., 2 * D:]
        dstates = torch.empty_like(states)
        dinit = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device) if ctx.has_init else None
        # forward-direction sweep: dq (entering states of every group are still in `states`)
        a = _lsm_args(q, k, v, gf, ctx.gmode, ctx.scale, B, T, H, G, cpg, states, gdecay, d_o=d_o, dq=dq)
        _lsm_launch(3, D, a)
        # reverse-direction: group summaries of dS, suffix combine, dk/dv sweep
        a2 = _lsm_args(q, k, v, gf, ctx.gmode, ctx.scale, B, T, H, G, cpg, dstates, None, d_o=d_o, dk=dk, dv=dv)
        _lsm_launch(1, D, a2)
        seed = None if dfinal is None else dfinal.float().contiguous()
        if ctx.lasp is not None:
            # the gradient of the state that leaves this rank arrives from the ranks after it; the decay gradient needs it
            need_r = ctx.gmode == 2 or (ctx.gmode == 1 and len(ctx.needs_input_grad) > 3 and ctx.needs_input_grad[3])
            r_out = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device) if need_r else None
            ctx.lasp.combine(1, dstates, gf if ctx.gmode == 1 else None, None, B * H, H, G, cpg, T, D,
                             gdecay=gdecay, dmode=1 if ctx.gmode == 2 else 0, r_out=r_out)
            dfinal = r_out
        else:
            _lsm_combine(1, dstates, gdecay, gf if ctx.gmode == 1 else None, seed, dinit, B * H, H, G, cpg, T, D)
        _lsm_launch(4, D, a2)
        dg = None
        if ctx.gmode == 2:
            # dg_t = sum_{i>=t} q_i.dq_i - sum_{j>=t} k_j.dk_j (+ <S_T, dS_T> when the final state has a gradient)
            s = ((q.float() * dq.float()).sum(-1) - (k.float() * dk.float()).sum(-1)).transpose(1, 2).contiguous()
            c = s.cumsum(-1)                             # scan along the innermost dimension of [B,H,T]
            dg = (c[..., -1:] - c + s).transpose(1, 2)
            if dfinal is not None:
                dg = dg + (final * dfinal.float()).sum((-1, -2))[:, None, :]
            dg = dg.to(ctx.g_dtype)
        elif ctx.gmode == 1 and len(ctx.needs_input_grad) > 3 and ctx.needs_input_grad[3]:
            s = (q.float() * dq.float()).sum(-1) - (k.float() * dk.float()).sum(-1)
            dgt = s.flip(1).cumsum(1).flip(1)
            if dfinal is not None:
                dgt = dgt + (final * dfinal.float()).sum((-1, -2))[:, None, :]
            dg = dgt.sum((0, 1)).to(ctx.g_dtype)
        return dq, dk, dv, dg, None, dinit


def _fused_base(q, k, v):
    """If q, k, v are the three slices of one [B,T,H,3D] tensor (a fused projection), return that tensor."""
    base = q._base                                   # root of the view chain, e.g. the projection output [B,T,H*3D]
    if base is None or k._base is not base or v._base is not base or not base.is_contiguous():
        return None
    if base.requires_grad != (q.requires_grad or k.requires_grad or v.requires_grad):
        return None                                  # a root outside the autograd graph would drop the gradients
    B, T, H, D = q.shape
    if base.numel() != B * T * H * 3 * D:
        return None
    e = base.element_size()
    if (q.data_ptr() != base.data_ptr() or k.data_ptr() != base.data_ptr() + D * e
            or v.data_ptr() != base.data_ptr() + 2 * D * e):
        return None
    want = (T * H * 3 * D, H * 3 * D, 3 * D, 1)
    if q.stride() != want or k.stride() != want or v.stride() != want:
        return None
    return base.view(B, T, H, 3 * D)


class _LsmScalarFused(torch.autograd.Function):
    """Same as ``_LsmScalar`` with q|k|v given as one fused ``[B,T,H,3D]`` tensor, so that the backward hands
    autograd one gradient tensor instead of three slices it would have to concatenate."""

    @staticmethod
    def forward(ctx, qkv, g, scale, init):
        D = qkv.shape[-1] // 3
        q, k, v = qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:]
        return _LsmScalar.forward(ctx, q, k, v, g, scale, init)

    @staticmethod
    def backward(ctx, d_o, dfinal):
        dq, dk, dv, dg, _, dinit = _LsmScalar.backward(ctx, d_o, dfinal)
        return dq._base, dg, None, dinit


def lsm_scalar(q, k, v, g, scale, initial_state, chunk_size):
    D = q.shape[-1]
    ok = (q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype and v.shape[-1] == D
          and k.shape[-1] == D and D in (64, 128))
    Dv = v.shape[-1]
    if (not ok and q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype and k.shape[-1] == D
            and D in (64, 128) and Dv < D):
        # value heads narrower than the key/state width (Mamba2: head dim 64, state 128): zero-pad the values
        scale = D ** -0.5 if scale is None else scale
        s0 = None if initial_state is None else F.pad(initial_state, (0, D - Dv))
        o, S = lsm_scalar(q, k, F.pad(v, (0, D - Dv)), g, scale, s0, chunk_size)
        return o[..., :Dv], (None if S is None else S[..., :Dv])
    if (not ok and q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype and k.shape[-1] == D
            and q.shape[1] > 1 and os.environ.get("LMOE_LSM_BLOCKED", "1") != "0"):
        # any other feature / value width (Based and Rebased feature maps, the normaliser's column of ones): the sum of
        # the kernel over 128-wide key blocks, one call per value block
        from .lsm_blocked import blocked_scalar
        return blocked_scalar(lsm_scalar, q, k, v, g, scale, initial_state, chunk_size)
    if not ok:
        return LT.chunk_scalar_gated(q, k, v, g, scale, initial_state, chunk_size)
    scale = D ** -0.5 if scale is None else scale
    if q.shape[1] == 1 and _LASP_CTX is None and not (torch.is_grad_enabled() and
                                                      any(t.requires_grad for t in (q, k, v) if t is not None)):
        return _lsm_step(q, k, v, g, None, scale, initial_state)
    base = _fused_base(q, k, v)
    if base is not None:
        return _LsmScalarFused.apply(base, g, scale, initial_state)
    return _LsmScalar.apply(q, k, v, g, scale, initial_state)


def _lsm_step(q, k, v, g, gk, scale, initial_state):
    """Decoding: one token per sequence, S' = e^g diag(e^gk) S + k^T v, o = scale q S' in one launch (csrc/lsm_step.cu).
    g: None | [H] | [B,1,H]; gk: None | [B,1,H,D]."""
    B, _, H, D = q.shape
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    gf = None
    if g is not None:
        gf = (g.float().expand(B, H) if g.dim() == 1 else g.float().reshape(B, H)).contiguous()
    gkf = None if gk is None else gk.float().reshape(B, H, D).contiguous()
    s_in = None if initial_state is None else initial_state.float().contiguous()
    s_out = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
    o = torch.empty(B, 1, H, D, dtype=q.dtype, device=q.device)
    ll = ctypes.c_longlong
    _check(lib().lmoe_lsm_scalar_step(_p(q), _p(k), _p(v), ll(q.stride(0)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(2)),
                                      ll(v.stride(0)), ll(v.stride(2)), _p(gf), _p(gkf), _p(s_in), _p(s_out), _p(o), ctypes.c_int(B),
                                      ctypes.c_int(H), ctypes.c_int(D), ctypes.c_float(scale), _st()), "lsm_scalar_step")
    return o, s_out


class _GlaArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("q", "k", "v", "d_o")] +
                [(n, ctypes.c_int64) for n in ("qs_b", "qs_t", "qs_h", "ks_b", "ks_t", "ks_h", "vs_b", "vs_t", "vs_h")] +
                [(n, ctypes.c_void_p) for n in ("o", "dq", "dk", "dv")] +
                [(n, ctypes.c_int64) for n in ("dqs_b", "dqs_t", "dqs_h", "dks_b", "dks_t", "dks_h", "dvs_b", "dvs_t", "dvs_h")] +
                [("gk", ctypes.c_void_p), ("scale", ctypes.c_float)] +
                [(n, ctypes.c_int) for n in ("B", "T", "H", "G", "cpg")] +
                [("states", ctypes.c_void_p), ("gdecay", ctypes.c_void_p)])


def _gla_args(q, k, v, gk, scale, B, T, H, G, cpg, states, gdecay, d_o=None, o=None, dq=None, dk=None, dv=None):
    a = _GlaArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.d_o = 0 if d_o is None else d_o.data_ptr()
    a.qs_b, a.qs_t, a.qs_h = q.stride(0), q.stride(1), q.stride(2)
    a.ks_b, a.ks_t, a.ks_h = k.stride(0), k.stride(1), k.stride(2)
    a.vs_b, a.vs_t, a.vs_h = v.stride(0), v.stride(1), v.stride(2)
    a.o = 0 if o is None else o.data_ptr()
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(a, name, 0 if t is None else t.data_ptr())
        if t is not None:
            setattr(a, name + "s_b", t.stride(0)), setattr(a, name + "s_t", t.stride(1)), setattr(a, name + "s_h", t.stride(2))
    a.gk, a.scale = gk.data_ptr(), float(scale)
    a.B, a.T, a.H, a.G, a.cpg = B, T, H, G, cpg
    a.states = states.data_ptr()
    a.gdecay = 0 if gdecay is None else gdecay.data_ptr()
    return a


def _gla_launch(which, D, args):
    _check(lib().lmoe_gla_launch(_i32(which), _i32(D), ctypes.byref(args), _st()), f"gla[{which}]")


def _gla_combine(rev, states, gdecay, seed, final_out, BH, G, D):
    _check(lib().lmoe_gla_combine(_i32(rev), _p(states), _p(gdecay), _p(seed), _p(final_out), _i32(BH), _i32(G), _i32(D),
                                  _st()), "gla_combine")


class _LsmVector(torch.autograd.Function):
    """o, S_T = linear attention with a log decay per key channel.  q,k,v bf16 [B,T,H,D]; gk [B,T,H,D]."""

    @staticmethod
    def forward(ctx, q, k, v, gk, scale, init):
        B, T, H, D = q.shape
        q, k, v = _inner_contig(q), _inner_contig(k), _inner_contig(v)
        gf = gk.float().contiguous()
        G, cpg = lsm_groups(B, H, T)
        states = torch.empty(B, H, G, D, D, dtype=torch.float32, device=q.device)
        gdecay = torch.empty(B, H, G, D, dtype=torch.float32, device=q.device)
        o = torch.empty(B, T, H, D, dtype=q.dtype, device=q.device)
        final = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
        seed = None if init is None else init.float().contiguous()
        a = _gla_args(q, k, v, gf, scale, B, T, H, G, cpg, states, gdecay, o=o)
        _gla_launch(0, D, a)
        lasp = _LASP_CTX if init is None else None
        if lasp is not None:       # sequence split over ranks: exchange fused into the combine kernel
            lasp.combine(0, states, None, final, B * H, H, G, cpg, T, D, gdecay=gdecay, dmode=2)
        else:
            _gla_combine(0, states, gdecay, seed, final, B * H, G, D)
        _gla_launch(2, D, a)
        ctx.lasp = lasp
        ctx.save_for_backward(q, k, v, gf, states, gdecay, final)
        ctx.scale, ctx.grid, ctx.has_init, ctx.g_dtype = scale, (G, cpg), init is not None, gk.dtype
        return o, final

    @staticmethod
    def backward(ctx, d_o, dfinal):
        q, k, v, gf, states, gdecay, final = ctx.saved_tensors
        B, T, H, D = q.shape
        G, cpg = ctx.grid
        d_o = d_o.contiguous().to(q.dtype)
        dqkv = torch.empty(B, T, H, 3 * D, dtype=q.dtype, device=q.device)
        dq, dk, dv = dqkv[..., :D], dqkv[..., D:2 * D], dqkv[..., 2 * D:]
        dstates = torch.empty_like(states)
        dinit = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device) if ctx.has_init else None
        a = _gla_args(q, k, v, gf, ctx.scale, B, T, H, G, cpg, states, None, d_o=d_o, dq=dq)
        _gla_launch(3, D, a)
        a2 = _gla_args(q, k, v, gf, ctx.scale, B, T, H, G, cpg, dstates, None, d_o=d_o, dk=dk, dv=dv)
        _gla_launch(1, D, a2)
        seed = None if dfinal is None else dfinal.float().contiguous()
        if ctx.lasp is not None:
            r_out = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
            ctx.lasp.combine(1, dstates, None, None, B * H, H, G, cpg, T, D, gdecay=gdecay, dmode=2, r_out=r_out)
            dfinal = r_out         # gradient of the state leaving this rank, folded from the ranks after it
        else:
            _gla_combine(1, dstates, gdecay, seed, dinit, B * H, G, D)
        _gla_launch(4, D, a2)
        # d gk_t = sum_{i>=t} q_i . dq_i - sum_{j>=t} k_j . dk_j per channel (+ <S_T, dS_T> rows with a final-state gradient)
        # (the scan runs along the innermost dimension of a [B,H,D,T] copy: a scan over an outer dimension is ~10x slower)
        dg = _gla_dg(q, k, dq, dk)
        if dfinal is not None:
            dg = dg + (final * dfinal.float()).sum(-1)[:, None]
        return dq, dk, dv, dg.to(ctx.g_dtype), None, dinit


class _LsmVectorFused(torch.autograd.Function):
    """``_LsmVector`` with q|k|v given as one fused ``[B,T,H,3D]`` tensor: one gradient tensor, no concatenation."""

    @staticmethod
    def forward(ctx, qkv, gk, scale, init):
        D = qkv.shape[-1] // 3
        return _LsmVector.forward(ctx, qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:], gk, scale, init)

    @staticmethod
    def backward(ctx, d_o, dfinal):
        dq, dk, dv, dg, _, dinit = _LsmVector.backward(ctx, d_o, dfinal)
        return dq._base, dg, None, dinit


class _DgArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("q", "k", "dq", "dk")] +
                [(n, ctypes.c_int64) for n in ("qs_b", "qs_t", "qs_h", "ks_b", "ks_t", "ks_h", "dqs_b", "dqs_t", "dqs_h",
                                               "dks_b", "dks_t", "dks_h")] +
                [("dg", ctypes.c_void_p), ("segsum", ctypes.c_void_p)] +
                [(n, ctypes.c_int) for n in ("B", "T", "H", "D", "nseg")])


def _gla_dg(q, k, dq, dk):
    """Reverse cumulative sum over time of ``q*dq - k*dk`` per channel -> fp32 ``[B,T,H,D]`` (two kernel launches)."""
    B, T, H, D = q.shape
    dg = torch.empty(B, T, H, D, dtype=torch.float32, device=q.device)
    nseg = (T + 255) // 256
    seg = torch.empty(B * H, nseg, D, dtype=torch.float32, device=q.device)
    a = _DgArgs()
    for name, t in (("q", q), ("k", k), ("dq", dq), ("dk", dk)):
        setattr(a, name, t.data_ptr())
        setattr(a, name + "s_b", t.stride(0)), setattr(a, name + "s_t", t.stride(1)), setattr(a, name + "s_h", t.stride(2))
    a.dg, a.segsum = dg.data_ptr(), seg.data_ptr()
    a.B, a.T, a.H, a.D, a.nseg = B, T, H, D, nseg
    _check(lib().lmoe_gla_dg(ctypes.byref(a), _st()), "gla_dg", 2)
    return dg


_HALF_CHUNK_DECAY_LIMIT = -80.0     # the gated-scan kernels rescale bf16 operands by e^{+-(decay over half a chunk)}


def _note_strong_decay(gk):
    """Record (without a host synchronisation) whether some key channel decays by more than ``e^-80`` inside one half
    chunk of 32 tokens: beyond that the rescaled bf16 operands of ``csrc/lsm_vector.cu`` overflow.  The flag is the
    third element of the status word that the trainer reads every step; ``check_status`` raises on it."""
    from ..parallel import fused_comm
    B, T, H, D = gk.shape
    g = gk.detach().float()
    if T % 32:
        g = F.pad(g, (0, 0, 0, 0, 0, 32 - T % 32))
    worst = g.view(B, -1, 32, H, D).sum(2).amin()
    fused_comm.status_word(gk.device)[2:3] += (worst < _HALF_CHUNK_DECAY_LIMIT).to(torch.int32)


def _lsm_vector_bonus(q, k, v, gk, scale, initial_state, bonus, chunk_size):
    """RWKV6 on the key-channel-gated kernels: ``o_t = r_t (S_{t-1} + diag(u) k_t^T v_t)``.

    The kernels compute ``q_t S_t`` with ``S_t`` including token ``t``.  ``r_t S_{t-1}`` is what they return at position
    ``t - 1`` when the query there is ``r_t``, so the queries are shifted one position to the left, the outputs one to the
    right (position 0 reads the initial state), and the bonus term is a per-token dot product.  Nothing is subtracted,
    so strong decays lose no precision; autograd differentiates the shifts."""
    B, T, H, D = q.shape
    if T > 1:
        _note_strong_decay(gk)            # RWKV6 decays -exp(.) are not bounded the way GLA's normalised log-sigmoids are
    q_shift = torch.cat([q[:, 1:], q.new_zeros(B, 1, H, D)], 1)
    out_s, S = lsm_vector(q_shift, k, v, gk, scale, initial_state, None, chunk_size)
    if initial_state is None:
        first = out_s.new_zeros(B, 1, H, v.shape[-1])
    else:
        first = (scale * torch.einsum("bhk,bhkv->bhv", q[:, 0].float(), initial_state.float())).to(out_s.dtype)[:, None]
    o_state = torch.cat([first, out_s[:, :-1]], 1)
    diag = (q.float() * k.float() * bonus.float()[None, None]).sum(-1, keepdim=True) * scale
    return o_state + (diag * v.float()).to(o_state.dtype), S


def lsm_vector(q, k, v, gk, scale, initial_state, bonus, chunk_size):
    D = q.shape[-1]
    ok = (q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype
          and v.shape[-1] == D and k.shape[-1] == D and D in (64, 128))
    if not ok:
        return LT.chunk_vector_gated(q, k, v, gk, scale, initial_state, 16, bonus)
    scale = D ** -0.5 if scale is None else scale
    if bonus is not None:
        # RWKV6.  Forward-only calls (evaluation, prefill, generation) run on the kernels.  With gradients the default is
        # the fp32 16-token torch form: the kernels' decay gradient is a reverse cumulative sum of q.dq - k.dk over bf16
        # dq / dk, accurate to a few per cent per element, which is not enough for RWKV6's slowly decaying channels (the
        # gradient of the decay projection came out with a cosine of 0.7 against the fp32 form on a small model).
        # LMOE_RWKV6_KERNEL=1 forces the kernels for training too, =0 forces the torch form everywhere.
        mode = os.environ.get("LMOE_RWKV6_KERNEL", "auto")
        needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, gk, bonus, initial_state))
        if mode == "0" or (mode != "1" and needs_grad):
            return LT.chunk_vector_gated(q, k, v, gk, scale, initial_state, 16, bonus)
        return _lsm_vector_bonus(q, k, v, gk, scale, initial_state, bonus, chunk_size)
    if q.shape[1] == 1 and not (torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, gk))):
        return _lsm_step(q, k, v, None, gk, scale, initial_state)
    base = _fused_base(q, k, v)
    if base is not None:
        return _LsmVectorFused.apply(base, gk, scale, initial_state)
    return _LsmVector.apply(q, k, v, gk, scale, initial_state)


class _tf32:
    """fp32 matmuls on the tensor cores (TF32) inside the block."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


class _DeltaArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("W", "U", "Qd", "Kd", "A", "gamma", "S0", "dO", "dSfinal", "O", "Vn", "Sn",
                                                 "Sfinal", "dVn", "dSn", "dS0")] + [("N", ctypes.c_int), ("dv", ctypes.c_int)])


def _delta_prepare(q, k, v, beta, g, scale, C=64):
    """State-independent tiles of the chunked (gated) delta rule (WY / UT transform), chunk-parallel, differentiable:
    ``W, U, Qd, Kd`` ``[B,H,N,C,d]``, ``A`` ``[B,H,N,C,C]`` in bf16 and ``gamma`` ``[B,H,N]`` fp32 (see csrc/lsm_delta.cu)."""
    B, T, H, dk = q.shape
    f = torch.float32
    N = (T + C - 1) // C
    pad = N * C - T

    def chunks(x):                                   # [B,T,H,...] -> [B,H,N,C,...]
        x = x.to(f)
        if pad:
            x = F.pad(x, (0, 0) * (x.dim() - 2) + (0, pad))
        x = x.reshape(B, N, C, *x.shape[2:])
        return x.permute(0, 3, 1, 2, *range(4, x.dim())).contiguous()
    qc, kc, vc = chunks(q), chunks(k), chunks(v)
    bc = chunks(beta)                                                           # [B,H,N,C]
    if g is None:
        b = torch.zeros_like(bc)
    else:
        b = chunks(g).cumsum(-1)
    tril = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    L = torch.where(tril, b[..., :, None] - b[..., None, :], torch.full((), float("-inf"), device=q.device)).exp()
    A_ = ((kc @ kc.transpose(-1, -2)) * L * bc[..., None]).tril(-1)
    eb = b.exp()
    rhs = torch.cat([vc * bc[..., None], kc * (bc * eb)[..., None]], dim=-1)
    eye = torch.eye(C, dtype=f, device=q.device)
    sol = torch.linalg.solve_triangular(eye + A_, rhs, upper=False, unitriangular=True)
    dv = v.shape[-1]
    U, W = sol[..., :dv], sol[..., dv:]
    qs = qc * scale
    Aqk = (qs @ kc.transpose(-1, -2)) * L
    btot = b[..., -1]
    Qd = qs * eb[..., None]
    Kd = kc * (btot[..., None] - b).exp()[..., None]
    # row-major tiles for the kernels: the triangular solve may return its result in column-major order, and a dtype
    # conversion keeps whatever dense layout it is given
    bf = torch.bfloat16
    return (W.to(bf).contiguous(), U.to(bf).contiguous(), Qd.to(bf).contiguous(), Kd.to(bf).contiguous(),
            Aqk.to(bf).contiguous(), btot.exp().contiguous())


class _DeltaPrepArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("q", "k", "v")] +
                [(n, ctypes.c_longlong) for n in ("qs_b", "qs_t", "qs_h", "ks_b", "ks_t", "ks_h", "vs_b", "vs_t", "vs_h")] +
                [(n, ctypes.c_void_p) for n in ("beta", "g", "W", "U", "Qd", "Kd", "A", "gamma")] +
                [(n, ctypes.c_int) for n in ("B", "T", "H", "N")] + [("scale", ctypes.c_float)])


def _delta_prepare_kernel(q, k, v, beta, g, scale, C=64):
    """The tiles of :func:`_delta_prepare` from one chunk-parallel kernel (``delta_prep_fwd_kernel``, csrc/lsm_delta.cu):
    K K^T, the triangular inverse (forward substitution in registers), W, U, Q K^T and the decay-scaled copies of Q, K.
    No autograd: used by the forward pass, which keeps only the inputs."""
    B, T, H, D = q.shape
    N = (T + C - 1) // C
    q, k, v = _inner_contig(q), _inner_contig(k), _inner_contig(v)
    bf, dev = torch.bfloat16, q.device
    W, U, Qd, Kd = (torch.empty(B, H, N, C, D, dtype=bf, device=dev) for _ in range(4))
    A = torch.empty(B, H, N, C, C, dtype=bf, device=dev)
    gamma = torch.empty(B, H, N, dtype=torch.float32, device=dev)
    bt = beta.float().contiguous()
    gt = None if g is None else g.float().contiguous()
    a = _DeltaPrepArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.qs_b, a.qs_t, a.qs_h = q.stride(0), q.stride(1), q.stride(2)
    a.ks_b, a.ks_t, a.ks_h = k.stride(0), k.stride(1), k.stride(2)
    a.vs_b, a.vs_t, a.vs_h = v.stride(0), v.stride(1), v.stride(2)
    a.beta, a.g = bt.data_ptr(), 0 if gt is None else gt.data_ptr()
    a.W, a.U, a.Qd, a.Kd, a.A, a.gamma = (t.data_ptr() for t in (W, U, Qd, Kd, A, gamma))
    a.B, a.T, a.H, a.N, a.scale = B, T, H, N, float(scale)
    _check(lib().lmoe_delta_prepare(_i32(D), ctypes.byref(a), _st()), "delta_prepare")
    return W, U, Qd, Kd, A, gamma


def _delta_scan_fwd(W, U, Qd, Kd, A, gamma, S0):
    """``delta_scan_fwd_kernel``: ``Vn = U - W S``, ``O = Qd S + A Vn``, ``S' = gamma S + Kd^T Vn`` over the chunks.
    Returns ``O, Vn`` ``[B,H,N,C,dv]`` bf16, the state entering every chunk ``Sn`` ``[B,H,N,dk,dv]`` bf16 and the final
    state in fp32."""
    B, H, N, C, dk = W.shape
    dv = U.shape[-1]
    dev = W.device
    bf = torch.bfloat16
    O = torch.empty(B, H, N, C, dv, dtype=bf, device=dev)
    Vn = torch.empty(B, H, N, C, dv, dtype=bf, device=dev)
    Sn = torch.empty(B, H, N, dk, dv, dtype=bf, device=dev)
    Sf = torch.empty(B, H, dk, dv, dtype=torch.float32, device=dev)
    s0 = None if S0 is None else S0.float().contiguous()
    a = _DeltaArgs()
    a.W, a.U, a.Qd, a.Kd, a.A, a.gamma = (t.data_ptr() for t in (W, U, Qd, Kd, A, gamma))
    a.S0 = 0 if s0 is None else s0.data_ptr()
    a.O, a.Vn, a.Sn, a.Sfinal = O.data_ptr(), Vn.data_ptr(), Sn.data_ptr(), Sf.data_ptr()
    a.N, a.dv = N, dv
    _check(lib().lmoe_delta_scan(_i32(0), _i32(dk), _i32(B * H), ctypes.byref(a), _st()), "delta_scan_fwd")
    return O, Vn, Sn, Sf


def _delta_scan_bwd(W, Qd, Kd, A, gamma, dO, dSf):
    """``delta_scan_bwd_kernel``: the reverse recurrence ``dVn = A^T dO + Kd dS'``, ``dS = gamma dS' + Qd^T dO - W^T dVn``.
    Returns ``dVn`` ``[B,H,N,C,dv]``, the gradient of the state leaving every chunk ``dSn`` ``[B,H,N,dk,dv]`` (bf16) and the
    gradient of the initial state (fp32)."""
    B, H, N, C, dk = W.shape
    dv = dO.shape[-1]
    dev = W.device
    bf = torch.bfloat16
    dVn = torch.empty(B, H, N, C, dv, dtype=bf, device=dev)
    dSn = torch.empty(B, H, N, dk, dv, dtype=bf, device=dev)
    dS0 = torch.empty(B, H, dk, dv, dtype=torch.float32, device=dev)
    dsf = None if dSf is None else dSf.float().contiguous()
    a = _DeltaArgs()
    a.W, a.Qd, a.Kd, a.A, a.gamma = (t.data_ptr() for t in (W, Qd, Kd, A, gamma))
    a.U = 0
    a.dO, a.dSfinal = dO.data_ptr(), 0 if dsf is None else dsf.data_ptr()
    a.dVn, a.dSn, a.dS0 = dVn.data_ptr(), dSn.data_ptr(), dS0.data_ptr()
    a.N, a.dv = N, dv
    _check(lib().lmoe_delta_scan(_i32(1), _i32(dk), _i32(B * H), ctypes.byref(a), _st()), "delta_scan_bwd")
    return dVn, dSn, dS0


class _DeltaChunkScan(torch.autograd.Function):
    """The recurrence over chunks of the (gated) delta rule on the kernels of ``csrc/lsm_delta.cu`` as an autograd node over
    the tiles.  Backward: the reverse state-gradient recurrence is the second kernel; the gradients of the tiles are
    chunk-parallel products of what the two kernels wrote."""

    @staticmethod
    def forward(ctx, W, U, Qd, Kd, A, gamma, S0):
        W, U, Qd, Kd, A, gamma = (t.contiguous() for t in (W, U, Qd, Kd, A, gamma))
        O, Vn, Sn, Sf = _delta_scan_fwd(W, U, Qd, Kd, A, gamma, S0)
        ctx.save_for_backward(W, Qd, Kd, A, gamma, Vn, Sn)
        ctx.has_s0 = S0 is not None
        return O, Sf

    @staticmethod
    def backward(ctx, dO, dSf):
        W, Qd, Kd, A, gamma, Vn, Sn = ctx.saved_tensors
        dO = dO.to(torch.bfloat16).contiguous()
        dVn, dSn, dS0 = _delta_scan_bwd(W, Qd, Kd, A, gamma, dO, dSf)
        SnT = Sn.transpose(-1, -2)
        dW = -(dVn @ SnT)
        dQd = dO @ SnT
        dA = (dO @ Vn.transpose(-1, -2)).tril()
        dKd = Vn @ dSn.transpose(-1, -2)
        dgamma = (dSn.float() * Sn.float()).sum((-1, -2))
        return dW, dVn, dQd, dKd, dA, dgamma, (dS0 if ctx.has_s0 else None)


class _DeltaPrepBwdArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("q", "k", "v")] +
                [(n, ctypes.c_longlong) for n in ("qs_b", "qs_t", "qs_h", "ks_b", "ks_t", "ks_h", "vs_b", "vs_t", "vs_h")] +
                [(n, ctypes.c_void_p) for n in ("beta", "g", "Sn", "dSn", "Vn", "dVn", "dO", "dq", "dk", "dv", "dbeta", "dg")] +
                [(n, ctypes.c_int) for n in ("B", "T", "H", "N")] + [("scale", ctypes.c_float)])


def _delta_prepare_bwd_kernel(q, k, v, beta, g, scale, Sn, dSn, Vn, dVn, dO):
    """Gradients of ``q, k, v, beta, g`` from what the two scan kernels wrote, one chunk-parallel kernel
    (``delta_prep_bwd_kernel``, csrc/lsm_delta.cu): the chunk-local scan equations, ``W = T Kb`` / ``U = T Vb``, the
    triangular inverse and the decay factors are differentiated in shared memory on the tensor cores."""
    B, T, H, D = q.shape
    N = Sn.shape[2]
    q, k, v = _inner_contig(q), _inner_contig(k), _inner_contig(v)
    dev = q.device
    dq, dk, dv = (torch.empty(B, T, H, D, dtype=torch.bfloat16, device=dev) for _ in range(3))
    dbeta = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    dg = None if g is None else torch.empty(B, T, H, dtype=torch.float32, device=dev)
    bt = beta.float().contiguous()
    gt = None if g is None else g.float().contiguous()
    a = _DeltaPrepBwdArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.qs_b, a.qs_t, a.qs_h = q.stride(0), q.stride(1), q.stride(2)
    a.ks_b, a.ks_t, a.ks_h = k.stride(0), k.stride(1), k.stride(2)
    a.vs_b, a.vs_t, a.vs_h = v.stride(0), v.stride(1), v.stride(2)
    a.beta, a.g = bt.data_ptr(), 0 if gt is None else gt.data_ptr()
    a.Sn, a.dSn, a.Vn, a.dVn, a.dO = (t.data_ptr() for t in (Sn, dSn, Vn, dVn, dO))
    a.dq, a.dk, a.dv, a.dbeta = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dbeta.data_ptr()
    a.dg = 0 if dg is None else dg.data_ptr()
    a.B, a.T, a.H, a.N, a.scale = B, T, H, N, float(scale)
    _check(lib().lmoe_delta_prepare_bwd(_i32(D), ctypes.byref(a), _st()), "delta_prepare_bwd")
    return dq, dk, dv, dbeta, dg


class _DeltaRuleScan(torch.autograd.Function):
    """(Gated) delta rule on the kernels of ``csrc/lsm_delta.cu``.  Forward: the chunk-parallel WY / UT tile kernel, then the
    scan kernel.  Only the inputs are kept.  Backward (bf16, equal key / value widths): tiles and forward scan again, the
    reverse scan, then the chunk-parallel tile-gradient kernel (``_delta_backward_kernels``).  Other dtypes / widths build
    the tiles with torch ops and differentiate that construction with autograd around the two scan kernels."""

    @staticmethod
    def forward(ctx, q, k, v, beta, g, initial_state, scale, chunk_size):
        B, T, H, dk = q.shape
        scale = dk ** -0.5 if scale is None else scale
        with torch.no_grad(), _tf32():
            ctx.kernel_tiles = (q.dtype == k.dtype == v.dtype == torch.bfloat16 and v.shape[-1] == dk
                                and os.environ.get("LMOE_DELTA_PREP_KERNEL", "1") != "0")
            if ctx.kernel_tiles:
                tiles = _delta_prepare_kernel(q, k, v, beta, g, scale)
            else:
                tiles = _delta_prepare(q, k, v, beta, g, scale)
            O, S = _DeltaChunkScan.apply(*tiles, initial_state)
        ctx.save_for_backward(q, k, v, beta, g, initial_state)
        ctx.scale = scale
        o = O.permute(0, 2, 3, 1, 4).reshape(B, -1, H, v.shape[-1])[:, :T]
        return o.to(q.dtype), S

    @staticmethod
    def backward(ctx, do, dS):
        saved = ctx.saved_tensors
        if ctx.kernel_tiles and os.environ.get("LMOE_DELTA_PREP_BWD_KERNEL", "1") != "0":
            return _DeltaRuleScan._backward_kernels(ctx, do, dS)
        ins = [None if t is None else t.detach().requires_grad_(t.is_floating_point()) for t in saved]
        q = ins[0]
        B, T, H, dk = q.shape
        with torch.enable_grad(), _tf32():
            tiles = _delta_prepare(*ins[:5], ctx.scale)
            O, S = _DeltaChunkScan.apply(*tiles, ins[5])
            N, C = O.shape[2], O.shape[3]
            dO = do.to(O.dtype)
            if N * C != T:
                dO = F.pad(dO, (0, 0, 0, 0, 0, N * C - T))
            dO = dO.reshape(B, N, C, H, -1).permute(0, 3, 1, 2, 4)
            outs, gouts = [O], [dO]
            if dS is not None:
                outs.append(S)
                gouts.append(dS)
            need = [t for t in ins if t is not None]
            grads = torch.autograd.grad(outs, need, gouts, allow_unused=True)
        it = iter(grads)
        full = [None if t is None else next(it) for t in ins]
        full = [None if gr is None else gr.to(t.dtype) for gr, t in zip(full, ins)]
        return (*full, None, None)


def _delta_backward_kernels(ctx, do, dS):
    """Backward of the (gated) delta rule on kernels only: rebuild the tiles, rerun the forward scan for ``Vn`` and the
    entering states, run the reverse scan, then one chunk-parallel kernel for every input gradient."""
    q, k, v, beta, g, s0 = ctx.saved_tensors
    B, T, H, D = q.shape
    with torch.no_grad():
        W, U, Qd, Kd, A, gamma = _delta_prepare_kernel(q, k, v, beta, g, ctx.scale)
        N, C = W.shape[2], W.shape[3]
        _, Vn, Sn, _ = _delta_scan_fwd(W, U, Qd, Kd, A, gamma, s0)
        dO = do.to(torch.bfloat16)
        if N * C != T:
            dO = F.pad(dO, (0, 0, 0, 0, 0, N * C - T))
        dO = dO.reshape(B, N, C, H, D).permute(0, 3, 1, 2, 4).contiguous()
        dVn, dSn, dS0 = _delta_scan_bwd(W, Qd, Kd, A, gamma, dO, dS)
        dq, dk, dv, dbeta, dg = _delta_prepare_bwd_kernel(q, k, v, beta, g, ctx.scale, Sn, dSn, Vn, dVn, dO)
    need = ctx.needs_input_grad
    return (dq.to(q.dtype) if need[0] else None, dk.to(k.dtype) if need[1] else None, dv.to(v.dtype) if need[2] else None,
            dbeta.to(beta.dtype) if need[3] else None, (dg.to(g.dtype) if (g is not None and need[4]) else None),
            (dS0.to(s0.dtype) if (s0 is not None and need[5]) else None), None, None)


_DeltaRuleScan._backward_kernels = staticmethod(_delta_backward_kernels)


class _DeltaRuleTorch(torch.autograd.Function):
    """Eager form of the (gated) delta rule for shapes the scan kernels do not take (head dims other than 64 / 128, value
    width not a multiple of 32): batched matmuls with a parallel scan over the chunks' affine state maps."""

    @staticmethod
    def forward(ctx, q, k, v, beta, g, initial_state, scale, chunk_size):
        with torch.no_grad(), _tf32():
            o, S = LT.chunk_delta_rule(q, k, v, beta, g, scale, initial_state, chunk_size, parallel_scan=True)
        ctx.save_for_backward(q, k, v, beta, g, initial_state)
        ctx.cfg = (scale, chunk_size)
        return o.to(q.dtype), S

    @staticmethod
    def backward(ctx, do, dS):
        saved = ctx.saved_tensors
        ins = [None if t is None else t.detach().requires_grad_(t.is_floating_point()) for t in saved]
        with torch.enable_grad(), _tf32():
            o, S = LT.chunk_delta_rule(*ins[:5], ctx.cfg[0], ins[5], ctx.cfg[1], parallel_scan=True)
            outs, gouts = [o], [do.to(o.dtype)]
            if dS is not None:
                outs.append(S)
                gouts.append(dS)
            need = [t for t in ins if t is not None]
            grads = torch.autograd.grad(outs, need, gouts, allow_unused=True)
        it = iter(grads)
        full = [None if t is None else next(it) for t in ins]
        full = [None if gr is None else gr.to(t.dtype) for gr, t in zip(full, ins)]
        return (*full, None, None)


def lsm_delta(q, k, v, beta, g, scale, initial_state, chunk_size):
    D = q.shape[-1]
    if (q.shape[1] == 1 and q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype
            and k.shape[-1] == D and v.shape[-1] == D and D in (64, 128)
            and not (torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, beta, g)))):
        return _lsm_delta_step(q, k, v, beta, g, D ** -0.5 if scale is None else scale, initial_state)
    if q.is_cuda and D in (64, 128) and k.shape[-1] == D and v.shape[-1] % 32 == 0 and os.environ.get("LMOE_DELTA_KERNEL", "1") != "0":
        return _DeltaRuleScan.apply(q, k, v, beta, g, initial_state, scale, chunk_size)
    return _DeltaRuleTorch.apply(q, k, v, beta, g, initial_state, scale, chunk_size)


def _lsm_delta_step(q, k, v, beta, g, scale, initial_state):
    """Decoding: one token of the (gated) delta rule in one launch (csrc/lsm_step.cu).  beta, g: [B,1,H]."""
    B, _, H, D = q.shape
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    bf = beta.float().reshape(B, H).contiguous()
    gf = None if g is None else g.float().reshape(B, H).contiguous()
    s_in = None if initial_state is None else initial_state.float().contiguous()
    s_out = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
    o = torch.empty(B, 1, H, D, dtype=q.dtype, device=q.device)
    ll = ctypes.c_longlong
    _check(lib().lmoe_lsm_delta_step(_p(q), _p(k), _p(v), ll(q.stride(0)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(2)),
                                     ll(v.stride(0)), ll(v.stride(2)), _p(gf), _p(bf), _p(s_in), _p(s_out), _p(o), ctypes.c_int(B),
                                     ctypes.c_int(H), ctypes.c_int(D), ctypes.c_float(scale), _st()), "lsm_delta_step")
    return o, s_out

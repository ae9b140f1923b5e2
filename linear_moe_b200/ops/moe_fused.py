"""MoE layer core with the expert-parallel exchange done by this framework's peer-memory kernels
(``csrc/moe_comm.cu``) and the expert MLPs by the grouped tcgen05 GEMM (``csrc/gemm_grouped.cu``).

Data flow of :func:`fused_moe` (replaces token_dispatcher.py:412-548 + experts.py:156-168 of the reference)::

    idx --route--> (dest rank, dest row) per (token, slot); padded expert offsets      [device only]
    h   --push---> owner ranks' receive buffers --grouped fc1 + SwiGLU + grouped fc2--> result buffers
    out <--pull--- sum_k prob[t,k] * result row (t,k)                                   [un-permute fused]

The backward pass is the mirror image: the gradient of the combine pushes ``prob * d_out`` rows to the owners, the
gradient of the dispatch pulls and sums the ``k`` input-gradient rows of every token.
"""
from __future__ import annotations

import torch

from . import gemm


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, ws, route):
        ctx.ws, ctx.route = ws, route
        return ws.push(h.contiguous(), route, None)

    @staticmethod
    def backward(ctx, d_recv):
        dh, _ = ctx.ws.pull(d_recv, ctx.route, None, False)
        return dh, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_local, probs, ws, route):
        w = probs.float().contiguous()
        out, rows = ws.pull(y_local, route, w, True)
        ctx.ws, ctx.route = ws, route
        ctx.save_for_backward(rows, w)
        ctx.pdtype = probs.dtype
        return out

    @staticmethod
    def backward(ctx, d_out):
        rows, w = ctx.saved_tensors
        route = ctx.route
        d_out = d_out.contiguous()
        T, k = route.T, route.k
        from . import cuda as K
        d_probs = K.moe_dprobs(rows, d_out, route.dest_rank, T, k)
        d_y = ctx.ws.push(d_out, route, w.reshape(-1), keep=False)
        return d_y, d_probs.to(ctx.pdtype), None, None


def fused_moe(h: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, ws) -> torch.Tensor:
    """``h [T, hid]`` bf16, ``probs/idx [T, k]``, local expert weights ``w1 [El, hid, 2f]``, ``w2 [El, f, hid]``."""
    from . import cuda as K
    route = ws.route(idx)
    xr = _Dispatch.apply(h, ws, route)
    # between ranks, the second GEMM writes its result, and the first GEMM's backward its input gradient, straight into
    # the buffer the peers pull from (no copy into it)
    res = ws.result_holder()
    y1 = gemm.GroupedLinear.apply(xr, w1, route.offs, None, res)
    act = K.swiglu(y1)
    y2 = gemm.GroupedLinear.apply(act, w2, route.offs, res, None)
    return _Combine.apply(y2, probs, ws, route)

"""LASP-2 sequence parallelism for every linear sequence model.

Each rank of the context-parallel group holds a contiguous slice of the sequence.  A linear
sequence model is an affine recurrence on the memory state, so a rank's whole slice acts on
the entering state ``P`` as ``S_out = A_r(P) + M_r`` where ``M_r`` is the state the slice
produces from zero and ``A_r`` is a per-head decay (scalar or per key channel) or, for the
delta-rule families, a ``dk x dk`` matrix.  LASP-2 therefore needs ONE exchange per layer
and direction: every rank computes ``(M_r, A_r)`` locally, the summaries are all-gathered,
each rank folds the summaries of the ranks before it into its entering state and then runs
its slice again with that state.

The reference implements this only for undecayed linear attention, drops the intra-block
term and uses NCCL ``all_gather_into_tensor`` (lasp2_without_mask_triton_op.py:673-750,
lasp2.py:62-79).  This module is the general algorithm, written on differentiable
collectives so that autograd produces the mirrored backward (gather of state gradients,
suffix combine).  On CUDA the scalar-decay family (constant or data-dependent decay) and the
key-channel-gated family take the fused paths ``ops.cuda.lasp2_scalar`` / ``lasp2_vector`` instead,
where the exchange happens inside the combine kernel through peer memory; the delta-rule
families and RWKV7's diagonal-plus-low-rank transition (``dk x dk`` matrices) use the form below.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from ..dist import collectives as C
from ..dist.mesh import Group
from ..ops import lsm_torch as LT


def _summaries(kind: str, q, k, v, g, gk, beta, scale, chunk_size, bonus, dplr=None):
    """Local state from zero ``M`` and transition ``A`` of this rank's slice."""
    B, T, H, dk = k.shape
    if kind == "value":
        # decay per value channel (first pass of gated slot attention): S_t = S_{t-1} diag(e^{gv_t}) + k_t^T v_t
        _, M = LT.chunk_value_gated(q, k, v, gk, scale, None)
        return M, gk.float().sum(1).exp()
    if kind == "dplr":
        # RWKV7: S_t = (diag(e^{w_t}) + b_t a_t^T) S_{t-1} + k_t v_t^T; the slice's transition is the product of the
        # per-token matrices, read off by sending the identity through the recurrence with zero values
        a, b = dplr
        sc = 1.0 if scale is None else scale
        _, M = ops.lsm_dplr(q, gk, k, v, a, b, sc, None)
        eye = torch.eye(dk, dtype=torch.float32, device=k.device).expand(B, H, dk, dk)
        zeros = torch.zeros(B, T, H, dk, dtype=v.dtype, device=v.device)
        _, A = ops.lsm_dplr(q, gk, k, zeros, a, b, sc, eye)
        return M, A
    if kind == "scalar":
        _, M = ops.lsm_scalar(q, k, v, g, scale, None, chunk_size)
        if g is None:
            A = None
        elif g.dim() == 1:
            A = (g.float() * T).exp()[None, :].expand(B, H)
        else:
            A = g.float().sum(1).exp()
        return M, A
    if kind == "vector":
        _, M = ops.lsm_vector(q, k, v, gk, scale, None, bonus, chunk_size)
        return M, gk.float().sum(1).exp()
    if kind == "delta":
        _, M = ops.lsm_delta(q, k, v, beta, g, scale, None, chunk_size)
        eye = torch.eye(dk, dtype=torch.float32, device=k.device).expand(B, H, dk, dk)
        zeros = torch.zeros(B, T, H, dk, dtype=v.dtype, device=v.device)
        _, A = ops.lsm_delta(q, k, zeros, beta, g, scale, eye, chunk_size)
        return M, A
    raise ValueError(kind)


def _apply(kind: str, A, P):
    if A is None:
        return P
    if kind == "scalar":
        return P * A[..., None, None]
    if kind == "vector":
        return P * A[..., None]
    if kind == "value":
        return P * A[..., None, :]
    return A @ P                       # delta rule and DPLR: a dk x dk matrix per head


def _recurrent(kind, q, k, v, g, gk, beta, scale, init, bonus):
    """``--la-mode fused_recurrent``: the token-by-token recurrence (exact, O(T) sequential steps)."""
    from ..ref import lsm as RL
    B, T, H, _ = q.shape
    if bonus is not None:
        # RWKV6: the output reads the state BEFORE the current token is written and adds the token's own contribution
        # weighted by the bonus u: o_t = q_t S_{t-1} + (q_t . (u * k_t)) v_t
        f = torch.float32
        sc = q.shape[-1] ** -0.5 if scale is None else scale
        qf, kf, vf, w = q.to(f) * sc, k.to(f), v.to(f), gk.to(f).exp()
        S = torch.zeros(B, H, q.shape[-1], v.shape[-1], dtype=f, device=q.device) if init is None else init.to(f)
        own = (qf * bonus.to(f)[None, None] * kf).sum(-1, keepdim=True) * vf
        outs = []
        for t in range(T):
            outs.append(torch.einsum("bhk,bhkv->bhv", qf[:, t], S) + own[:, t])
            S = S * w[:, t][..., None] + kf[:, t][..., None] * vf[:, t][..., None, :]
        return torch.stack(outs, 1).to(v.dtype), S
    gg = g if (g is None or g.dim() == 3) else g[None, None, :].expand(B, T, H)
    o, S = RL.recurrent_lsm(q, k, v, g=gg, gk=gk, beta=beta, scale=scale, initial_state=init)
    return o.to(v.dtype), S


def _parallel(kind, q, k, v, g, scale, init):
    """``--la-mode parallel``: the quadratic (attention-like) form ``o = ((Q K^T) . decay mask) V`` of the scalar-decay
    family; the final state is one extra weighted sum."""
    if kind != "scalar" or init is not None:
        raise ValueError("--la-mode parallel exists for the scalar-decay family without an initial state only")
    B, T, H, dk = q.shape
    f = torch.float32
    scale = dk ** -0.5 if scale is None else scale
    if g is None:
        b = torch.zeros(B, T, H, dtype=f, device=q.device)
    elif g.dim() == 1:
        b = g.to(f)[None, None, :] * torch.arange(1, T + 1, device=q.device, dtype=f)[None, :, None]
    else:
        b = g.to(f).cumsum(1)
    bt = b.permute(0, 2, 1)                                                  # [B,H,T]
    diff = bt[..., :, None] - bt[..., None, :]
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    dec = torch.where(mask, diff, torch.full((), float("-inf"), device=q.device)).exp()
    s = torch.einsum("bihd,bjhd->bhij", q.to(f) * scale, k.to(f)) * dec
    o = torch.einsum("bhij,bjhd->bihd", s, v.to(f))
    kd = k.to(f) * (bt[..., -1:] - bt).exp().permute(0, 2, 1)[..., None]
    S = torch.einsum("bjhk,bjhv->bhkv", kd, v.to(f))
    return o.to(v.dtype), S


def lasp2(kind: str, q, k, v, *, group: Group, g=None, gk=None, beta=None, scale=None,
          chunk_size: int = 64, bonus=None, initial_state=None, mode: str = "chunk",
          dplr=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Run a linear sequence model whose sequence is split over ``group`` (rank order = sequence
    order).  ``kind``: ``scalar`` | ``vector`` | ``value`` (``gk`` = log decay per value channel) | ``delta`` | ``dplr`` (RWKV7: ``q`` = receptance, ``gk`` = log decay,
    ``dplr = (a, b)`` the low-rank factors of the transition).  Returns the local output and the state
    after this rank's slice.  ``mode`` (``--la-mode``): ``chunk`` / ``fused_chunk`` = the chunked kernels (one fused
    implementation serves both names), ``fused_recurrent`` = token recurrence, ``parallel`` = quadratic form."""
    if mode not in ("chunk", "fused_chunk", "fused_recurrent", "parallel"):
        raise ValueError(f"unknown --la-mode {mode!r}")

    def run(init):
        if kind == "value":
            return LT.chunk_value_gated(q, k, v, gk, scale, init)
        if kind == "dplr":
            return ops.lsm_dplr(q, gk, k, v, dplr[0], dplr[1], 1.0 if scale is None else scale, init)
        if mode == "fused_recurrent":
            return _recurrent(kind, q, k, v, g, gk, beta, scale, init, bonus)
        if mode == "parallel":
            return _parallel(kind, q, k, v, g, scale, init)
        if kind == "scalar":
            return ops.lsm_scalar(q, k, v, g, scale, init, chunk_size)
        if kind == "vector":
            return ops.lsm_vector(q, k, v, gk, scale, init, bonus, chunk_size)
        return ops.lsm_delta(q, k, v, beta, g, scale, init, chunk_size)

    if group.is_trivial:
        return run(initial_state)
    if mode == "parallel":
        raise ValueError("--la-mode parallel cannot be combined with sequence parallelism (the quadratic form has no state)")
    if (q.is_cuda and kind == "scalar" and initial_state is None and mode != "fused_recurrent"
            and ops._K().fused_lasp_available(group, q, k, v, g)):
        return ops._K().lasp2_scalar(q, k, v, g, scale, group, chunk_size)
    if (q.is_cuda and kind == "vector" and bonus is None and initial_state is None and mode != "fused_recurrent"
            and ops._K().fused_lasp_available(group, q, k, v, None)):
        return ops._K().lasp2_vector(q, k, v, gk, scale, group, chunk_size)

    M, A = _summaries(kind, q, k, v, g, gk, beta, scale, chunk_size, bonus, dplr)
    W, r = group.size, group.rank
    allM = C.all_gather(M[None].contiguous(), group, dim=0)                 # [W, B, H, dk, dv]
    allA = None if A is None else C.all_gather(A[None].contiguous(), group, dim=0)
    P = torch.zeros_like(M) if initial_state is None else initial_state.float()
    for j in range(r):
        P = _apply(kind, None if allA is None else allA[j], P) + allM[j]
    # Every rank must reach the backward collective of the two gathers, also the ranks whose
    # entering state uses none (rank 0) or only some of the gathered summaries.
    P = P + 0.0 * allM.sum(0)
    if allA is not None:
        P = P + 0.0 * allA.sum().to(P.dtype)
    return run(P)

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
suffix combine).  On CUDA the scalar-decay family takes the fused path of
``ops.cuda.lasp2_scalar`` instead, where the exchange happens inside the scan kernels
through peer memory.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from ..dist import collectives as C
from ..dist.mesh import Group


def _summaries(kind: str, q, k, v, g, gk, beta, scale, chunk_size, bonus):
    """Local state from zero ``M`` and transition ``A`` of this rank's slice."""
    B, T, H, dk = k.shape
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
    return A @ P


def lasp2(kind: str, q, k, v, *, group: Group, g=None, gk=None, beta=None, scale=None,
          chunk_size: int = 64, bonus=None, initial_state=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Run a linear sequence model whose sequence is split over ``group`` (rank order = sequence
    order).  ``kind``: ``scalar`` | ``vector`` | ``delta``.  Returns the local output and the state
    after this rank's slice."""
    def run(init):
        if kind == "scalar":
            return ops.lsm_scalar(q, k, v, g, scale, init, chunk_size)
        if kind == "vector":
            return ops.lsm_vector(q, k, v, gk, scale, init, bonus, chunk_size)
        return ops.lsm_delta(q, k, v, beta, g, scale, init, chunk_size)

    if group.is_trivial:
        return run(initial_state)
    if q.is_cuda and kind == "scalar" and initial_state is None and ops._K().fused_lasp_available(group, q, k, v, g):
        return ops._K().lasp2_scalar(q, k, v, g, scale, group, chunk_size)

    M, A = _summaries(kind, q, k, v, g, gk, beta, scale, chunk_size, bonus)
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

"""Scalar-decay linear attention for feature / value widths the scan kernels have no instantiation for.

The kernels of ``csrc/lsm_scalar.cu`` exist for square states of width 64 and 128.  Based and Rebased expand 16 query /
key channels to 153 Taylor or quadratic features (reference ``sequence_modeling/based/based.py:69-72``,
``rebased/rebased.py``), and the normalised forms divide by ``q . sum k``, which is one more value column
(``linear_attention/linear_attention.py`` with ``do_feature_map_norm``).  Both fit the kernels once two facts are used:

* ``o = ((Q K^T) . mask) V`` and ``S = K^T V`` are additive over a partition of the feature dimension and separate
  per value column, so a ``[F, Dv]`` problem is the sum over 128-wide key blocks of independent ``[128, 128]`` problems,
  one per value block (zero padding of either side contributes nothing);
* a remainder of a few value columns without decay (the column of ones of the normaliser) needs no ``T x T`` work at
  all: ``o_t[c] = q_t . (S0[:, c] + sum_{s<=t} k_s v_s[c])`` is a cumulative sum over the sequence.

``inner`` is the square-state implementation (the kernel dispatch on CUDA, any reference on CPU), so the same
composition is what the CPU tests check against the unblocked definition.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.nn.functional as F

NARROW_MAX = 4          # value remainders up to this many columns take the cumulative-sum form (no decay only)


def narrow_columns(q, k, vn, scale: float, s0n: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Undecayed linear attention for a handful of value columns as cumulative sums (fp32).

    q, k ``[B,T,H,F]``; vn ``[B,T,H,r]``; s0n ``[B,H,F,r]`` or None.  Returns ``o [B,T,H,r]`` (fp32) and the state
    ``[B,H,F,r]`` after the last token."""
    qf, kf = q.float(), k.float()
    cols, states = [], []
    for c in range(vn.shape[-1]):
        kv = (kf * vn[..., c:c + 1].float()).cumsum(1)                       # [B,T,H,F]
        if s0n is not None:
            kv = kv + s0n[..., c].float()[:, None]
        cols.append((qf * kv).sum(-1) * scale)
        states.append(kv[:, -1])
    return torch.stack(cols, -1), torch.stack(states, -1)


def blocked_scalar(inner: Callable, q, k, v, g, scale: Optional[float], initial_state, chunk_size: int,
                   width: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``inner(q, k, v, g, scale, initial_state, chunk_size) -> (o, S)`` for square ``width``-wide blocks, composed to
    feature width ``F`` and value width ``Dv`` of any size.  Returns ``o [B,T,H,Dv]`` in v's dtype and ``S [B,H,F,Dv]``
    fp32."""
    Fd, Dv = q.shape[-1], v.shape[-1]
    if width is None:
        width = 64 if max(Fd, Dv) <= 64 else 128
    W = width
    scale = Fd ** -0.5 if scale is None else scale
    nf = -(-Fd // W)
    full, rem = divmod(Dv, W)
    narrow = rem if (g is None and 0 < rem <= NARROW_MAX and full > 0) else 0
    nv = full + (1 if (rem and not narrow) else 0)
    qp = F.pad(q, (0, nf * W - Fd)) if nf * W != Fd else q
    kp = F.pad(k, (0, nf * W - Fd)) if nf * W != Fd else k
    wide = Dv - narrow
    vp = v[..., :wide]
    if nv * W != wide:
        vp = F.pad(vp, (0, nv * W - wide))
    s0 = None
    if initial_state is not None:
        s0 = F.pad(initial_state[..., :wide].float(), (0, nv * W - wide, 0, nf * W - Fd))
    outs, cols = [], []
    for j in range(nv):
        vj = vp[..., j * W:(j + 1) * W]
        acc, rows = None, []
        for i in range(nf):
            sij = None if s0 is None else s0[..., i * W:(i + 1) * W, j * W:(j + 1) * W]
            o_ij, S_ij = inner(qp[..., i * W:(i + 1) * W], kp[..., i * W:(i + 1) * W], vj, g, scale, sij, chunk_size)
            acc = o_ij.float() if acc is None else acc + o_ij.float()
            rows.append(S_ij.float())
        outs.append(acc)
        cols.append(torch.cat(rows, dim=-2))
    o = torch.cat(outs, dim=-1)[..., :wide]
    S = torch.cat(cols, dim=-1)[..., :Fd, :wide]
    if narrow:
        s0n = None if initial_state is None else initial_state[..., wide:]
        on, Sn = narrow_columns(q, k, v[..., wide:], scale, s0n)
        o, S = torch.cat([o, on], dim=-1), torch.cat([S, Sn], dim=-1)
    return o.to(v.dtype), S

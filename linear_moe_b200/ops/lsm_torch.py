"""Chunked linear-sequence-model operators in plain differentiable torch.

Used (a) on CPU tensors (tests, gloo runs), (b) as the eager comparator the CUDA
kernels are timed against, and (c) for the few families that have no CUDA kernel yet.
Every function computes in fp32 and returns ``(o, final_state)``; autograd provides the
backward.  The chunk algebra is the standard one: with ``b`` the in-chunk cumulative log
decay, ``O = ((Q e^{b})(K e^{-b})^T . mask) V + (Q e^{b}) S`` and
``S' = e^{b_C} S + (K e^{b_C - b})^T V``; the delta-rule families add the WY/UT transform
``T = (I + tril(diag(beta) K K^T . L, -1))^{-1} diag(beta)``.

Layout: q, k ``[B,T,H,dk]``, v ``[B,T,H,dv]``, state ``[B,H,dk,dv]``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def _pad_to_chunks(x: torch.Tensor, C: int, value: float = 0.0):
    T = x.shape[1]
    pad = (-T) % C
    if pad:
        shp = list(x.shape)
        shp[1] = pad
        x = torch.cat([x, x.new_full(shp, value)], dim=1)
    return x, pad


def _chunk(x: torch.Tensor, C: int) -> torch.Tensor:
    B, T = x.shape[:2]
    return x.reshape(B, T // C, C, *x.shape[2:])


def chunk_scalar_gated(q, k, v, g: Optional[torch.Tensor], scale: Optional[float] = None,
                       initial_state: Optional[torch.Tensor] = None, chunk_size: int = 64
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Linear attention with a scalar log decay per token and head.

    ``g``: ``[B,T,H]`` (per token), ``[H]`` (constant per head: retention, lightning) or
    ``None`` (no decay: basic linear attention)."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    C = min(chunk_size, max(T, 1))
    scale = dk ** -0.5 if scale is None else scale
    f = torch.float32
    if g is None:
        g = torch.zeros(B, T, H, dtype=f, device=q.device)
    elif g.dim() == 1:
        g = g.to(f)[None, None, :].expand(B, T, H)
    q, _ = _pad_to_chunks(q.to(f) * scale, C)
    k, _ = _pad_to_chunks(k.to(f), C)
    v, _ = _pad_to_chunks(v.to(f), C)
    g, pad = _pad_to_chunks(g.to(f), C)           # padded tokens: k=v=0 and g=0, so the state is unchanged
    qc, kc, vc, gc = _chunk(q, C), _chunk(k, C), _chunk(v, C), _chunk(g, C)
    N = qc.shape[1]
    b = gc.cumsum(2)                               # [B,N,C,H]
    bt = b.permute(0, 1, 3, 2)                     # [B,N,H,C]
    diff = bt[..., :, None] - bt[..., None, :]     # b_i - b_j
    mask = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    Dm = torch.where(mask, diff, torch.full_like(diff, float("-inf"))).exp()
    A = torch.einsum("bnihk,bnjhk->bnhij", qc, kc) * Dm
    o = torch.einsum("bnhij,bnjhv->bnihv", A, vc)
    btot = b[:, :, -1]                             # [B,N,H]
    kd = kc * (btot[:, :, None] - b).exp()[..., None]
    M = torch.einsum("bnchk,bnchv->bnhkv", kd, vc)
    gam = btot.exp()
    S = torch.zeros(B, H, dk, dv, dtype=f, device=q.device) if initial_state is None else initial_state.to(f)
    states = []
    for n in range(N):
        states.append(S)
        S = S * gam[:, n][..., None, None] + M[:, n]
    Sn = torch.stack(states, 1)                    # state entering each chunk
    o = o + torch.einsum("bnchk,bnhkv->bnchv", qc * b.exp()[..., None], Sn)
    o = o.reshape(B, N * C, H, dv)[:, :T]
    return o, S


def chunk_vector_gated(q, k, v, gk, scale: Optional[float] = None, initial_state=None,
                       chunk_size: int = 16, bonus: Optional[torch.Tensor] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Linear attention with a log decay per key channel (GLA, HGRN2, RWKV6).

    The in-chunk score is formed as ``sum_d q_id k_jd e^{b_id - b_jd}`` with the exponent
    taken after the subtraction, so no ``e^{-b}`` ever overflows.  ``bonus`` ``[H,dk]``
    switches to the RWKV6 form: the output reads the state *before* the token's own decay
    and update, and the diagonal uses ``u`` instead of 1 (rwkv6.py:82)."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    C = min(chunk_size, max(T, 1))
    scale = dk ** -0.5 if scale is None else scale
    f = torch.float32
    q, _ = _pad_to_chunks(q.to(f) * scale, C)
    k, _ = _pad_to_chunks(k.to(f), C)
    v, _ = _pad_to_chunks(v.to(f), C)
    gk, _ = _pad_to_chunks(gk.to(f), C)
    qc, kc, vc, gc = _chunk(q, C), _chunk(k, C), _chunk(v, C), _chunk(gk, C)
    N = qc.shape[1]
    b = gc.cumsum(2)                               # [B,N,C,H,dk]  inclusive
    bq = b - gc if bonus is not None else b        # RWKV6 reads S_{t-1}: exclusive cumsum on the query side
    diff = bq[:, :, :, None] - b[:, :, None, :]    # [B,N,i,j,H,dk]
    strict = bonus is not None
    mask = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(-1 if strict else 0)
    diff = torch.where(mask[None, None, :, :, None, None], diff, torch.full_like(diff, float("-inf")))
    A = torch.einsum("bnihk,bnjhk,bnijhk->bnhij", qc, kc, diff.exp())
    if bonus is not None:
        diag = torch.einsum("bnihk,bnihk,hk->bnhi", qc, kc, bonus.to(f))
        A = A + torch.diag_embed(diag)
    o = torch.einsum("bnhij,bnjhv->bnihv", A, vc)
    btot = b[:, :, -1]                             # [B,N,H,dk]
    kd = kc * (btot[:, :, None] - b).exp()
    M = torch.einsum("bnchk,bnchv->bnhkv", kd, vc)
    gam = btot.exp()
    S = torch.zeros(B, H, dk, dv, dtype=f, device=q.device) if initial_state is None else initial_state.to(f)
    states = []
    for n in range(N):
        states.append(S)
        S = S * gam[:, n][..., None] + M[:, n]
    Sn = torch.stack(states, 1)
    o = o + torch.einsum("bnchk,bnhkv->bnchv", qc * bq.exp(), Sn)
    o = o.reshape(B, N * C, H, dv)[:, :T]
    return o, S


def chunk_delta_rule(q, k, v, beta, g: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                     initial_state=None, chunk_size: int = 64, parallel_scan: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """(Gated) delta rule: ``S_t = e^{g_t} S_{t-1}``, ``S_t += beta_t k_t^T (v_t - k_t S_t)``."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    C = min(chunk_size, max(T, 1))
    scale = dk ** -0.5 if scale is None else scale
    f = torch.float32
    if g is None:
        g = torch.zeros(B, T, H, dtype=f, device=q.device)
    q, _ = _pad_to_chunks(q.to(f) * scale, C)
    k, _ = _pad_to_chunks(k.to(f), C)
    v, _ = _pad_to_chunks(v.to(f), C)
    beta, _ = _pad_to_chunks(beta.to(f), C)
    g, _ = _pad_to_chunks(g.to(f), C)
    # contiguous [B,N,H,C,d] copies: every later elementwise op then runs the vectorised kernels instead of strided ones
    qc, kc, vc = (_chunk(x, C).permute(0, 1, 3, 2, 4).contiguous() for x in (q, k, v))
    bc = _chunk(beta, C).permute(0, 1, 3, 2).contiguous()                     # [B,N,H,C]
    b = _chunk(g, C).permute(0, 1, 3, 2).contiguous().cumsum(-1)              # [B,N,H,C], scan along the innermost dim
    N = qc.shape[1]
    diff = b[..., :, None] - b[..., None, :]
    tril = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    L = torch.where(tril, diff, torch.full_like(diff, float("-inf"))).exp()
    KK = torch.einsum("bnhik,bnhjk->bnhij", kc, kc) * L
    A = (KK * bc[..., None]).tril(-1)
    eye = torch.eye(C, dtype=f, device=q.device)
    rhs = torch.cat([vc * bc[..., None], kc * (bc * b.exp())[..., None]], dim=-1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
    U, W = sol[..., :dv], sol[..., dv:]
    QK = torch.einsum("bnhik,bnhjk->bnhij", qc, kc) * L
    qd = qc * b.exp()[..., None]
    btot = b[..., -1]
    kd = kc * (btot[..., None] - b).exp()[..., None]
    gam = btot.exp()
    S = torch.zeros(B, H, dk, dv, dtype=f, device=q.device) if initial_state is None else initial_state.to(f)
    if parallel_scan:
        # Every chunk is an affine map of its entering state, S' = M S + Nb with M = gamma I - kd^T W and
        # Nb = kd^T U; a Hillis-Steele scan over the chunks composes them in log2(N) batched matmuls, after which
        # outputs of all chunks are computed at once (no Python loop over chunks, no per-chunk launches).
        kdT = kd.transpose(-1, -2)
        M = gam[..., None, None] * torch.eye(dk, dtype=f, device=q.device) - kdT @ W          # [B,N,H,dk,dk]
        P = torch.cat([M, kdT @ U], dim=-1)                                                   # [B,N,H,dk,dk+dv]
        d = 1
        while d < N:
            hi, lo = P[:, d:], P[:, :-d]
            comp = hi[..., :dk] @ lo
            comp = torch.cat([comp[..., :dk], comp[..., dk:] + hi[..., dk:]], dim=-1)
            P = torch.cat([P[:, :d], comp], dim=1)
            d *= 2
        after = P[..., :dk] @ S[:, None] + P[..., dk:]                                        # state after chunk n
        enter = torch.cat([S[:, None], after[:, :-1]], dim=1)                                 # state entering chunk n
        vn = U - W @ enter
        o = qd @ enter + QK @ vn
        o = o.permute(0, 1, 3, 2, 4).reshape(B, N * C, H, dv)[:, :T]
        return o, after[:, -1]
    outs = []
    for n in range(N):
        vn = U[:, n] - W[:, n] @ S
        outs.append(qd[:, n] @ S + QK[:, n] @ vn)
        S = S * gam[:, n][..., None, None] + kd[:, n].transpose(-1, -2) @ vn
    o = torch.stack(outs, 1).permute(0, 1, 3, 2, 4).reshape(B, N * C, H, dv)[:, :T]
    return o, S


def normalizer_denominator(q, k, scale: float = 1.0, eps: float = 1e-10,
                           initial_ksum: Optional[torch.Tensor] = None):
    """``q_t . sum_{i<=t} k_i + eps`` for the normalised linear attention of Based/Rebased and
    ``--la-do-feature-map-norm``-style models.  Returns the denominator and the final key sum."""
    z = torch.cumsum(k.float(), dim=1)
    if initial_ksum is not None:
        z = z + initial_ksum[:, None]
    den = (q.float() * scale * z).sum(-1, keepdim=True) + eps
    return den, z[:, -1]


def recurrent_dplr(r, w, k, v, a, b, scale: float = 1.0, initial_state=None):
    """RWKV7 transition, differentiable token loop (state ``[B,H,dk,dv]``)."""
    B, T, H, dk = r.shape
    f = torch.float32
    r, w, k, v, a, b = (x.to(f) for x in (r, w, k, v, a, b))
    S = torch.zeros(B, H, dk, v.shape[-1], dtype=f, device=r.device) if initial_state is None else initial_state.to(f)
    outs = []
    ew = w.exp()
    for t in range(T):
        aS = torch.einsum("bhk,bhkv->bhv", a[:, t], S)
        S = S * ew[:, t][..., None] + b[:, t][..., None] * aS[..., None, :] + k[:, t][..., None] * v[:, t][..., None, :]
        outs.append(torch.einsum("bhk,bhkv->bhv", r[:, t] * scale, S))
    return torch.stack(outs, 1), S


def ssd_chunked(x, dt, A, Bm, Cm, D=None, initial_state=None, chunk_size: int = 128):
    """Mamba2 SSD through the scalar-gated chunk form: q=C, k=B, v=dt*x, g=dt*A."""
    H = x.shape[2]
    rep = H // Bm.shape[2]
    kk = Bm.repeat_interleave(rep, dim=2)
    qq = Cm.repeat_interleave(rep, dim=2)
    g = dt.float() * A.float()[None, None, :]
    y, S = chunk_scalar_gated(qq, kk, x.float() * dt.float()[..., None], g, scale=1.0,
                              initial_state=initial_state, chunk_size=chunk_size)
    if D is not None:
        y = y + x.float() * D.float()[None, None, :, None]
    return y, S


def chunk_value_gated(q, k, v, gv, scale: Optional[float] = None, initial_state=None, chunk_size: int = 16):
    """Linear attention whose state decays per *value* channel:
    ``S_t = S_{t-1} diag(e^{gv_t}) + k_t^T v_t``, ``o_t = scale q_t S_t``.  First pass of gated slot
    attention (slots play the role of value channels)."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    C = min(chunk_size, max(T, 1))
    scale = dk ** -0.5 if scale is None else scale
    f = torch.float32
    q, _ = _pad_to_chunks(q.to(f) * scale, C)
    k, _ = _pad_to_chunks(k.to(f), C)
    v, _ = _pad_to_chunks(v.to(f), C)
    gv, _ = _pad_to_chunks(gv.to(f), C)
    qc, kc, vc, gc = _chunk(q, C), _chunk(k, C), _chunk(v, C), _chunk(gv, C)
    N = qc.shape[1]
    b = gc.cumsum(2)                                           # [B,N,C,H,dv]
    A = torch.einsum("bnihk,bnjhk->bnhij", qc, kc)
    mask = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    diff = b[:, :, :, None] - b[:, :, None, :]                 # [B,N,i,j,H,dv]
    diff = torch.where(mask[None, None, :, :, None, None], diff, torch.full_like(diff, float("-inf")))
    o = torch.einsum("bnhij,bnjhv,bnijhv->bnihv", A, vc, diff.exp())
    btot = b[:, :, -1]
    vd = vc * (btot[:, :, None] - b).exp()
    M = torch.einsum("bnchk,bnchv->bnhkv", kc, vd)
    gam = btot.exp()                                           # [B,N,H,dv]
    S = torch.zeros(B, H, dk, dv, dtype=f, device=q.device) if initial_state is None else initial_state.to(f)
    states = []
    for n in range(N):
        states.append(S)
        S = S * gam[:, n][:, :, None, :] + M[:, n]
    Sn = torch.stack(states, 1)
    o = o + torch.einsum("bnchk,bnhkv->bnchv", qc, Sn) * b.exp()
    return o.reshape(B, N * C, H, dv)[:, :T], S

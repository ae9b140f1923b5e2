"""Token-by-token fp32 definitions of every linear sequence model.

These are the oracles every chunked implementation and every CUDA kernel is tested
against.  They implement the recurrences that the reference obtains from external
Triton packages (call sites: basic_linear_attention.py:133, retention.py:91,
lightning_attention.py:123, gla.py:94, hgrn2.py:76, deltanet.py:127-130,
gated_deltanet.py:112, rwkv6.py:82, rwkv7.py:86, mamba_mixer.py:244-260).

Layout everywhere: q, k ``[B, T, H, dk]``, v ``[B, T, H, dv]``, state ``[B, H, dk, dv]``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def recurrent_lsm(q, k, v, *, g: Optional[torch.Tensor] = None, gk: Optional[torch.Tensor] = None,
                  beta: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                  initial_state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Generic gated (delta-rule) linear attention.

    ``S_t = diag(e^{gk_t}) e^{g_t} S_{t-1}``; then ``S_t += k_t^T v_t`` (or, with ``beta``,
    ``S_t += beta_t k_t^T (v_t - k_t S_t)``); ``o_t = scale * q_t S_t``.

    g: ``[B,T,H]`` log decay per token and head (a constant per-head decay is passed
    expanded); gk: ``[B,T,H,dk]`` log decay per key channel; beta: ``[B,T,H]``.
    """
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    f = torch.float32
    q, k, v = q.to(f), k.to(f), v.to(f)
    S = torch.zeros(B, H, dk, dv, dtype=f, device=q.device) if initial_state is None else initial_state.to(f).clone()
    o = torch.empty(B, T, H, dv, dtype=f, device=q.device)
    for t in range(T):
        if g is not None:
            S = S * g[:, t].to(f).exp()[..., None, None]
        if gk is not None:
            S = S * gk[:, t].to(f).exp()[..., None]
        kt, vt = k[:, t], v[:, t]
        if beta is not None:
            vt = (vt - torch.einsum("bhk,bhkv->bhv", kt, S)) * beta[:, t].to(f)[..., None]
        S = S + kt[..., None] * vt[..., None, :]
        o[:, t] = torch.einsum("bhk,bhkv->bhv", q[:, t] * scale, S)
    return o, S


def recurrent_linear_attn_normalized(q, k, v, scale=1.0, eps=1e-10):
    """Basic linear attention with the sum normaliser
    ``o_t = (q_t S_t) / (q_t . sum_{i<=t} k_i + eps)`` (fla ``normalize=True``)."""
    o, S = recurrent_lsm(q, k, v, scale=scale)
    z = torch.cumsum(k.float(), dim=1)
    den = (q.float() * scale * z).sum(-1, keepdim=True) + eps
    return o / den, S


def recurrent_rwkv6(r, k, v, w, u, scale=None, initial_state=None):
    """``o_t = r_t (S_{t-1} + diag(u) k_t^T v_t)``; ``S_t = diag(e^{w_t}) S_{t-1} + k_t^T v_t``.
    w: ``[B,T,H,dk]`` log decay (<= 0); u: ``[H,dk]`` bonus."""
    B, T, H, dk = r.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    f = torch.float32
    r, k, v, w, u = r.to(f), k.to(f), v.to(f), w.to(f), u.to(f)
    S = torch.zeros(B, H, dk, dv, dtype=f, device=r.device) if initial_state is None else initial_state.to(f).clone()
    o = torch.empty(B, T, H, dv, dtype=f, device=r.device)
    for t in range(T):
        kv = k[:, t][..., None] * v[:, t][..., None, :]
        o[:, t] = torch.einsum("bhk,bhkv->bhv", r[:, t] * scale, S + u[None, :, :, None] * kv)
        S = S * w[:, t].exp()[..., None] + kv
    return o, S


def recurrent_rwkv7(r, w, k, v, a, b, scale=None, initial_state=None):
    """Diagonal-plus-low-rank transition (generalised delta rule), state ``[dk, dv]``:
    ``S_t = diag(e^{w_t}) S_{t-1} + b_t^T (a_t S_{t-1}) + k_t^T v_t``; ``o_t = r_t S_t``."""
    B, T, H, dk = r.shape
    dv = v.shape[-1]
    scale = 1.0 if scale is None else scale
    f = torch.float32
    r, w, k, v, a, b = (x.to(f) for x in (r, w, k, v, a, b))
    S = torch.zeros(B, H, dk, dv, dtype=f, device=r.device) if initial_state is None else initial_state.to(f).clone()
    o = torch.empty(B, T, H, dv, dtype=f, device=r.device)
    for t in range(T):
        aS = torch.einsum("bhk,bhkv->bhv", a[:, t], S)
        S = S * w[:, t].exp()[..., None] + b[:, t][..., None] * aS[..., None, :] + k[:, t][..., None] * v[:, t][..., None, :]
        o[:, t] = torch.einsum("bhk,bhkv->bhv", r[:, t] * scale, S)
    return o, S


def recurrent_ssd(x, dt, A, Bm, Cm, D=None, initial_state=None):
    """Mamba2 state-space duality recurrence.

    x ``[B,T,H,P]``, dt ``[B,T,H]`` (already softplus'ed), A ``[H]`` (negative),
    Bm/Cm ``[B,T,G,N]`` with ``H % G == 0``; state ``[B,H,N,P]``:
    ``h_t = e^{dt_t A} h_{t-1} + dt_t B_t^T x_t``; ``y_t = C_t h_t + D x_t``."""
    Bsz, T, H, P = x.shape
    G = Bm.shape[2]
    rep = H // G
    kk = Bm.repeat_interleave(rep, dim=2)
    qq = Cm.repeat_interleave(rep, dim=2)
    g = dt.float() * A.float()[None, None, :]
    vv = x.float() * dt.float()[..., None]
    y, S = recurrent_lsm(qq, kk, vv, g=g, scale=1.0, initial_state=initial_state)
    if D is not None:
        y = y + x.float() * D.float()[None, None, :, None]
    return y, S


def slopes_power_of_2(n: int):
    start = 2 ** (-(2 ** -(math.log2(n) - 3)))
    return [start * start ** i for i in range(n)]


def lightning_slopes(num_heads: int) -> torch.Tensor:
    """ALiBi-style per-head decay rates ``s_h`` (decay per token ``e^{-s_h}``), as built by
    lightning_attention.py:79-105."""
    if math.log2(num_heads).is_integer():
        s = slopes_power_of_2(num_heads)
    else:
        p = 2 ** math.floor(math.log2(num_heads))
        s = slopes_power_of_2(p) + lightning_slopes(2 * p).tolist()[0::2][: num_heads - p]
    return torch.tensor(s, dtype=torch.float32)


def retention_log_decay(num_heads: int) -> torch.Tensor:
    """``log(1 - 2^{-5-h})`` per head (fla retention)."""
    return torch.log(1.0 - 2.0 ** (-5.0 - torch.arange(num_heads, dtype=torch.float32)))

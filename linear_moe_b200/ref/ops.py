"""Eager fp32 definitions of the non-LSM operators (norms, activations, rotary, attention,
router, expert MLP, cross entropy, short convolution).

They are the oracle for the CUDA kernels and the implementation used for CPU tensors.
Everything is differentiable by autograd.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ---- norms ---------------------------------------------------------------
def rms_norm(x, weight=None, eps: float = 1e-6):
    """``x * rsqrt(mean(x^2) + eps) * w`` in fp32, cast back (qwen2/rms_norm.py:13-17)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    y = F.layer_norm(x.float(), (x.shape[-1],), None if weight is None else weight.float(),
                     None if bias is None else bias.float(), eps)
    return y.to(x.dtype)


def gated_rms_norm(x, z, weight, eps: float = 1e-5, group_size: Optional[int] = None):
    """``rmsnorm(x * silu(z)) * w`` with the norm taken over groups of ``group_size`` channels
    (Mamba2 ``RMSNormGated`` with ``norm_before_gate=False``, mamba_mixer.py:190-197)."""
    xf = x.float() * F.silu(z.float())
    d = x.shape[-1]
    gs = group_size or d
    xg = xf.reshape(*xf.shape[:-1], d // gs, gs)
    y = (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)).reshape_as(xf)
    return (y * weight.float()).to(x.dtype)


def group_norm_heads(x, weight=None, bias=None, eps: float = 1e-5):
    """GroupNorm with one group per head over ``[..., H, d]`` (``--la-output-norm groupnorm``)."""
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def l2_norm(x, eps: float = 1e-6):
    """``x * rsqrt(sum(x^2) + eps)`` (common_modules/l2norm.py:22-46)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


# ---- activations -----------------------------------------------------------
def swiglu(x):
    """``silu(x[..., :f]) * x[..., f:]`` (activations.py:304-329; experts.py GLU convention)."""
    a, b = x.float().chunk(2, dim=-1)
    return (F.silu(a) * b).to(x.dtype)


def swish_gate(o, g):
    """LSM output gate ``o * swish(g)`` (linear_attention.py:255)."""
    return (o.float() * F.silu(g.float())).to(o.dtype)


def logsigmoid(x):
    return F.logsigmoid(x.float()).to(x.dtype)


ACT2FN = {
    "swish": F.silu, "silu": F.silu, "gelu": F.gelu, "relu": F.relu, "sigmoid": torch.sigmoid,
    "logsigmoid": F.logsigmoid, "tanh": torch.tanh, "identity": lambda x: x,
    "sqrelu": lambda x: F.relu(x).pow(2), "elu": F.elu,
}


# ---- rotary ----------------------------------------------------------------
def rope_freqs(seq_len: int, dim: int, base: float = 10000.0, offset: int = 0, device=None,
               interpolation_factor: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[seq_len, dim/2]`` in fp32."""
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    pos = torch.arange(offset, offset + seq_len, dtype=torch.float32, device=device)
    if interpolation_factor:
        pos = pos / interpolation_factor
    ang = pos[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def yarn_find_correction_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_freqs(seq_len: int, dim: int, base: float, factor: float, original_max_pos: int = 4096,
               beta_fast: float = 32, beta_slow: float = 1, mscale: float = 1.0, mscale_all_dim: float = 0.0,
               offset: int = 0, device=None) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """YaRN-scaled tables (deepseek_v2/yarn_rotary_pos_embedding.py:19-207).  Returns cos, sin (already
    multiplied by ``mscale/mscale_all_dim``) and the factor whose square multiplies the softmax scale."""
    freq_extra = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    freq_inter = freq_extra / factor
    low = max(math.floor(yarn_find_correction_dim(beta_fast, dim, base, original_max_pos)), 0)
    high = min(math.ceil(yarn_find_correction_dim(beta_slow, dim, base, original_max_pos)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
    inv_mask = 1.0 - ramp
    inv = freq_inter * (1 - inv_mask) + freq_extra * inv_mask
    pos = torch.arange(offset, offset + seq_len, dtype=torch.float32, device=device)
    ang = pos[:, None] * inv[None, :]

    def get_mscale(scale, m):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
    m = get_mscale(factor, mscale) / get_mscale(factor, mscale_all_dim)
    return ang.cos() * m, ang.sin() * m, get_mscale(factor, mscale_all_dim)


def apply_rope(x, cos, sin, interleaved: bool = False):
    """Rotate the first ``2*cos.shape[-1]`` channels of ``x [B,T,H,D]``; cos/sin ``[T, R/2]``.
    Non-interleaved pairs channel i with i+R/2 (Megatron/NeoX); interleaved pairs 2i with 2i+1."""
    R = cos.shape[-1] * 2
    xf = x.float()
    xr, xp = xf[..., :R], xf[..., R:]
    c, s = cos[None, :, None, :].float(), sin[None, :, None, :].float()
    if interleaved:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).flatten(-2)
    else:
        x1, x2 = xr[..., : R // 2], xr[..., R // 2:]
        o = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    return torch.cat([o, xp], dim=-1).to(x.dtype)


# ---- softmax attention -----------------------------------------------------
def softmax_attention(q, k, v, scale: Optional[float] = None, causal: bool = True, q_offset: int = 0,
                      window: Optional[int] = None):
    """Naive attention with GQA.  q ``[B,Tq,Hq,D]``, k/v ``[B,Tk,Hkv,D(v)]``.  ``q_offset`` is the
    absolute position of q[0] relative to k[0] (sequence-parallel ranks hold a suffix of the keys'
    positions; dot_product_attention.py:139-183 is the unfused form this replaces)."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    rep = Hq // Hkv
    kf = k.float().repeat_interleave(rep, dim=2)
    vf = v.float().repeat_interleave(rep, dim=2)
    s = torch.einsum("bihd,bjhd->bhij", q.float() * scale, kf)
    if causal:
        i = torch.arange(Tq, device=q.device)[:, None] + q_offset
        j = torch.arange(Tk, device=q.device)[None, :]
        m = j <= i
        if window is not None:
            m = m & (j > i - window)
        s = s.masked_fill(~m, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhij,bjhd->bihd", p, vf).to(q.dtype)


# ---- short convolution -----------------------------------------------------
def causal_conv1d(x, weight, bias=None, activation: Optional[str] = "silu",
                  initial_state: Optional[torch.Tensor] = None):
    """Depthwise causal convolution over time.  x ``[B,T,D]``, weight ``[D,K]``; tap ``K-1`` multiplies
    the current token (causal_conv1d convention, mamba_mixer.py:291-296).  ``initial_state``
    ``[B,K-1,D]`` holds the tokens before x[0] (previous sequence-parallel rank or decode cache).
    Returns ``(y, final_state)``."""
    B, T, D = x.shape
    K = weight.shape[-1]
    xf = x.float()
    if initial_state is None:
        initial_state = xf.new_zeros(B, K - 1, D)
    xp = torch.cat([initial_state.float(), xf], dim=1)            # [B, T+K-1, D]
    y = sum(xp[:, i:i + T] * weight.float()[:, i] for i in range(K))
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    return y.to(x.dtype), xp[:, T:].to(x.dtype)


# ---- cross entropy ---------------------------------------------------------
def linear_cross_entropy(h, weight, labels, ignore_index: int = -100):
    """Per-token loss of ``softmax(h W^T)`` against ``labels`` without reducing; ignored labels give 0."""
    logits = h.float() @ weight.float().t()
    return F.cross_entropy(logits, labels, reduction="none", ignore_index=ignore_index)


# ---- router ----------------------------------------------------------------
def router_topk(logits, k: int, order: str = "softmax_topk"):
    """``softmax_topk``: softmax over all experts then top-k, no renormalisation
    (qwen2/moe/router.py:70-76).  ``topk_softmax``: top-k logits then softmax over the k
    (mixtral/moe/router.py:159-160).  Returns (probs ``[T,k]`` fp32, indices ``[T,k]``, full softmax)."""
    lf = logits.float()
    full = torch.softmax(lf, dim=-1)
    if order == "softmax_topk":
        p, idx = torch.topk(full, k, dim=-1)
    else:
        top, idx = torch.topk(lf, k, dim=-1)
        p = torch.softmax(top, dim=-1)
    return p, idx, full


def switch_load_balancing_loss(full_probs, indices, num_experts: int, coeff: float):
    """``E * sum_e mean_t(p_te) * mean_t(1[e in topk(t)]) * coeff`` (mixtral/moe/moe_utils.py:17-33)."""
    T, k = indices.shape
    counts = torch.zeros(num_experts, dtype=torch.float32, device=indices.device)
    counts.scatter_add_(0, indices.reshape(-1), torch.ones(T * k, dtype=torch.float32, device=indices.device))
    return (full_probs.mean(0) * (counts / (T * k))).sum() * num_experts * coeff


def z_loss(logits, coeff: float):
    """``mean(logsumexp(logits)^2) * coeff`` (mixtral/moe/moe_utils.py:36-48)."""
    return torch.logsumexp(logits.float(), dim=-1).pow(2).mean() * coeff


def sinkhorn(cost, tol: float = 1e-4, max_iter: int = 100):
    """Sinkhorn normalisation for ``--moe-router-load-balancing-type sinkhorn`` (moe_utils.py:51-73)."""
    cost = torch.exp(cost.float())
    d0 = torch.ones(cost.size(0), device=cost.device)
    d1 = torch.ones(cost.size(1), device=cost.device)
    eps = 1e-8
    err = 1e9
    it = 0
    while err > tol and it < max_iter:
        d0 = (1 / d0.size(0)) / (torch.sum(d1 * cost, 1) + eps)
        d1_new = (1 / d1.size(0)) / (torch.sum(d0.unsqueeze(1) * cost, 0) + eps)
        err = torch.mean(torch.abs(d1 - d1_new)).item()
        d1 = d1_new
        it += 1
    return d1 * cost * d0.unsqueeze(1)


# ---- expert MLP ------------------------------------------------------------
def grouped_mlp(x_sorted, tokens_per_expert, w1, w2):
    """Expert-sorted tokens through per-expert SwiGLU MLPs.  w1 ``[E, h, 2f]``, w2 ``[E, f, h]``
    (GroupedMLP layout, experts.py:59-82,156-168)."""
    outs = []
    start = 0
    counts = tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)
    for e, n in enumerate(counts):
        xe = x_sorted[start:start + n]
        he = swiglu(xe @ w1[e].to(xe.dtype))
        outs.append(he @ w2[e].to(xe.dtype))
        start += n
    return torch.cat(outs, 0) if outs else x_sorted.new_zeros(0, w2.shape[-1])

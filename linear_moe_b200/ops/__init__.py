"""Operator API used by every layer.

Each function takes torch tensors and is differentiable.  For CUDA tensors it runs the
hand-written sm_100a kernels of ``linear_moe_b200/csrc`` (through :mod:`.cuda`; a missing
or stale kernel library is an error there, not a silent fallback); for CPU tensors it runs
the eager fp32 definitions of :mod:`linear_moe_b200.ref`.  Plain dense GEMMs go to cuBLAS
through ``torch.nn.functional.linear`` unless the fused tcgen05 variants are requested.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ..ref import ops as R
from . import lsm_torch as LT


def _cuda(x: torch.Tensor) -> bool:
    return x.is_cuda


def _K():
    from . import cuda as K
    return K


# ---- GEMM-shaped -----------------------------------------------------------
def linear(x, weight, bias=None):
    if _cuda(x) and x.dtype == torch.bfloat16:
        return _K().linear(x, weight, bias)
    return F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


def linear_swiglu(x, weight, bias=None):
    """``swiglu(x W^T)`` with W = [gate; up]; on CUDA the activation runs in the GEMM epilogue."""
    if _cuda(x) and x.dtype == torch.bfloat16 and bias is None:
        return _K().linear_swiglu(x, weight)
    return swiglu(linear(x, weight, bias))


def mlp_swiglu(x, w1, w2):
    """``fc2(swiglu(fc1(x)))`` without biases (``w1 [2f, h]`` = [gate; up], ``w2 [h, f]``)."""
    if _cuda(x):
        return _K().mlp_swiglu(x, w1, w2)
    return linear(linear_swiglu(x, w1), w2)


def allgather_linear(x, weight, bias, group, dim: int = 1):
    """All-gather ``x`` along ``dim`` over ``group`` then ``linear`` (sequence-parallel column layer)."""
    from ..dist import collectives as C
    if _cuda(x) and not group.is_trivial and _K().fused_tp_available(group):
        return _K().allgather_linear(x, weight, bias, group, dim)
    return linear(C.all_gather(x, group, dim=dim), weight, bias)


def linear_reducescatter(x, weight, group, dim: int = 1):
    """``linear`` then reduce-scatter along ``dim`` (sequence-parallel row layer)."""
    from ..dist import collectives as C
    if _cuda(x) and not group.is_trivial and _K().fused_tp_available(group):
        return _K().linear_reducescatter(x, weight, group, dim)
    return C.reduce_scatter(linear(x, weight, None), group, dim=dim)


class _ChunkedLinearCE(torch.autograd.Function):
    """LM head + cross entropy without the full logits: per chunk of tokens compute logits, the
    log-sum-exp and the target logit; backward recomputes the chunk's logits."""

    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, chunk):
        T = h.shape[0]
        loss = torch.empty(T, dtype=torch.float32, device=h.device)
        lse = torch.empty(T, dtype=torch.float32, device=h.device)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            logits = _K().mm_nt(h[s:e], weight.to(h.dtype)) if _cuda(h) else F.linear(h[s:e], weight.to(h.dtype))
            if _cuda(h):
                _K().softmax_ce_fwd(logits, labels[s:e], loss[s:e], lse[s:e], ignore_index)
            else:
                lf = logits.float()
                l = torch.logsumexp(lf, -1)
                lab = labels[s:e]
                valid = lab != ignore_index
                tgt = lf.gather(-1, lab.clamp(min=0)[:, None]).squeeze(-1)
                loss[s:e] = torch.where(valid, l - tgt, torch.zeros_like(l))
                lse[s:e] = l
        ctx.save_for_backward(h, weight, labels, lse)
        ctx.ignore_index, ctx.chunk = ignore_index, chunk
        return loss

    @staticmethod
    def backward(ctx, gl):
        h, weight, labels, lse = ctx.saved_tensors
        T, chunk = h.shape[0], ctx.chunk
        dh = torch.empty_like(h)
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=h.device)
        wd = weight.to(h.dtype)
        gl = gl.float().contiguous()
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            logits = _K().mm_nt(h[s:e], wd) if _cuda(h) else F.linear(h[s:e], wd)
            if _cuda(h):
                g = _K().softmax_ce_bwd(logits, labels[s:e], lse[s:e], gl[s:e], ctx.ignore_index)
            else:
                p = (logits.float() - lse[s:e, None]).exp()
                lab = labels[s:e]
                valid = (lab != ctx.ignore_index).float()
                p.scatter_add_(-1, lab.clamp(min=0)[:, None], -torch.ones_like(p[:, :1]))
                g = (p * (gl[s:e] * valid)[:, None]).to(h.dtype)
            dh[s:e] = _K().mm_nn(g, wd) if _cuda(h) else g @ wd
            if _cuda(h) and g.dtype != torch.float32:
                dw += _K().mm_tn(g, h[s:e], out_dtype=torch.float32)       # bf16 operands, fp32 accumulate + output
            else:
                dw.addmm_(g.t().float(), h[s:e].float())
        return dh, dw.to(weight.dtype), None, None, None


class _CachedLinearCE(torch.autograd.Function):
    """LM head + cross entropy that keeps ``Z = softmax(logits) - onehot(label)`` in bf16 instead of
    recomputing the logits in the backward: forward = one GEMM + two passes over the logits (log-sum-exp,
    then in-place conversion to Z); backward = ``dh = g * (Z W)`` and ``dW = Z^T (g * h)``, two GEMMs.
    Costs ``T*V*2`` bytes; used when that fits the budget of :func:`linear_cross_entropy`."""

    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index):
        T = h.shape[0]
        wd = weight if weight.dtype == h.dtype else weight.to(h.dtype)
        Z = _K().mm_nt(h, wd)
        loss = torch.empty(T, dtype=torch.float32, device=h.device)
        lse = torch.empty(T, dtype=torch.float32, device=h.device)
        K = _K()
        K.softmax_ce_fwd(Z, labels, loss, lse, ignore_index)
        K.softmax_ce_bwd(Z, labels, lse, torch.ones(T, dtype=torch.float32, device=h.device), ignore_index)
        ctx.save_for_backward(h, wd, Z)
        ctx.wdtype, ctx.weight = weight.dtype, weight
        return loss

    @staticmethod
    def backward(ctx, gl):
        h, wd, Z = ctx.saved_tensors
        g = gl.to(h.dtype)[:, None]
        dh = _K().mm_nn(Z, wd) * g
        hg = h * g
        if _K().wgrad_into_main_grad(ctx.weight, Z, hg):
            return dh, None, None, None
        dw = _K().mm_tn(Z, hg)
        return dh, dw.to(ctx.wdtype), None, None


_CE_CACHE_BYTES = 8 << 30


def linear_cross_entropy(h, weight, labels, ignore_index: int = -100, chunk: int = 4096):
    """Per-token loss ``[T]`` of ``softmax(h W^T)`` vs ``labels``; h ``[T,hid]``, W ``[V,hid]``."""
    if (_cuda(h) and h.dtype == torch.bfloat16 and torch.is_grad_enabled()
            and h.shape[0] * weight.shape[0] * 2 <= _CE_CACHE_BYTES):
        return _CachedLinearCE.apply(h, weight, labels.contiguous(), ignore_index)
    return _ChunkedLinearCE.apply(h, weight, labels, ignore_index, chunk)


def embedding(ids, weight, id_offset: int = 0, sharded: bool = False):
    """Rows ``ids - id_offset`` of ``weight``; with ``sharded`` (vocabulary split over tensor-parallel ranks) ids outside
    this shard give zero rows."""
    if _cuda(weight):
        return _K().embedding(ids, weight, id_offset, sharded)
    if not sharded:
        return F.embedding(ids, weight)
    local = ids - id_offset
    oob = (local < 0) | (local >= weight.shape[0])
    return F.embedding(local.masked_fill(oob, 0), weight).masked_fill(oob[..., None], 0.0)


# ---- norms / activations / rotary -----------------------------------------
def rms_norm(x, weight=None, eps: float = 1e-6):
    if _cuda(x):
        return _K().rms_norm(x, weight, eps)
    return R.rms_norm(x, weight, eps)


def add_rms_norm(x, residual, weight, eps: float = 1e-6):
    """``r = x + residual; y = rmsnorm(r)``; returns ``(y, r)`` (bias-dropout-add with p=0 fused into
    the following norm; transformer_layer.py:218-221 + rms_norm.py:13-17)."""
    if _cuda(x):
        return _K().add_rms_norm(x, residual, weight, eps)
    r = x + residual
    return R.rms_norm(r, weight, eps), r


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if _cuda(x):
        return _K().layer_norm(x, weight, bias, eps)
    return R.layer_norm(x, weight, bias, eps)


def add_layer_norm(x, residual, weight, bias, eps: float = 1e-5):
    """``r = x + residual; y = layernorm(r)``; returns ``(y, r)`` (the LayerNorm counterpart of :func:`add_rms_norm`)."""
    if _cuda(x):
        return _K().add_layer_norm(x, residual, weight, bias, eps)
    r = x + residual
    return R.layer_norm(r, weight, bias, eps), r


def group_norm_heads(x, weight=None, bias=None, eps: float = 1e-5):
    """GroupNorm with one group per head over ``[..., H, d]`` = LayerNorm over the head dimension (same kernel on CUDA)."""
    if _cuda(x):
        return _K().layer_norm(x, weight, bias, eps)
    return R.group_norm_heads(x, weight, bias, eps)


def gated_rms_norm(x, z, weight, eps: float = 1e-5, group_size: Optional[int] = None):
    if _cuda(x):
        return _K().gated_rms_norm(x, z, weight, eps, group_size)
    return R.gated_rms_norm(x, z, weight, eps, group_size)


def head_norm_gate(o, weight, gate, eps: float = 1e-5, gate_fn: str = "swish", norm: str = "rmsnorm"):
    """LSM epilogue: per-head output norm over ``o [B,T,H,dv]`` then ``* gate_fn(gate [B,T,H*dv])``
    (lightning_attention.py:124 + linear_attention.py:255), one pass on CUDA."""
    B, T, H, dv = o.shape
    if _cuda(o) and norm in ("rmsnorm", "identity") and gate_fn in ("swish", "silu"):
        return _K().head_norm_gate(o, weight, gate, eps, norm == "rmsnorm")
    if norm == "rmsnorm":
        y = R.rms_norm(o, weight, eps)
    elif norm == "groupnorm":
        y = group_norm_heads(o, weight, None, eps)
    else:
        y = o
    y = y.reshape(B, T, H * dv)
    return (y.float() * R.ACT2FN[gate_fn](gate.float())).to(o.dtype)


def l2_norm(x, eps: float = 1e-6):
    if _cuda(x):
        return _K().l2_norm(x, eps)
    return R.l2_norm(x, eps)


def swiglu(x):
    if _cuda(x):
        return _K().swiglu(x)
    return R.swiglu(x)


def swish_gate(o, g):
    return R.swish_gate(o, g)


def apply_rope(x, cos, sin, interleaved: bool = False):
    if _cuda(x):
        return _K().apply_rope(x, cos, sin, interleaved)
    return R.apply_rope(x, cos, sin, interleaved)


def rope_positions(T: int, batch: int, device, seqlen_offsets=None, cu_seqlens=None):
    """Token positions for rotary embeddings of sequences that do not all start at 0.

    ``seqlen_offsets``: an int or an int tensor ``[batch]`` -- sequence ``b`` starts at position ``offsets[b]`` (decoding
    with caches of different lengths).  ``cu_seqlens``: int tensor ``[n + 1]`` of a packed batch (``batch == 1``, ``T`` =
    total tokens) -- positions restart at every boundary.  The two can be combined (one offset per packed sequence).
    Same contract as the ``seqlen_offsets`` / ``cu_seqlens`` arguments of the reference's rotary kernel
    (common_modules/rotary.py:40-134).  Returns an int64 tensor ``[batch, T]``."""
    ar = torch.arange(T, device=device, dtype=torch.int64)
    if cu_seqlens is not None:
        cu = cu_seqlens.to(device=device, dtype=torch.int64)
        seq_id = torch.searchsorted(cu[1:].contiguous(), ar, right=True)            # packed sequence of every token
        pos = ar - cu[seq_id]
        if seqlen_offsets is not None:
            off = torch.as_tensor(seqlen_offsets, device=device, dtype=torch.int64)
            pos = pos + (off[seq_id] if off.dim() else off)
        return pos[None, :].expand(batch, T)
    pos = ar[None, :].expand(batch, T)
    if seqlen_offsets is not None:
        off = torch.as_tensor(seqlen_offsets, device=device, dtype=torch.int64)
        pos = pos + (off[:, None] if off.dim() else off)
    return pos


def apply_rope_at(x, cos_table, sin_table, positions, interleaved: bool = False):
    """Rotary embedding with an explicit position per token: ``x`` ``[B,T,H,D]``, tables ``[P, R/2]`` covering every
    position, ``positions`` int ``[B,T]`` (see :func:`rope_positions`).  The per-token rows of the tables are gathered
    once and the ordinary kernel runs on the batch flattened into one sequence."""
    B, T, H, D = x.shape
    idx = positions.reshape(-1)
    cos, sin = cos_table.index_select(0, idx), sin_table.index_select(0, idx)
    return apply_rope(x.reshape(1, B * T, H, D), cos, sin, interleaved).reshape(B, T, H, D)


def gated_add(a, s, g):
    """``a + s * sigmoid(g)``; ``a``, ``s`` ``[..., N]``, ``g`` ``[..., 1]`` gate logits (the shared expert of a Qwen2-MoE
    layer joining the routed experts' output)."""
    if _cuda(a):
        return _K().gated_add(a, s, g)
    return a + s * torch.sigmoid(g)


def causal_conv1d(x, weight, bias=None, activation="silu", initial_state=None):
    if _cuda(x):
        return _K().causal_conv1d(x, weight, bias, activation, initial_state)
    return R.causal_conv1d(x, weight, bias, activation, initial_state)


# ---- attention -------------------------------------------------------------
def softmax_attention(q, k, v, scale=None, causal=True, q_offset: int = 0, window=None):
    if _cuda(q):
        return _K().flash_attention(q, k, v, scale, causal, q_offset, window)
    return R.softmax_attention(q, k, v, scale, causal, q_offset, window)


# ---- linear sequence models -----------------------------------------------
def lsm_scalar(q, k, v, g=None, scale=None, initial_state=None, chunk_size: int = 64):
    """Scalar-decay family (basic LA, retention, lightning, simple-GLA, SSD).  Returns (o, S_T)."""
    if _cuda(q):
        return _K().lsm_scalar(q, k, v, g, scale, initial_state, chunk_size)
    return LT.chunk_scalar_gated(q, k, v, g, scale, initial_state, chunk_size)


def lsm_vector(q, k, v, gk, scale=None, initial_state=None, bonus=None, chunk_size: int = 64):
    """Vector-decay family (GLA, HGRN2, RWKV6 with ``bonus``)."""
    if _cuda(q):
        return _K().lsm_vector(q, k, v, gk, scale, initial_state, bonus, chunk_size)
    return LT.chunk_vector_gated(q, k, v, gk, scale, initial_state, 16, bonus)


def lsm_delta(q, k, v, beta, g=None, scale=None, initial_state=None, chunk_size: int = 64):
    """(Gated) delta rule (DeltaNet, Gated DeltaNet)."""
    if _cuda(q):
        return _K().lsm_delta(q, k, v, beta, g, scale, initial_state, chunk_size)
    return LT.chunk_delta_rule(q, k, v, beta, g, scale, initial_state, chunk_size)


def lsm_dplr(r, w, k, v, a, b, scale=1.0, initial_state=None):
    """RWKV7 diagonal-plus-low-rank transition."""
    return LT.recurrent_dplr(r, w, k, v, a, b, scale, initial_state)


def ssd(x, dt, A, Bm, Cm, D=None, initial_state=None, chunk_size: int = 128):
    """Mamba2 SSD: q=C, k=B (shared by the heads of a group), v=dt*x, g=dt*A."""
    H = x.shape[2]
    rep = H // Bm.shape[2]
    kk = Bm.repeat_interleave(rep, dim=2) if rep > 1 else Bm
    qq = Cm.repeat_interleave(rep, dim=2) if rep > 1 else Cm
    g = dt.float() * A.float()[None, None, :]
    vv = (x.float() * dt.float()[..., None]).to(x.dtype)
    y, S = lsm_scalar(qq, kk, vv, g, 1.0, initial_state, min(chunk_size, 64) if _cuda(x) else chunk_size)
    if D is not None:
        y = y + (x.float() * D.float()[None, None, :, None]).to(y.dtype)
    return y, S


# ---- MoE -------------------------------------------------------------------
def router_topk(logits, k: int, order: str = "softmax_topk"):
    if _cuda(logits):
        return _K().router_topk(logits, k, order)
    return R.router_topk(logits, k, order)


def grouped_mlp(x_sorted, tokens_per_expert, w1, w2):
    if _cuda(x_sorted):
        return _K().grouped_mlp(x_sorted, tokens_per_expert, w1, w2)
    return R.grouped_mlp(x_sorted, tokens_per_expert, w1, w2)

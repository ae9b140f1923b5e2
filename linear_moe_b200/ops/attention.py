"""Softmax attention on CUDA tensors.

``flash_attention`` runs this framework's causal GQA flash-attention kernel (``csrc/flash_attn.cu``) when
the shape is supported and otherwise falls back to torch's scaled-dot-product attention (a library
kernel), which also serves as the comparator in the tests.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..ref import ops as R


def sdpa_reference(q, k, v, scale, causal, q_offset, window):
    """Library attention: q [B,Tq,Hq,D], k/v [B,Tk,Hkv,D]."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    plain_causal = causal and q_offset == 0 and Tq == Tk and window is None
    if plain_causal or not causal:
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=plain_causal, scale=scale, enable_gqa=Hq != Hkv)
    else:
        i = torch.arange(Tq, device=q.device)[:, None] + q_offset
        j = torch.arange(Tk, device=q.device)[None, :]
        m = j <= i
        if window is not None:
            m = m & (j > i - window)
        o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=m, scale=scale, enable_gqa=Hq != Hkv)
    return o.transpose(1, 2)


def flash_attention(q, k, v, scale: Optional[float], causal: bool, q_offset: int, window: Optional[int]):
    from . import flash
    if flash.supported(q, k, v, causal, window):
        return flash.FlashAttention.apply(q, k, v, scale if scale is not None else q.shape[-1] ** -0.5, q_offset, window)
    if q.dtype in (torch.bfloat16, torch.float16) and v.shape[-1] == q.shape[-1]:
        return sdpa_reference(q, k, v, scale, causal, q_offset, window)
    return R.softmax_attention(q, k, v, scale, causal, q_offset, window)

"""Binding of the causal GQA flash-attention kernels (``csrc/flash_attn.cu``)."""
from __future__ import annotations

import torch


def supported(q, k, v, causal, window) -> bool:
    return False


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, q_offset):
        raise NotImplementedError

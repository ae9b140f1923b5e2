"""Norm modules with the call contract of the reference's ``common_modules/layernorm.py``.

``RMSNorm`` / ``LayerNorm`` / ``GroupNorm`` (layernorm.py:536-665): ``forward(x, residual=None, prenorm=False,
residual_in_fp32=False)`` normalises ``x + residual`` and, with ``prenorm``, also returns the summed residual stream.
``RMSNormLinear`` / ``LayerNormLinear`` / ``GroupNormLinear`` (layernorm.py:668-940): the same followed by a linear
layer whose weight and bias are call arguments, as ONE autograd node that keeps only its inputs and recomputes the
normalised activation in the backward pass, so the ``[tokens, hidden]`` output of the norm is never stored.

Everything runs on the kernels behind ``ops`` for CUDA tensors (RMSNorm / LayerNorm with fused residual add, the dense
GEMM with its bias epilogue) and on the fp32 definitions for CPU tensors.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops


def _group_norm(x, groups: int, weight, bias, eps: float):
    """Normalise every one of ``groups`` equal slices of the last dimension on its own (affine per channel)."""
    shape = x.shape
    h = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    h = ops.group_norm_heads(h, None, None, eps).reshape(shape)
    if weight is not None:
        h = h * weight.to(h.dtype)
    if bias is not None:
        h = h + bias.to(h.dtype)
    return h


class _NormBase(nn.Module):
    kind = "rms"

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, bias: bool = False, eps: float = 1e-5,
                 num_groups: Optional[int] = None, dtype=None, device=None):
        super().__init__()
        self.hidden_size, self.eps, self.num_groups = hidden_size, eps, num_groups
        if num_groups is not None and hidden_size % num_groups:
            raise ValueError("num_channels must be divisible by num_groups")
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device)) if elementwise_affine else None
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device)) if (elementwise_affine and bias) else None

    def _norm(self, x, residual, residual_in_fp32: bool):
        """``(normalised x + residual, residual stream)``."""
        if residual is not None:
            if self.kind == "rms" and self.bias is None and self.weight is not None and not residual_in_fp32:
                return ops.add_rms_norm(x, residual.to(x.dtype), self.weight, self.eps)       # one kernel: add + norm
            if self.kind == "layer" and self.weight is not None and not residual_in_fp32:
                b = self.bias if self.bias is not None else torch.zeros_like(self.weight)
                return ops.add_layer_norm(x, residual.to(x.dtype), self.weight, b, self.eps)
            stream = (x.float() + residual.float()) if residual_in_fp32 else x + residual.to(x.dtype)
        else:
            stream = x.float() if residual_in_fp32 else x
        h = stream.to(x.dtype)
        if self.kind == "rms":
            y = ops.rms_norm(h, self.weight, self.eps)
            if self.bias is not None:
                y = y + self.bias.to(y.dtype)
        elif self.kind == "layer":
            w = self.weight if self.weight is not None else torch.ones(self.hidden_size, dtype=h.dtype, device=h.device)
            b = self.bias if self.bias is not None else torch.zeros(self.hidden_size, dtype=h.dtype, device=h.device)
            y = ops.layer_norm(h, w, b, self.eps)
        else:
            y = _group_norm(h, self.num_groups, self.weight, self.bias, self.eps)
        return y, stream

    def forward(self, x, residual=None, prenorm: bool = False, residual_in_fp32: bool = False):
        y, stream = self._norm(x, residual, residual_in_fp32)
        return (y, stream) if prenorm else y

    def extra_repr(self) -> str:
        g = "" if self.num_groups is None else f"{self.num_groups}, "
        return f"{g}{self.hidden_size}, eps={self.eps}, affine={self.weight is not None}, bias={self.bias is not None}"


class RMSNorm(_NormBase):
    kind = "rms"


class LayerNorm(_NormBase):
    kind = "layer"


class GroupNorm(_NormBase):
    kind = "group"

    def __init__(self, num_groups: int, hidden_size: int, elementwise_affine: bool = True, bias: bool = False,
                 eps: float = 1e-5, dtype=None, device=None):
        super().__init__(hidden_size, elementwise_affine, bias, eps, num_groups=num_groups, dtype=dtype, device=device)


class _NormLinearMixin:
    """``forward(x, weight, bias, residual=None, prenorm=False, residual_in_fp32=False)`` = ``linear(norm(x + residual))``
    with the normalised activation recomputed in backward instead of stored."""

    def forward(self, x, weight, bias=None, residual=None, prenorm: bool = False, residual_in_fp32: bool = False):
        def run(x_, weight_, bias_, residual_):
            y, stream = self._norm(x_, residual_, residual_in_fp32)
            return ops.linear(y, weight_, bias_), stream

        if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, weight, bias, residual, self.weight)):
            out, stream = checkpoint(run, x, weight, bias, residual, use_reentrant=False)
        else:
            out, stream = run(x, weight, bias, residual)
        return (out, stream) if prenorm else out


class RMSNormLinear(_NormLinearMixin, RMSNorm):
    pass


class LayerNormLinear(_NormLinearMixin, LayerNorm):
    pass


class GroupNormLinear(_NormLinearMixin, GroupNorm):
    pass

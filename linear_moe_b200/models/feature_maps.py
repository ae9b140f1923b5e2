"""Feature maps for linear attention (reference: common_modules/feature_map.py:38-300).

All maps act on the last dimension of ``[B, T, H, d]`` tensors.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


def _outer_upper(x, y, offset: int = 0):
    z = torch.einsum("...i,...j->...ij", x, y)
    n = z.size(-1)
    iu = torch.triu_indices(n, n, offset, device=x.device)
    return z[..., iu[0], iu[1]]


def _outer_off1(x, y):
    z = torch.einsum("...i,...j->...ij", x, y)
    n = z.size(-1)
    iu = torch.triu_indices(n, n, 1, device=x.device)
    d = torch.arange(n, device=x.device)
    return z[..., iu[0], iu[1]], z[..., d, d]


class Hedgehog(nn.Module):
    def __init__(self, head_dim: int):
        super().__init__()
        self.layer = nn.Linear(head_dim, head_dim)
        with torch.no_grad():
            self.layer.weight.copy_(torch.eye(head_dim))
            self.layer.bias.zero_()

    def forward(self, x):
        x = self.layer(x)
        return torch.cat([2 * x, -2 * x], dim=-1).softmax(-1)


class T2R(nn.Module):
    def __init__(self, head_dim: int, dot_dim: Optional[int] = None, bias: bool = False):
        super().__init__()
        self.layer = nn.Linear(head_dim, dot_dim or head_dim, bias=bias)

    def forward(self, x):
        return self.layer(x).relu()


class DPFP(nn.Module):
    def __init__(self, head_dim: int, nu: int = 4):
        super().__init__()
        self.nu = nu

    def forward(self, x):
        x = torch.cat([x.relu(), -x.relu()], dim=-1)
        rolled = torch.cat([x.roll(shifts=j, dims=-1) for j in range(1, self.nu + 1)], dim=-1)
        return torch.cat([x] * self.nu, dim=-1) * rolled


class Hadamard(nn.Module):
    def __init__(self, head_dim: int):
        super().__init__()
        self.layer1 = nn.Linear(head_dim, head_dim)
        self.layer2 = nn.Linear(head_dim, head_dim)

    def forward(self, x):
        return self.layer1(x) * self.layer2(x)


class LearnableOuterProduct(nn.Module):
    def __init__(self, head_dim: int, feature_dim: int):
        super().__init__()
        self.layer1 = nn.Linear(head_dim, feature_dim, bias=False)
        self.layer2 = nn.Linear(head_dim, feature_dim, bias=False)

    def forward(self, x):
        return _outer_upper(self.layer1(x), self.layer2(x))


class LearnablePolySketch(nn.Module):
    def __init__(self, head_dim: int, sketch_size: Optional[int] = None, degree: int = 2):
        super().__init__()
        assert degree >= 2 and degree & (degree - 1) == 0
        self.head_dim, self.degree = head_dim, degree
        s = sketch_size or head_dim
        self.gamma = nn.Parameter(torch.ones(head_dim))
        self.beta = nn.Parameter(torch.zeros(head_dim))
        n_extra = max(int(math.log2(degree)) - 2, 0)
        self.sketches1 = nn.ModuleList([nn.Linear(head_dim, s, bias=False)] +
                                       [nn.Linear(s, s, bias=False) for _ in range(n_extra)])
        self.sketches2 = nn.ModuleList([nn.Linear(head_dim, s, bias=False)] +
                                       [nn.Linear(s, s, bias=False) for _ in range(n_extra)])

    def forward(self, x):
        x = F.layer_norm(x.float(), (self.head_dim,), self.gamma.float(), self.beta.float()).to(x.dtype)
        x = self.sketches1[0](x) * self.sketches2[0](x) * self.head_dim ** -0.5
        for i in range(1, len(self.sketches1)):
            x = self.sketches1[i](x) * self.sketches2[i](x) * self.head_dim ** -0.5
        return _outer_upper(x, x)


class Taylor(nn.Module):
    """2nd-order Taylor expansion of exp(q.k): features (1, x/d^(1/4), x_i^2/(sqrt2 sqrt d), x_i x_j/sqrt d)."""

    def __init__(self, head_dim: int):
        super().__init__()
        self.rd = math.sqrt(head_dim)
        self.rrd = math.sqrt(self.rd)
        self.r2 = math.sqrt(2)

    def forward(self, x):
        off, diag = _outer_off1(x, x)
        return torch.cat([torch.ones_like(x[..., :1]), x / self.rrd, diag / (self.rd * self.r2), off / self.rd], -1)


class RebasedMap(nn.Module):
    """Learnable affine layer norm followed by the quadratic map (feature_map.py:206-245)."""

    def __init__(self, head_dim: int, use_gamma=True, use_beta=True, normalize=True):
        super().__init__()
        self.head_dim, self.normalize = head_dim, normalize
        self.gamma = nn.Parameter(torch.ones(head_dim)) if use_gamma else None
        self.beta = nn.Parameter(torch.zeros(head_dim)) if use_beta else None

    def forward(self, x, flatten: bool = True):
        if self.normalize:
            x = F.layer_norm(x.float(), (self.head_dim,), self.gamma.float(), self.beta.float()).to(x.dtype)
        elif self.gamma is not None and self.beta is not None:
            x = torch.addcmul(self.beta, x, self.gamma)
        elif self.gamma is not None:
            x = x * self.gamma
        else:
            raise RuntimeError("unsupported combination of use_gamma/use_beta/normalize")
        if not flatten:
            return x
        off, diag = _outer_off1(x, x)
        return torch.cat([diag * self.head_dim ** -0.5, off * (2 / self.head_dim) ** 0.5], dim=-1)


class _Fn(nn.Module):
    def __init__(self, fn):
        super().__init__()
        self.fn = fn

    def forward(self, x):
        return self.fn(x)


def elu_p1(x):
    return F.elu(x) + 1.0


def keyed_init(module: nn.Module, key: str, device=None) -> nn.Module:
    """Re-draw every ``nn.Linear`` inside a learnable feature map from a generator seeded by ``(init seed, key)``, with
    ``nn.Linear``'s own bound ``1 / sqrt(fan_in)``: the constructor drew them from the process-global generator, which is
    seeded differently on every data- and context-parallel rank, so replicas would start from different weights.
    Hedgehog's identity initialisation is left alone."""
    from ..parallel.tensor_parallel import init_uniform
    if module is None or isinstance(module, Hedgehog):
        return module
    with torch.no_grad():
        for name, m in module.named_modules():
            if isinstance(m, nn.Linear):
                bound = 1.0 / math.sqrt(m.in_features)
                m.weight.copy_(init_uniform(tuple(m.weight.shape), -bound, bound, f"{key}.{name}.weight", device))
                if m.bias is not None:
                    m.bias.copy_(init_uniform(tuple(m.bias.shape), -bound, bound, f"{key}.{name}.bias", device))
    return module


def build_feature_map(name: Optional[str], head_dim: int, key: Optional[str] = None) -> Optional[nn.Module]:
    """``key``: parameter-name prefix that seeds the learnable maps' initial weights (same on every rank)."""
    if key is not None:
        return keyed_init(build_feature_map(name, head_dim), key)
    if name is None:
        return None
    simple = {
        "elu": elu_p1, "relu": F.relu, "identity": lambda x: x, "swish": F.silu, "silu": F.silu,
        "sigmoid": torch.sigmoid, "gelu": F.gelu, "sqrelu": lambda x: F.relu(x).pow(2),
    }
    if name in simple:
        return _Fn(simple[name])
    if name == "hedgehog":
        return Hedgehog(head_dim)
    if name == "t2r":
        return T2R(head_dim)
    if name == "elementwise_product":
        return Hadamard(head_dim)
    if name == "dpfp":
        return DPFP(head_dim)
    if name == "taylor":
        return Taylor(head_dim)
    if name == "rebased":
        return RebasedMap(head_dim)
    if name == "learnable_outer_product":
        return LearnableOuterProduct(head_dim, head_dim)
    if name == "polysketch":
        return LearnablePolySketch(head_dim)
    raise NotImplementedError(f"unsupported feature map {name!r}")

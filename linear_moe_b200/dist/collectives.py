"""Autograd-aware collectives over a :class:`~linear_moe_b200.dist.mesh.Group`.

Counterparts of the Megatron ``tensor_parallel.mappings`` the reference imports
(token_dispatcher.py:20-22,126-145,245,375,439,451,477,503,525,544;
router.py:339-344): gather/scatter/reduce along the first or last dimension, all-to-all
with uneven splits, and the sequence-parallel <-> hidden-parallel all-to-all.

Every function is the identity on a group of size 1, so single-process models need no
``torch.distributed`` at all.  On the gloo backend (CPU runs) reduce-scatter is emulated
with all-reduce + slice, since gloo has no reduce-scatter.  The fused P2P kernels of
:mod:`linear_moe_b200.parallel` replace these calls on the hot paths of GPU runs; what is
left here is control-plane traffic and the comparator path.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .mesh import Group


def _is_gloo(g: Group) -> bool:
    return dist.get_backend(g.pg) == "gloo"


# ---- raw (non-differentiable) ---------------------------------------------
def all_reduce_(x: torch.Tensor, g: Group, op=dist.ReduceOp.SUM) -> torch.Tensor:
    if not g.is_trivial:
        dist.all_reduce(x, op=op, group=g.pg)
    return x


def all_gather_raw(x: torch.Tensor, g: Group, dim: int = 0) -> torch.Tensor:
    if g.is_trivial:
        return x
    x = x.contiguous()
    if x.dim() == 0:
        x = x.reshape(1)
    out = torch.empty((g.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=g.pg)
    if dim == 0:
        return out
    return torch.cat(list(out.chunk(g.size, dim=0)), dim=dim)


def reduce_scatter_raw(x: torch.Tensor, g: Group, dim: int = 0) -> torch.Tensor:
    if g.is_trivial:
        return x
    if dim != 0:
        x = torch.cat(x.chunk(g.size, dim=dim), dim=0)
    x = x.contiguous()
    n = x.shape[0] // g.size
    if _is_gloo(g):
        dist.all_reduce(x, group=g.pg)
        return x[g.rank * n:(g.rank + 1) * n].clone()
    out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=g.pg)
    return out


def broadcast_(x: torch.Tensor, g: Group, src_group_rank: int = 0) -> torch.Tensor:
    if not g.is_trivial:
        dist.broadcast(x, src=g.ranks[src_group_rank], group=g.pg)
    return x


def all_to_all_raw(x: torch.Tensor, g: Group, out_splits: Optional[List[int]] = None,
                   in_splits: Optional[List[int]] = None) -> torch.Tensor:
    if g.is_trivial:
        return x
    x = x.contiguous()
    n_out = x.shape[0] if out_splits is None else sum(out_splits)
    out = torch.empty((n_out,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=g.pg)
    return out


# ---- differentiable --------------------------------------------------------
class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, dim):
        ctx.g, ctx.dim = g, dim
        return all_gather_raw(x, g, dim)

    @staticmethod
    def backward(ctx, gy):
        return reduce_scatter_raw(gy, ctx.g, ctx.dim), None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, dim):
        ctx.g, ctx.dim = g, dim
        return reduce_scatter_raw(x, g, dim)

    @staticmethod
    def backward(ctx, gy):
        return all_gather_raw(gy, ctx.g, ctx.dim), None, None


class _AllReduce(torch.autograd.Function):
    """Forward all-reduce, backward identity (row-parallel output)."""
    @staticmethod
    def forward(ctx, x, g):
        return all_reduce_(x.clone(), g)

    @staticmethod
    def backward(ctx, gy):
        return gy, None


class _CopyToRegion(torch.autograd.Function):
    """Forward identity, backward all-reduce (column-parallel input)."""
    @staticmethod
    def forward(ctx, x, g):
        ctx.g = g
        return x

    @staticmethod
    def backward(ctx, gy):
        return all_reduce_(gy.clone(), ctx.g), None


class _Scatter(torch.autograd.Function):
    """Forward keep own slice, backward all-gather."""
    @staticmethod
    def forward(ctx, x, g, dim):
        ctx.g, ctx.dim = g, dim
        return x.chunk(g.size, dim=dim)[g.rank].contiguous()

    @staticmethod
    def backward(ctx, gy):
        return all_gather_raw(gy, ctx.g, ctx.dim), None, None


class _GatherSlice(torch.autograd.Function):
    """Forward all-gather, backward keep own slice (no reduction): for tensors whose gradient
    is already identical on every rank of the group."""
    @staticmethod
    def forward(ctx, x, g, dim):
        ctx.g, ctx.dim = g, dim
        return all_gather_raw(x, g, dim)

    @staticmethod
    def backward(ctx, gy):
        return gy.chunk(ctx.g.size, dim=ctx.dim)[ctx.g.rank].contiguous(), None, None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, out_splits, in_splits):
        ctx.g, ctx.out_splits, ctx.in_splits = g, out_splits, in_splits
        return all_to_all_raw(x, g, out_splits, in_splits)

    @staticmethod
    def backward(ctx, gy):
        return all_to_all_raw(gy, ctx.g, ctx.in_splits, ctx.out_splits), None, None, None


def all_gather(x, g: Group, dim: int = 0):
    return x if g.is_trivial else _AllGather.apply(x, g, dim)


def reduce_scatter(x, g: Group, dim: int = 0):
    return x if g.is_trivial else _ReduceScatter.apply(x, g, dim)


def all_reduce(x, g: Group):
    return x if g.is_trivial else _AllReduce.apply(x, g)


def copy_to_region(x, g: Group):
    return x if g.is_trivial else _CopyToRegion.apply(x, g)


def scatter(x, g: Group, dim: int = 0):
    return x if g.is_trivial else _Scatter.apply(x, g, dim)


def gather_no_reduce(x, g: Group, dim: int = 0):
    return x if g.is_trivial else _GatherSlice.apply(x, g, dim)


def all_to_all(x, g: Group, out_splits=None, in_splits=None):
    return x if g.is_trivial else _AllToAll.apply(x, g, out_splits, in_splits)


def all_to_all_sp2hp(x, g: Group):
    """``[T/W, h] -> [T, h/W]``: trade sequence sharding for hidden sharding
    (token_dispatcher.py:439)."""
    if g.is_trivial:
        return x
    parts = torch.cat(x.chunk(g.size, dim=-1), dim=0)
    return all_to_all(parts, g)


def all_to_all_hp2sp(x, g: Group):
    """``[T, h/W] -> [T/W, h]`` (token_dispatcher.py:544)."""
    if g.is_trivial:
        return x
    y = all_to_all(x, g)
    return torch.cat(y.chunk(g.size, dim=0), dim=-1)

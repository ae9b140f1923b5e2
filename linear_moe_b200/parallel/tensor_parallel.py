"""Tensor-parallel linear layers, vocab-parallel embedding and LM head + cross entropy.

Counterparts of Megatron's ``ColumnParallelLinear`` / ``RowParallelLinear`` /
``VocabParallelEmbedding`` / ``vocab_parallel_cross_entropy`` which every layer spec of the
reference instantiates (qwen2/layer_specs.py:94-96,200-203; hybrid_model.py:20-22,211-221).

Activations are ``[B, T, h]``.  With ``sequence_parallel`` the tensors between TP regions are
sharded along T; a column-parallel layer then all-gathers its input along T and a
row-parallel layer reduce-scatters its output along T.  On CUDA these two pairs run as
fused AG->GEMM / GEMM->RS kernels over peer memory when the mesh has a symmetric-memory
workspace (``parallel/fused_tp.py``); otherwise the collectives of ``dist.collectives`` are
used.

Weights are created from a generator seeded by ``(seed, parameter key)`` at full (unsharded)
shape and then sliced, so a TP/EP-sharded model holds exactly the shards of the
single-process model with the same seed.
"""
from __future__ import annotations

import os

import hashlib
import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..dist import collectives as C
from ..dist.mesh import Mesh, single_process_mesh

_INIT_SEED = 1234


def set_init_seed(seed: int):
    global _INIT_SEED
    _INIT_SEED = int(seed)


def _key_seed(key: str) -> int:
    h = hashlib.sha256(f"{_INIT_SEED}:{key}".encode()).digest()
    return int.from_bytes(h[:8], "little") % (2 ** 63 - 1)


def init_normal(shape, std: float, key: str, device=None, dtype=torch.float32) -> torch.Tensor:
    """N(0, std) tensor that depends only on (global init seed, key, shape)."""
    device = torch.device(device) if device is not None else torch.device("cpu")
    gen = torch.Generator(device=device)
    gen.manual_seed(_key_seed(key))
    w = torch.empty(shape, dtype=torch.float32, device=device)
    w.normal_(0.0, std, generator=gen)
    return w.to(dtype)


def init_uniform(shape, lo: float, hi: float, key: str, device=None, dtype=torch.float32) -> torch.Tensor:
    device = torch.device(device) if device is not None else torch.device("cpu")
    gen = torch.Generator(device=device)
    gen.manual_seed(_key_seed(key))
    w = torch.empty(shape, dtype=torch.float32, device=device)
    w.uniform_(lo, hi, generator=gen)
    return w.to(dtype)


class ColumnParallelLinear(nn.Module):
    """``y = x W^T (+ b)`` with W ``[out, in]`` split along ``out`` over the TP group.

    ``stride`` > 1 splits a fused weight (e.g. gate|up for SwiGLU) per part, so each rank
    holds ``[part0_shard; part1_shard; ...]`` (mlp.py:157-230 keeps the same convention in
    its sharded state dict); ``part_sizes`` does the same for parts of unequal width (Mamba2 in_proj).  ``group_size`` splits in units of rows (a GQA query group, a head)."""

    def __init__(self, in_features: int, out_features: int, *, mesh: Optional[Mesh] = None, bias: bool = False,
                 std: float = 0.02, key: str = "", gather_output: bool = False, sequence_parallel: bool = False,
                 stride: int = 1, dtype=torch.float32, device=None, is_expert: bool = False,
                 part_sizes=None):
        super().__init__()
        self.mesh = mesh or single_process_mesh()
        tp = self.mesh.tp
        self.part_sizes = list(part_sizes) if part_sizes is not None else None
        if self.part_sizes is not None:
            assert sum(self.part_sizes) == out_features and all(p % tp == 0 for p in self.part_sizes)
        assert out_features % (tp * stride) == 0, (out_features, tp, stride)
        self.in_features, self.out_features = in_features, out_features
        self.out_per_rank = out_features // tp
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel and tp > 1
        full = init_normal((out_features, in_features), std, key + ".weight", device)
        self.weight = nn.Parameter(self._shard(full, stride).to(dtype))
        self.weight.tensor_parallel = tp > 1
        self.weight.partition_dim, self.weight.partition_stride = 0, stride
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.out_per_rank, dtype=dtype, device=device))
            self.bias.tensor_parallel, self.bias.partition_dim, self.bias.partition_stride = tp > 1, 0, stride
        else:
            self.register_parameter("bias", None)

    def _shard(self, full: torch.Tensor, stride: int) -> torch.Tensor:
        tp, r = self.mesh.tp, self.mesh.tp_rank
        if tp == 1:
            return full
        parts = full.split(self.part_sizes, dim=0) if self.part_sizes is not None else full.chunk(stride, dim=0)
        return torch.cat([p.chunk(tp, dim=0)[r] for p in parts], dim=0).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g = self.mesh["tp"]
        if self.sequence_parallel:
            y = ops.allgather_linear(x, self.weight, self.bias, g, dim=1)
        else:
            x = C.copy_to_region(x, g)
            y = ops.linear(x, self.weight, self.bias)
        if self.gather_output:
            y = C.all_gather(y, g, dim=-1)
        return y


class RowParallelLinear(nn.Module):
    """``y = x W^T (+ b)`` with W ``[out, in]`` split along ``in``; partial sums are all-reduced, or
    reduce-scattered along T under sequence parallelism."""

    def __init__(self, in_features: int, out_features: int, *, mesh: Optional[Mesh] = None, bias: bool = False,
                 std: float = 0.02, key: str = "", input_is_parallel: bool = True, sequence_parallel: bool = False,
                 dtype=torch.float32, device=None, is_expert: bool = False):
        super().__init__()
        self.mesh = mesh or single_process_mesh()
        tp = self.mesh.tp
        assert in_features % tp == 0
        self.in_features, self.out_features = in_features, out_features
        self.input_is_parallel, self.sequence_parallel = input_is_parallel, sequence_parallel and tp > 1
        full = init_normal((out_features, in_features), std, key + ".weight", device)
        w = full.chunk(tp, dim=1)[self.mesh.tp_rank].contiguous() if tp > 1 else full
        self.weight = nn.Parameter(w.to(dtype))
        self.weight.tensor_parallel, self.weight.partition_dim, self.weight.partition_stride = tp > 1, 1, 1
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g = self.mesh["tp"]
        if not self.input_is_parallel:
            x = C.scatter(x, g, dim=-1)
        if self.sequence_parallel:
            y = ops.linear_reducescatter(x, self.weight, g, dim=1)
        else:
            y = C.all_reduce(ops.linear(x, self.weight, None), g)
        if self.bias is not None:
            y = y + self.bias
        return y


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary; out-of-shard ids contribute zero and the partial
    results are summed (or reduce-scattered along T under sequence parallelism)."""

    def __init__(self, vocab: int, hidden: int, *, mesh: Optional[Mesh] = None, std: float = 0.02,
                 key: str = "embedding.word_embeddings", sequence_parallel: bool = False,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.mesh = mesh or single_process_mesh()
        tp = self.mesh.tp
        assert vocab % tp == 0
        self.vocab, self.per_rank = vocab, vocab // tp
        self.start = self.mesh.tp_rank * self.per_rank
        self.sequence_parallel = sequence_parallel and tp > 1
        full = init_normal((vocab, hidden), std, key + ".weight", device)
        self.weight = nn.Parameter(full[self.start:self.start + self.per_rank].clone().to(dtype))
        self.weight.tensor_parallel, self.weight.partition_dim, self.weight.partition_stride = tp > 1, 0, 1

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        g = self.mesh["tp"]
        if g.is_trivial:
            return ops.embedding(ids, self.weight)
        e = ops.embedding(ids, self.weight, self.start, sharded=True)
        if self.sequence_parallel:
            return C.reduce_scatter(e, g, dim=1)
        return C.all_reduce(e, g)


def _ce_kernel_labels(labels, vocab_start, width, ignore_index):
    """Labels as the per-shard kernels want them: the local column for targets inside this shard, ``ignore_index`` for
    ignored rows, and for rows whose target lives in another shard a value that matches no column (the row still gets
    the softmax part of its gradient)."""
    local = labels - vocab_start
    inshard = (local >= 0) & (local < width) & (labels != ignore_index)
    nowhere = -1 if ignore_index != -1 else -2
    fwd = torch.where(inshard, local, torch.full_like(local, ignore_index))
    bwd = torch.where(labels != ignore_index, torch.where(inshard, local, torch.full_like(local, nowhere)),
                      torch.full_like(local, ignore_index))
    return inshard, fwd, bwd


def vocab_shard_stats(logits2d, labels1d, vocab_start, ignore_index):
    """Per-shard statistics of the vocabulary-parallel cross entropy on the softmax kernels: the log-sum-exp over this
    shard's columns and the target logit where the target is in the shard (0 elsewhere).  No ``[tokens, vocab]``
    temporary is made."""
    K = ops._K()
    T = logits2d.shape[0]
    inshard, lab_fwd, lab_bwd = _ce_kernel_labels(labels1d, vocab_start, logits2d.shape[1], ignore_index)
    loss = torch.empty(T, dtype=torch.float32, device=logits2d.device)
    lse = torch.empty(T, dtype=torch.float32, device=logits2d.device)
    K.softmax_ce_fwd(logits2d, lab_fwd, loss, lse, ignore_index)
    tgt = torch.where(inshard, lse - loss, torch.zeros_like(lse))
    return lse, tgt, lab_bwd


class _VocabParallelCE(torch.autograd.Function):
    """Cross entropy over logits split along the vocabulary (``vocab_parallel_cross_entropy`` of the reference's engine).

    CUDA: every rank runs the softmax kernels on its shard (log-sum-exp and target logit per token), ONE all-gather
    exchanges the two numbers per token, and the backward kernel turns the shard's logits into its gradient in place with
    the global log-sum-exp; nothing of size ``[tokens, vocab]`` is allocated.  CPU (gloo tests): the eager form with three
    all-reduces (max, sum-exp, target logit)."""

    @staticmethod
    def forward(ctx, logits, labels, g, vocab_start, ignore_index):
        if logits.is_cuda and os.environ.get("LMOE_TP_CE_KERNEL", "1") != "0":
            l2 = logits.reshape(-1, logits.shape[-1])
            if not l2.is_contiguous():
                l2 = l2.contiguous()
            lab = labels.reshape(-1)
            lse_loc, tgt_loc, lab_bwd = vocab_shard_stats(l2, lab, vocab_start, ignore_index)
            both = C.all_gather_raw(torch.stack([lse_loc, tgt_loc])[None].contiguous(), g, dim=0)     # [tp, 2, T]
            lse = torch.logsumexp(both[:, 0], dim=0)
            tgt = both[:, 1].sum(0)
            valid = lab != ignore_index
            loss = torch.where(valid, lse - tgt, torch.zeros_like(lse))
            ctx.save_for_backward(l2, lab_bwd, lse)
            ctx.kernel, ctx.ignore, ctx.shape = True, ignore_index, logits.shape
            return loss.reshape(labels.shape)
        ctx.kernel = False
        lf = logits.float()
        m = lf.max(-1).values
        C.all_reduce_(m, g, op=torch.distributed.ReduceOp.MAX)
        ex = (lf - m[..., None]).exp()
        se = ex.sum(-1)
        C.all_reduce_(se, g)
        local = labels - vocab_start
        inshard = (local >= 0) & (local < lf.shape[-1]) & (labels != ignore_index)
        tgt = lf.gather(-1, local.clamp(0, lf.shape[-1] - 1)[..., None]).squeeze(-1)
        tgt = torch.where(inshard, tgt, torch.zeros_like(tgt))
        C.all_reduce_(tgt, g)
        valid = labels != ignore_index
        loss = torch.where(valid, se.log() + m - tgt, torch.zeros_like(tgt))
        ctx.save_for_backward(ex / se[..., None], local, inshard, valid)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, gl):
        if ctx.kernel:
            l2, lab_bwd, lse = ctx.saved_tensors
            # the logits are this node's alone (the LM head's output): they are overwritten with their gradient
            grad = ops._K().softmax_ce_bwd(l2, lab_bwd, lse, gl.reshape(-1).float().contiguous(), ctx.ignore)
            return grad.view(ctx.shape), None, None, None, None
        p, local, inshard, valid = ctx.saved_tensors
        grad = p.clone()
        idx = local.clamp(0, p.shape[-1] - 1)[..., None]
        grad.scatter_add_(-1, idx, -inshard[..., None].float())
        grad = grad * (gl * valid.float())[..., None]
        return grad.to(ctx.dtype), None, None, None, None


class LMHead(nn.Module):
    """Column-parallel output projection fused with the per-token cross entropy.

    With labels, the ``[tokens, vocab]`` logits are never materialised for the whole batch: the
    projection and the loss run per chunk of ``cross_entropy_chunk`` tokens
    (``ops.linear_cross_entropy``).  Without labels it returns logits (gathered over TP unless
    ``parallel_output``)."""

    def __init__(self, hidden: int, vocab: int, *, mesh: Optional[Mesh] = None, std: float = 0.02,
                 key: str = "output_layer", tied: Optional[nn.Parameter] = None, chunk: int = 4096,
                 sequence_parallel: bool = False, dtype=torch.float32, device=None):
        super().__init__()
        self.mesh = mesh or single_process_mesh()
        tp = self.mesh.tp
        self.vocab, self.per_rank, self.chunk = vocab, vocab // tp, chunk
        self.start = self.mesh.tp_rank * self.per_rank
        self.sequence_parallel = sequence_parallel and tp > 1
        if tied is not None:
            self.weight = tied
        else:
            full = init_normal((vocab, hidden), std, key + ".weight", device)
            self.weight = nn.Parameter(full[self.start:self.start + self.per_rank].clone().to(dtype))
            self.weight.tensor_parallel, self.weight.partition_dim, self.weight.partition_stride = tp > 1, 0, 1

    def forward(self, h: torch.Tensor, labels: Optional[torch.Tensor] = None, parallel_output: bool = False,
                ignore_index: int = -100):
        g = self.mesh["tp"]
        if self.sequence_parallel:
            h = C.all_gather(h, g, dim=1)
        else:
            h = C.copy_to_region(h, g)
        if labels is None:
            logits = ops.linear(h, self.weight, None)
            return logits if parallel_output else C.gather_no_reduce(logits, g, dim=-1)
        if g.is_trivial:
            return ops.linear_cross_entropy(h.reshape(-1, h.shape[-1]), self.weight, labels.reshape(-1),
                                            ignore_index=ignore_index, chunk=self.chunk).reshape(labels.shape)
        logits = ops.linear(h, self.weight, None)
        return _VocabParallelCE.apply(logits, labels, g, self.start, ignore_index)

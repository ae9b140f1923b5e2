"""Gradient buffers, data-parallel reduction and the mixed-precision Adam optimizer (with ZeRO-1).

This one module plays the roles of Megatron's ``DistributedDataParallel`` (contiguous grad
buffers, fp32 accumulation, bucketed reduce), ``Float16OptimizerWithFloat16Params`` /
``DistributedOptimizer`` (fp32 master weights, reduce-scatter -> shard update -> all-gather),
gradient clipping by global norm and Apex ``FusedAdam`` — the external pieces the reference
reaches through ``setup_model_and_optimizer`` / ``optimizer.step`` (training.py:113,278-298,
343-351; run_pretrain_qwen.sh:321-328).

Layout (B200-first): parameters are grouped into at most four *flat* buffers —
(dense | expert) x (weight-decay | no-weight-decay).  Each buffer holds the model-dtype
parameters, an fp32 gradient accumulator, and fp32 master / exp_avg / exp_avg_sq either in full or,
under ZeRO-1, only for this rank's contiguous shard.  Module parameters are views into the flat
parameter buffer, so an optimizer step is ONE fused kernel per buffer
(``ops.cuda.fused_adam``) and a gradient reduction is ONE collective per buffer — or, with the
symmetric-memory workspace, the fused reduce-scatter + Adam + all-gather kernel over NVLS
(``ops.cuda.zero1_fused_step``), no NCCL.

Reduction groups: dense parameters average over ``dp_cp``; expert parameters sum over ``edp``
and are scaled by ``1/(dp*cp)`` (their gradients already contain the tokens of the whole EP group;
experts.py:153-154 ``allreduce=False``).  Parameters tagged ``sequence_parallel_grad`` (norm
weights, router, shared-expert gate) are additionally summed over TP under sequence parallelism.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config.model_config import TrainConfig
from ..dist import collectives as C
from ..dist.mesh import Group, Mesh

_ALIGN = 128


def _no_weight_decay(name: str, p: nn.Parameter) -> bool:
    return getattr(p, "_no_weight_decay", False) or p.dim() <= 1 or name.endswith(".bias")


@dataclass
class _Slot:
    name: str
    param: nn.Parameter
    start: int
    numel: int


class FlatBuffer:
    """One flat parameter/gradient buffer and its optimizer state."""

    def __init__(self, slots: List[Tuple[str, nn.Parameter]], *, expert: bool, weight_decay: bool, group: Group,
                 grad_scale: float, zero1: bool, master: bool, symmetric: bool = False):
        self.expert, self.weight_decay, self.group, self.grad_scale, self.zero1 = expert, weight_decay, group, grad_scale, zero1
        p0 = slots[0][1]
        self.device, self.dtype = p0.device, p0.dtype
        self.slots: List[_Slot] = []
        off = 0
        for name, p in slots:
            self.slots.append(_Slot(name, p, off, p.numel()))
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        shard_mult = _ALIGN * (group.size if zero1 else 1)
        self.numel = (off + shard_mult - 1) // shard_mult * shard_mult
        self.fused = None
        if symmetric and self.dtype == torch.bfloat16:
            # parameters and gradients live in symmetric memory so that the fused ZeRO-1 kernels can reduce the
            # gradients and broadcast the parameters through NVSwitch without NCCL
            from ..parallel.fused_comm import ZeroBufferWorkspace
            self.fused = ZeroBufferWorkspace(group, self.numel, self.device)
            self.params, self.grads = self.fused.params, self.fused.grads
            self.params.zero_(), self.grads.zero_()
        else:
            self.params = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
            self.grads = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        for s in self.slots:
            view = self.params[s.start:s.start + s.numel].view_as(s.param)
            view.copy_(s.param.data)
            s.param.data = view
            s.param.main_grad = self.grads[s.start:s.start + s.numel].view_as(s.param)
        if zero1 and group.size > 1:
            n = self.numel // group.size
            self.shard = (group.rank * n, (group.rank + 1) * n)
        else:
            self.shard = (0, self.numel)
        lo, hi = self.shard
        self.master = self.params[lo:hi].float().clone() if master else None
        self.exp_avg = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
        # tensor-parallel duplicates are counted once in the gradient norm: mask of slots that are
        # replicated over TP (norm weights, router, ...)
        self.tp_dup = [not getattr(s.param, "tensor_parallel", False) for s in self.slots]

    def shard_view(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.shard[0]:self.shard[1]]

    def reload_master(self):
        """Refresh fp32 masters from the model parameters (``optimizer.reload_model_params()``,
        finetune_utils.py:317-327)."""
        if self.master is not None:
            self.master.copy_(self.shard_view(self.params).float())


class MixedPrecisionAdam:
    """AdamW over flat buffers with fp32 masters, global-norm clipping, optional dynamic loss scaling
    and optional ZeRO-1 sharding over the data-parallel group."""

    def __init__(self, model: nn.Module, mesh: Mesh, tc: TrainConfig, *, zero1: bool = False,
                 sequence_parallel: bool = False, fused_comm: bool = True, overlap_grad_reduce: bool = False):
        self.mesh, self.tc, self.zero1 = mesh, tc, zero1 and (mesh.dp * mesh.cp) > 1
        self.overlap_grad_reduce = overlap_grad_reduce
        self.overlap_active = False            # set by the schedule while the LAST micro-batch's backward runs
        # CTAs of a bucket reduce launched next to the backward pass: few, so that the GEMMs keep their SMs
        self.bucket_blocks = int(os.environ.get("LMOE_ZERO_BUCKET_BLOCKS", "48"))
        self._side_stream = None
        self._bucket_state = None              # per fused buffer: list of [lo, hi) ranges already reduced this step
        self.sequence_parallel = sequence_parallel and mesh.tp > 1
        self.fused_comm = fused_comm
        self.step_count = 0
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        seen, uniq = set(), []
        for n, p in named:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        self.named = uniq
        self._tp_partial = mesh.tp > 1 and any(getattr(p, "tp_partial_grad", False) for _, p in uniq)
        self._pp_shared = any(getattr(p, "pp_shared_grad", None) is not None for _, p in uniq)
        groups: Dict[Tuple[bool, bool], List[Tuple[str, nn.Parameter]]] = {}
        for n, p in uniq:
            key = (bool(getattr(p, "expert_parallel", False)), not _no_weight_decay(n, p))
            groups.setdefault(key, []).append((n, p))
        dpcp = mesh.dp * mesh.cp
        self.buffers: List[FlatBuffer] = []
        for (expert, wd), slots in sorted(groups.items()):
            g = mesh["edp"] if expert else mesh["dp_cp"]
            by_dtype: Dict[torch.dtype, list] = {}
            for n, p in slots:
                by_dtype.setdefault(p.dtype, []).append((n, p))
            for dt, sl in by_dtype.items():
                self.buffers.append(FlatBuffer(sl, expert=expert, weight_decay=wd, group=g, grad_scale=1.0 / dpcp,
                                               zero1=self.zero1, master=dt != torch.float32,
                                               symmetric=self._want_fused(g, dt)))
        self._hooks = []
        for n, p in uniq:
            self._hooks.append(p.register_post_accumulate_grad_hook(self._accumulate))
        # loss scaling (fp16 only)
        self.loss_scale = None
        if tc.fp16:
            self.loss_scale = tc.loss_scale if tc.loss_scale else tc.initial_loss_scale
            self._growth_tracker, self._hysteresis = 0, tc.hysteresis
        self.dynamic_scale = tc.fp16 and not tc.loss_scale
        self.skipped_iters = 0

    def _want_fused(self, group: Group, dtype) -> bool:
        """Symmetric-memory buffers + fused NVLS kernels: ZeRO-1 on a multi-GPU NCCL group with bf16 parameters."""
        if self.tc.optimizer != "adam":
            return False                         # the fused update kernel is Adam
        if not (self.zero1 and self.fused_comm and not group.is_trivial and dtype == torch.bfloat16):
            return False
        return torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl"

    # ------------------------------------------------------------------
    @staticmethod
    def _accumulate(p: nn.Parameter):
        if p.grad is not None:
            if getattr(p, "_direct_wgrad", False) and getattr(p, "_main_grad_fresh", False):
                p.main_grad.zero_()            # its accumulator is not cleared by zero_grad (direct weights): clear it now
            if p.grad.is_cuda and p.grad.dtype in (torch.bfloat16, torch.float32) and p.grad.is_contiguous():
                from ..ops import cuda as K
                K.accumulate_grad(p.main_grad, p.grad)      # one pass: fp32 accumulator += bf16 gradient
            else:
                p.main_grad.add_(p.grad.to(torch.float32))
            p.grad = None
            p._main_grad_fresh = False

    def zero_grad(self):
        """Clear the fp32 accumulators.  A weight whose gradient GEMM stores straight into its accumulator (the first
        write after this call overwrites, ``_main_grad_fresh``) needs no clearing, so once such weights are known only the
        remaining ranges (norm weights, biases, the embedding table, padding) are zeroed: for the 1.7 B-parameter
        benchmark model that is 1 GB instead of 6.7 GB per step.  ``reduce_grads`` clears a direct weight that was not
        written in a step."""
        for b in self.buffers:
            direct = [bool(getattr(s.param, "_direct_wgrad", False)) for s in b.slots]
            if not any(direct) or os.environ.get("LMOE_SKIP_ZERO", "1") == "0":
                b.grads.zero_()
                continue
            key = tuple(direct)
            if getattr(b, "_zero_key", None) != key:
                ranges, pos = [], 0
                for s, d in zip(b.slots, direct):
                    if d:
                        if s.start > pos:
                            ranges.append((pos, s.start))
                        pos = s.start + s.numel
                if pos < b.numel:
                    ranges.append((pos, b.numel))
                b._zero_key, b._zero_ranges = key, ranges
            for lo, hi in b._zero_ranges:
                b.grads[lo:hi].zero_()
        for _, p in self.named:
            p.grad = None
            p._main_grad_fresh = True          # the next direct weight-gradient GEMM may overwrite instead of add

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss if self.loss_scale is None else loss * self.loss_scale

    # ------------------------------------------------------------------
    def _reduce_sequence_parallel_grads(self):
        """Complete, over the tensor-parallel group, the gradients of replicated parameters that every rank computes
        from only part of the data: those applied to the sequence-sharded stream under sequence parallelism
        (``sequence_parallel_grad``: norm weights, router) and those applied per head to the rank's own heads
        (``tp_partial_grad``: per-head output norms, q / k layer norms, learnable feature maps).  One all-reduce."""
        if self.mesh.tp <= 1:
            return
        g = self.mesh["tp"]
        ts = [p.main_grad for _, p in self.named
              if getattr(p, "tp_partial_grad", False) or (self.sequence_parallel and getattr(p, "sequence_parallel_grad", False))]
        if ts:
            flat = torch.cat([t.reshape(-1) for t in ts])
            C.all_reduce_(flat, g)
            off = 0
            for t in ts:
                t.copy_(flat[off:off + t.numel()].view_as(t))
                off += t.numel()

    def _reduce_pipeline_shared_grads(self):
        """Sum the gradients of parameters that live on more than one pipeline stage (or model chunk of a stage):
        ``pp_shared_grad == "all"``: a copy on every stage and chunk (HGRN2's lower-bound table), summed over the local
        chunks and all-reduced over the pipeline group; ``"embedding"``: the tied word embedding on the first stage and
        its copy under the LM head on the last (Megatron's embedding group), exchanged point to point.  Every copy then
        holds the full gradient and receives the same update."""
        if not self._pp_shared:
            return
        import torch.distributed as dist
        g = self.mesh["pp"]
        every = [p for _, p in self.named if getattr(p, "pp_shared_grad", None) == "all"]
        if every:
            by_shape: Dict[Tuple[int, ...], List[nn.Parameter]] = {}
            for p in every:
                by_shape.setdefault(tuple(p.shape), []).append(p)
            for ps in by_shape.values():                     # one table per model chunk on this stage: same shape
                total = ps[0].main_grad.clone()
                for p in ps[1:]:
                    total += p.main_grad
                if not g.is_trivial:
                    C.all_reduce_(total, g)
                for p in ps:
                    p.main_grad.copy_(total)
        tied = [p for _, p in self.named if getattr(p, "pp_shared_grad", None) == "embedding"]
        if tied and not g.is_trivial:
            first, last = g.ranks[0], g.ranks[-1]
            for p in tied:
                grad = p.main_grad
                if self.mesh.rank == last:
                    dist.send(grad, dst=first, group=g.pg)
                    dist.recv(grad, src=first, group=g.pg)
                elif self.mesh.rank == first:
                    other = torch.empty_like(grad)
                    dist.recv(other, src=last, group=g.pg)
                    grad += other
                    dist.send(grad, dst=last, group=g.pg)

    def _is_shared_copy(self, p) -> bool:
        """A parameter whose gradient was summed into an identical copy elsewhere and must be counted once in the
        gradient norm: the owner is the first pipeline stage (first model chunk)."""
        tag = getattr(p, "pp_shared_grad", None)
        if tag is None:
            return False
        if self.mesh.pp_rank != 0:
            return True
        if tag == "all":
            first = next(q for _, q in self.named if getattr(q, "pp_shared_grad", None) == "all" and q.shape == p.shape)
            return first is not p
        return False

    # ---- gradient reduction overlapped with the backward pass (--overlap-grad-reduce) -------------------------------
    def _layer_range(self, b: "FlatBuffer", layer: int):
        """``[lo, hi)`` of the flat buffer holding the parameters of ``decoder.layers.<layer>`` (contiguous: slots are in
        model order), or None."""
        cache = b.__dict__.setdefault("_layer_ranges", {})
        if layer not in cache:
            # slot names carry the position of the model chunk in the optimizer's module list ("0.decoder.layers.3...")
            pre = f"decoder.layers.{layer}."
            sl = [s for s in b.slots if s.name.startswith(pre) or f".{pre}" in s.name]
            cache[layer] = None if not sl else (min(s.start for s in sl), max(s.start + s.numel for s in sl))
        return cache[layer]

    def bucket_ready(self, layer: int):
        """Called from the backward pass when every gradient of block ``layer`` has been written (a hook on the block's
        input): the reduce-scatter of that block's range starts at once on a side stream, overlapping the backward of the
        blocks before it (Megatron's ``overlap_grad_reduce``, training.py:278-298).  Only the fused NVLS buffers and only
        the last micro-batch of a step take part; everything else is reduced by :meth:`reduce_grads`."""
        if not (self.overlap_grad_reduce and self.overlap_active) or self.sequence_parallel or self._tp_partial \
                or self._pp_shared:
            return                    # gradients that still need the tensor-parallel all-reduce must not be reduced early
        fused = [b for b in self.buffers if b.fused is not None]
        if not fused:
            return
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream()
        main = torch.cuda.current_stream()
        if self._bucket_state is None:
            self._bucket_state = {}
            for b in fused:
                b.fused.begin_step()
                self._bucket_state[id(b)] = []
        ev = torch.cuda.Event()
        ev.record(main)
        self._side_stream.wait_event(ev)
        with torch.cuda.stream(self._side_stream):
            for b in fused:
                r = self._layer_range(b, layer)
                if r is None:
                    continue
                b.fused.reduce_range(r[0], r[1], b.shard, b.grad_scale, blocks=self.bucket_blocks)
                self._bucket_state[id(b)].append(r)

    def _finish_bucketed_with(self, b: "FlatBuffer", state):
        """Reduce what the hooks did not cover (embedding, final norm, LM head, padding) after the backward pass."""
        done = sorted(state[id(b)])
        pos = 0
        for lo, hi in done + [(b.numel, b.numel)]:
            if lo > pos:
                b.fused.reduce_range(pos, lo, b.shard, b.grad_scale, blocks=None)
            pos = max(pos, hi)

    def reduce_grads(self):
        """Data-parallel reduction of every buffer: all-reduce, or reduce-scatter into this rank's
        shard under ZeRO-1 (the rest of the buffer is then stale until the next zero_grad)."""
        for _, p in self.named:                 # a direct weight that saw no gradient this step still holds the last one
            if getattr(p, "_direct_wgrad", False) and getattr(p, "_main_grad_fresh", False):
                p.main_grad.zero_()
        self._reduce_sequence_parallel_grads()
        self._reduce_pipeline_shared_grads()
        bucketed = self._bucket_state
        self._bucket_state = None
        if bucketed is not None:
            torch.cuda.current_stream().wait_stream(self._side_stream)
        for b in self.buffers:
            if b.fused is not None and bucketed is not None:
                self._finish_bucketed_with(b, bucketed)
                continue
            if b.fused is not None:
                # barrier + in-switch reduce-scatter + scale + partial sum of squares, one kernel, no NCCL
                b.fused.reduce(b.shard, b.grad_scale)
                continue
            if b.grad_scale != 1.0:
                b.grads.mul_(b.grad_scale)
            g = b.group
            if g.is_trivial:
                continue
            if self.zero1:
                out = C.reduce_scatter_raw(b.grads, g, dim=0)
                b.shard_view(b.grads).copy_(out)
            else:
                C.all_reduce_(b.grads, g)

    # ------------------------------------------------------------------
    def _grad_sq_and_finite(self) -> Tuple[torch.Tensor, torch.Tensor]:
        mesh = self.mesh
        dev = self.buffers[0].device
        dense = torch.zeros((), dtype=torch.float32, device=dev)
        expert = torch.zeros((), dtype=torch.float32, device=dev)
        for b in self.buffers:
            lo, hi = b.shard
            if mesh.tp > 1 and mesh.tp_rank != 0:
                # drop TP-replicated parameters from all but TP rank 0
                sq = torch.zeros((), dtype=torch.float32, device=dev)
                for s, dup in zip(b.slots, b.tp_dup):
                    if dup:
                        continue
                    a, e = max(s.start, lo), min(s.start + s.numel, hi)
                    if e > a:
                        sq = sq + torch.linalg.vector_norm(b.grads[a:e]).square()
            else:
                sq = torch.linalg.vector_norm(b.grads[lo:hi]).square()
            for s, dup in (zip(b.slots, b.tp_dup) if self._pp_shared else ()):   # copies of pipeline-shared parameters count once
                if self._is_shared_copy(s.param) and not (dup and mesh.tp > 1 and mesh.tp_rank != 0):
                    a, e = max(s.start, lo), min(s.start + s.numel, hi)
                    if e > a:
                        sq = sq - torch.linalg.vector_norm(b.grads[a:e]).square()
            if b.expert:
                expert = expert + sq
            else:
                dense = dense + sq
        if self.zero1:
            C.all_reduce_(dense, mesh["dp_cp"])
            C.all_reduce_(expert, mesh["edp"])
        C.all_reduce_(expert, mesh["ep"])
        total = dense + expert
        C.all_reduce_(total, mesh["mp"])
        return total, torch.isfinite(total)

    @torch.no_grad()
    def step(self, lr: float, weight_decay: float, pre_update=None) -> Tuple[bool, Optional[float], int]:
        """Returns (update_successful, grad_norm, num_zeros_in_grad) like Megatron's optimizer.step
        (training.py:343-351).  ``pre_update`` is called after the gradient norm is known (the device is synchronised
        then) and before any parameter is touched; it may raise to abandon the step."""
        tc = self.tc
        inv_scale = 1.0 if self.loss_scale is None else 1.0 / self.loss_scale
        total_sq, finite = self._grad_sq_and_finite()
        if self.loss_scale is not None:
            ok = bool(finite)
            self._update_loss_scale(ok)
            if not ok:
                self.skipped_iters += 1
                return False, None, 0
        grad_norm = float(total_sq.sqrt()) * inv_scale if (tc.clip_grad > 0 or tc.log_interval) else None
        clip = 1.0
        if tc.clip_grad > 0 and grad_norm is not None and math.isfinite(grad_norm):
            clip = min(1.0, tc.clip_grad / (grad_norm + 1e-6))
        if grad_norm is None and pre_update is not None and total_sq.is_cuda:
            torch.cuda.synchronize()
        if pre_update is not None:
            pre_update()
        if grad_norm is not None and not math.isfinite(grad_norm) and tc.check_for_nan_in_loss_and_grad:
            raise FloatingPointError(f"non-finite gradient norm {grad_norm} on rank {self.mesh.rank}")
        self.step_count += 1
        b1, b2, eps = tc.adam_beta1, tc.adam_beta2, tc.adam_eps
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        gscale = inv_scale * clip
        for b in self.buffers:
            lo, hi = b.shard
            wd = weight_decay if b.weight_decay else 0.0
            g = b.grads[lo:hi]
            pshard = b.params[lo:hi]
            if tc.optimizer == "sgd":
                # --optimizer sgd: torch.optim.SGD's rule (L2 weight decay added to the gradient, momentum buffer in the
                # first-moment slot, no dampening / Nesterov), in eager tensor ops on the flat shard
                w = b.master if b.master is not None else pshard
                gg = g.float() * gscale
                if wd:
                    gg = gg.add(w.float(), alpha=wd)
                if tc.sgd_momentum:
                    gg = b.exp_avg.mul_(tc.sgd_momentum).add_(gg)
                w.add_(gg.to(w.dtype), alpha=-lr)
                if b.master is not None:
                    pshard.copy_(w)
                if self.zero1 and not b.group.is_trivial:
                    b.params.copy_(C.all_gather_raw(pshard.clone(), b.group, dim=0))
                continue
            if b.fused is not None:
                # Adam on the shard + multicast store of the bf16 parameters to every rank + barrier, one kernel
                b.fused.adam_broadcast(b.shard, b.master, b.exp_avg, b.exp_avg_sq, lr, b1, b2, eps, wd, bc1, bc2, gscale)
                continue
            if g.is_cuda:
                from ..ops import cuda as K
                K.fused_adam(pshard, b.master, g, b.exp_avg, b.exp_avg_sq, lr, b1, b2, eps, wd, bc1, bc2, gscale)
            else:
                w = b.master if b.master is not None else pshard
                gg = g * gscale
                b.exp_avg.mul_(b1).add_(gg, alpha=1 - b1)
                b.exp_avg_sq.mul_(b2).addcmul_(gg, gg, value=1 - b2)
                denom = (b.exp_avg_sq / bc2).sqrt_().add_(eps)
                w.mul_(1.0 - lr * wd).addcdiv_(b.exp_avg / bc1, denom, value=-lr)
                if b.master is not None:
                    pshard.copy_(w)
            if self.zero1 and not b.group.is_trivial:
                gathered = C.all_gather_raw(pshard.clone(), b.group, dim=0)
                b.params.copy_(gathered)
        return True, grad_norm, 0

    def count_zeros(self) -> int:
        z = torch.zeros((), dtype=torch.float32, device=self.buffers[0].device)
        for b in self.buffers:
            lo, hi = b.shard
            z += (b.grads[lo:hi] == 0).sum()
        return int(z)

    def _update_loss_scale(self, ok: bool):
        if not self.dynamic_scale:
            return
        tc = self.tc
        if not ok:
            self._growth_tracker = 0
            self._hysteresis -= 1
            if self._hysteresis <= 0:
                self.loss_scale = max(self.loss_scale / 2.0, tc.min_loss_scale)
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= tc.loss_scale_window:
                self._growth_tracker, self._hysteresis = 0, tc.hysteresis
                self.loss_scale *= 2.0

    def reload_model_params(self):
        for b in self.buffers:
            b.reload_master()

    # ---- checkpointing -------------------------------------------------
    def state_dict(self) -> dict:
        return {
            "step": self.step_count, "loss_scale": self.loss_scale, "zero1": self.zero1,
            "buffers": [{"expert": b.expert, "weight_decay": b.weight_decay, "shard": b.shard, "numel": b.numel,
                         "names": [s.name for s in b.slots],
                         "master": None if b.master is None else b.master.cpu(),
                         "exp_avg": b.exp_avg.cpu(), "exp_avg_sq": b.exp_avg_sq.cpu()} for b in self.buffers],
        }

    def load_state_dict(self, sd: dict):
        self.step_count = sd["step"]
        self.loss_scale = sd.get("loss_scale", self.loss_scale)
        assert len(sd["buffers"]) == len(self.buffers), "optimizer layout changed"
        for b, s in zip(self.buffers, sd["buffers"]):
            assert s["numel"] == b.numel and tuple(s["shard"]) == tuple(b.shard), \
                "optimizer shard layout differs (use ckpt.reshard_optimizer for a new DP size)"
            if b.master is not None and s["master"] is not None:
                b.master.copy_(s["master"])
            b.exp_avg.copy_(s["exp_avg"])
            b.exp_avg_sq.copy_(s["exp_avg_sq"])


class OptimizerParamScheduler:
    """Learning-rate and weight-decay schedules (Megatron ``OptimizerParamScheduler``, reached by the
    reference through training.py:30): linear warm-up then constant / linear / cosine /
    inverse-square-root decay; constant / linear / cosine weight-decay increment."""

    def __init__(self, tc: TrainConfig):
        self.tc = tc
        self.num_steps = 0
        self.decay_steps = tc.lr_decay_iters if tc.lr_decay_iters is not None else tc.train_iters
        self.warmup = tc.lr_warmup_iters
        self.start_wd = tc.start_weight_decay if tc.start_weight_decay is not None else tc.weight_decay
        self.end_wd = tc.end_weight_decay if tc.end_weight_decay is not None else tc.weight_decay

    def get_lr(self) -> float:
        tc, n = self.tc, self.num_steps
        if self.warmup > 0 and n <= self.warmup:
            return tc.lr_warmup_init + (tc.lr - tc.lr_warmup_init) * n / self.warmup
        if tc.lr_decay_style == "constant":
            return tc.lr
        if n > self.decay_steps:
            return tc.min_lr
        if tc.lr_decay_style == "inverse-square-root":
            w = max(self.warmup, 1)
            return max(tc.min_lr, tc.lr * math.sqrt(w) / math.sqrt(max(n, 1)))
        ratio = (n - self.warmup) / max(self.decay_steps - self.warmup, 1)
        delta = tc.lr - tc.min_lr
        if tc.lr_decay_style == "linear":
            coeff = 1.0 - ratio
        elif tc.lr_decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        else:
            raise ValueError(tc.lr_decay_style)
        return tc.min_lr + coeff * delta

    def get_wd(self) -> float:
        tc = self.tc
        if tc.weight_decay_incr_style == "constant" or self.start_wd == self.end_wd:
            return self.end_wd
        ratio = min(self.num_steps / max(self.decay_steps, 1), 1.0)
        if tc.weight_decay_incr_style == "linear":
            coeff = ratio
        elif tc.weight_decay_incr_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * (1 - ratio)) + 1.0)
        else:
            raise ValueError(tc.weight_decay_incr_style)
        return self.start_wd + coeff * (self.end_wd - self.start_wd)

    def step(self, increment: int = 1):
        self.num_steps += increment

    _SAVED = ("lr", "min_lr", "lr_decay_style", "lr_warmup_init", "weight_decay_incr_style")

    def state_dict(self):
        sd = {"num_steps": self.num_steps, "decay_steps": self.decay_steps, "warmup": self.warmup,
              "start_wd": self.start_wd, "end_wd": self.end_wd}
        sd.update({k: getattr(self.tc, k) for k in self._SAVED})
        return sd

    def load_state_dict(self, sd):
        """The step count always comes from the checkpoint.  The schedule's shape comes from the command line
        (``--override-opt_param-scheduler``, also the default here, with a note when the two differ) or from the checkpoint
        (``--use-checkpoint-opt_param-scheduler``)."""
        self.num_steps = sd["num_steps"]
        mine = self.state_dict()
        differ = sorted(k for k in sd if k != "num_steps" and k in mine and sd[k] != mine[k])
        if not differ:
            return
        if getattr(self.tc, "use_checkpoint_opt_param_scheduler", False):
            for k in ("decay_steps", "warmup", "start_wd", "end_wd"):
                if k in sd:
                    setattr(self, k, sd[k])
            for k in self._SAVED:
                if k in sd:
                    setattr(self.tc, k, sd[k])
        elif not getattr(self.tc, "override_opt_param_scheduler", False):
            print(f"> learning-rate schedule: the command line differs from the checkpoint in {differ}; using the command "
                  "line (--use-checkpoint-opt_param-scheduler keeps the checkpoint's)", flush=True)

"""Micro-batch schedules: no pipelining, 1F1B, and interleaved (virtual stages).

Counterpart of Megatron's ``get_forward_backward_func`` and ``p2p_communication`` which the
reference's train step calls (training.py:36,322-331; lm_evaluate.py:28-29).  Stage-to-stage
activations travel as point-to-point messages of the process-group backend (NCCL on GPUs, gloo
on CPU): pipeline traffic is the one path that stays on the library, by design.

``forward_step(batch, model, hidden_in) -> (output, loss_fn)``: on the last stage ``output`` is
what ``loss_fn`` consumes and ``loss_fn(output) -> (scalar loss, dict for logging)``; on other
stages ``output`` is the hidden state sent downstream.
"""
from __future__ import annotations

from typing import Callable, Iterator, List, Optional

import torch
import torch.distributed as dist

from ..dist.mesh import Mesh


_PENDING: list = []


def _send(t: torch.Tensor, dst: int, mesh: Mesh):
    """Asynchronous send; the request (and the tensor) is kept until ``_drain`` so that a stage never
    blocks on a receiver that is still busy with earlier micro-batches."""
    t = t.contiguous()
    _PENDING.append((dist.isend(t, dst=dst, group=mesh["pp"].pg), t))


def _drain():
    for req, _ in _PENDING:
        req.wait()
    _PENDING.clear()


def _recv(shape, dtype, device, src: int, mesh: Mesh) -> torch.Tensor:
    t = torch.empty(shape, dtype=dtype, device=device)
    dist.recv(t, src=src, group=mesh["pp"].pg)
    return t


def forward_backward_no_pipelining(forward_step: Callable, data_iter: Iterator, model, num_microbatches: int,
                                   optimizer=None, forward_only: bool = False) -> List[dict]:
    logs = []
    for i in range(num_microbatches):
        batch = next(data_iter)
        out, loss_fn = forward_step(batch, model, None)
        loss, log = loss_fn(out)
        if not forward_only:
            loss = loss / num_microbatches
            if optimizer is not None and hasattr(optimizer, "overlap_active"):
                optimizer.overlap_active = i == num_microbatches - 1      # gradients are final after this backward
            (optimizer.scale_loss(loss) if optimizer is not None else loss).backward()
            if optimizer is not None and hasattr(optimizer, "overlap_active"):
                optimizer.overlap_active = False
        logs.append(log)
    return logs


def forward_backward_1f1b(forward_step: Callable, data_iter: Iterator, model, num_microbatches: int, mesh: Mesh,
                          hidden_shape, dtype, optimizer=None, forward_only: bool = False) -> List[dict]:
    """One-forward-one-backward pipeline schedule.  Stage p runs ``pp-1-p`` warm-up forwards, then
    alternates forward/backward, then drains the remaining backwards."""
    pp, r = mesh.pp, mesh.pp_rank
    first, last = mesh.is_first_stage, mesh.is_last_stage
    prev_rank, next_rank = mesh.prev_stage_rank, mesh.next_stage_rank
    device = next(model.parameters()).device
    n_warm = min(pp - r - 1, num_microbatches)
    n_steady = num_microbatches - n_warm
    inputs, outputs, logs = [], [], []

    def fwd():
        batch = next(data_iter)
        hin = None
        if not first:
            hin = _recv(hidden_shape, dtype, device, prev_rank, mesh)
            hin.requires_grad_(not forward_only)
        out, loss_fn = forward_step(batch, model, hin)
        if last:
            loss, log = loss_fn(out)
            logs.append(log)
            out = loss / num_microbatches
            if optimizer is not None and not forward_only:
                out = optimizer.scale_loss(out)
        else:
            _send(out.detach(), next_rank, mesh)
        if not forward_only:
            inputs.append(hin)
            outputs.append(out)

    def bwd():
        hin, out = inputs.pop(0), outputs.pop(0)
        if last:
            out.backward()
        else:
            g = _recv(out.shape, out.dtype, device, next_rank, mesh)
            torch.autograd.backward(out, grad_tensors=g)
        if not first:
            _send(hin.grad, prev_rank, mesh)

    for _ in range(n_warm):
        fwd()
    for i in range(n_steady):
        fwd()
        if not forward_only:
            bwd()
    if not forward_only:
        for _ in range(n_warm):
            bwd()
    _drain()
    return logs


def forward_backward_interleaved(forward_step: Callable, data_iters: List[Iterator], models: List, num_microbatches: int,
                                 mesh: Mesh, hidden_shape, dtype, optimizer=None, forward_only: bool = False) -> List[dict]:
    """Virtual-pipeline schedule over ``len(models)`` model chunks per stage.  Chunk ``c`` of stage ``p``
    is virtual stage ``c*pp + p``.  All micro-batches flow forward through the virtual stages in order
    and backward in reverse order (breadth-first); activations of a chunk live until its backward."""
    pp, r = mesh.pp, mesh.pp_rank
    V = len(models)
    device = next(models[0].parameters()).device
    prev_rank, next_rank = mesh.prev_stage_rank, mesh.next_stage_rank
    saved = [[None] * num_microbatches for _ in range(V)]
    logs: List[dict] = []
    for c in range(V):
        vs = c * pp + r
        is_first, is_last = vs == 0, vs == V * pp - 1
        for m in range(num_microbatches):
            batch = next(data_iters[c])
            hin = None
            if not is_first:
                hin = _recv(hidden_shape, dtype, device, prev_rank, mesh)
                hin.requires_grad_(not forward_only)
            out, loss_fn = forward_step(batch, models[c], hin)
            if is_last:
                loss, log = loss_fn(out)
                logs.append(log)
                out = loss / num_microbatches
                if optimizer is not None and not forward_only:
                    out = optimizer.scale_loss(out)
            else:
                _send(out.detach(), next_rank, mesh)
            saved[c][m] = (hin, out)
    if forward_only:
        _drain()
        return logs
    for c in reversed(range(V)):
        vs = c * pp + r
        is_first, is_last = vs == 0, vs == V * pp - 1
        for m in range(num_microbatches):
            hin, out = saved[c][m]
            if is_last:
                out.backward()
            else:
                g = _recv(out.shape, out.dtype, device, next_rank, mesh)
                torch.autograd.backward(out, grad_tensors=g)
            if not is_first:
                _send(hin.grad, prev_rank, mesh)
            saved[c][m] = None
    _drain()
    return logs


def get_forward_backward_func(mesh: Mesh):
    if mesh.pp == 1:
        return forward_backward_no_pipelining
    if mesh.par.virtual_pipeline_model_parallel_size:
        return forward_backward_interleaved
    return forward_backward_1f1b

"""Forward passes of a model that is split over pipeline stages and tensor-parallel ranks, for generation and evaluation.

The reference's inference loop relays the activations stage to stage and then broadcasts the sampled tokens and the
"done" flag from the last pipeline stage to the first (generation/generation.py:120-351, communication helpers
``broadcast_from_last_pipeline_stage`` / ``broadcast_from_last_to_first_pipeline_stage``); its evaluation adaptor does the
same recv / forward / send per request and gathers the vocabulary-parallel logits over the tensor-parallel group
(lm_evaluate.py:93-116).  Here:

* tensor parallelism needs nothing extra: ``LMHead`` gathers the logits over the TP group unless ``parallel_output``;
* pipeline parallelism: :func:`stage_forward` receives the hidden states from the previous stage, runs this stage (with
  its own decoding caches) and sends them on; the last stage returns logits, the others ``None``;
* :func:`broadcast_from_last_stage` hands a tensor computed on the last stage (sampled tokens, log-probabilities, a
  slice of logits) to every stage, so that all stages keep identical token buffers and termination flags.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _mesh(model):
    return getattr(getattr(model, "module", model), "mesh")


def is_last_stage(model) -> bool:
    m = _mesh(model)
    return m.pp == 1 or m.is_last_stage


def stage_forward(model, tokens: torch.Tensor, caches: Optional[List[dict]] = None, position_offset: int = 0):
    """Run ``tokens [B, t]`` through this rank's stage.  Returns logits ``[B, t, V]`` on the last stage, else ``None``."""
    mesh = _mesh(model)
    if mesh.pp == 1:
        return model(tokens, caches=caches, position_offset=position_offset)
    from ..train.schedules import _drain, _recv, _send
    inner = getattr(model, "module", model)
    hidden = None
    if not mesh.is_first_stage:
        hidden = _recv((tokens.shape[0], tokens.shape[1], inner.cfg.hidden_size), inner.cfg.params_dtype, tokens.device,
                       mesh.prev_stage_rank, mesh)
    out = model(tokens, hidden_in=hidden, caches=caches, position_offset=position_offset)
    if mesh.is_last_stage:
        return out
    _send(out, mesh.next_stage_rank, mesh)
    _drain()
    return None


def broadcast_from_last_stage(model, t: Optional[torch.Tensor], shape, dtype, device) -> torch.Tensor:
    """The tensor ``t`` of the last pipeline stage on every stage (a no-op without pipeline parallelism)."""
    mesh = _mesh(model)
    if mesh.pp == 1:
        return t
    g = mesh["pp"]
    buf = t.to(dtype).contiguous() if mesh.is_last_stage else torch.empty(shape, dtype=dtype, device=device)
    dist.broadcast(buf, src=g.ranks[-1], group=g.pg)
    return buf


def full_logits(model, tokens: torch.Tensor, last_only: bool = False) -> torch.Tensor:
    """Logits of ``tokens`` on EVERY rank (all positions, or the last one with ``last_only``)."""
    inner = getattr(model, "module", model)
    logits = stage_forward(model, tokens)
    if logits is not None and last_only:
        logits = logits[:, -1:]
    B, T = tokens.shape
    shape = (B, 1 if last_only else T, inner.cfg.vocab_size)
    return broadcast_from_last_stage(model, None if logits is None else logits.float(), shape, torch.float32, tokens.device)

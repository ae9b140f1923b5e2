"""Epoch-based supervised fine-tuning.

Reference: linear_moe/finetune_utils.py:82-105 (DistributedSampler loader), :159-265 (``_train``: epochs over the
train loader, periodic eval / save, ``--keep-last`` drops the ragged last batch), :268-350 (``finetune``: build
datasets, load ``--pretrained-checkpoint``, ``optimizer.reload_model_params()``, train).  Built on ``Trainer``:
the data iterator is swapped for an epoch iterator over the SFT dataset (labels masked on the prompt).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..config.model_config import ModelConfig, ParallelConfig, TrainConfig
from ..data.datasets import make_batch, slice_for_context_parallel
from ..dist.mesh import Mesh
from .loop import Trainer, print_rank_0


class EpochIterator:
    """Deals the samples of one epoch to the data-parallel ranks (a DistributedSampler with optional shuffle) and
    raises ``StopIteration`` at the end of the epoch."""

    def __init__(self, dataset, micro_batch_size: int, mesh: Mesh, device, epoch: int, shuffle: bool = True,
                 seed: int = 1234, keep_last: bool = False, pad_token: Optional[int] = None):
        self.ds, self.mbs, self.mesh, self.device = dataset, micro_batch_size, mesh, device
        n = len(dataset)
        g = torch.Generator().manual_seed(seed + epoch)
        order = torch.randperm(n, generator=g).tolist() if shuffle else list(range(n))
        per_step = micro_batch_size * mesh.dp
        usable = n if keep_last else n // per_step * per_step
        order = order[:usable]
        if keep_last and len(order) % per_step:
            order += order[: per_step - len(order) % per_step]          # wrap to fill the last batch
        self.order = order[mesh.dp_rank * micro_batch_size:]
        self.stride, self.pos, self.pad = per_step, 0, pad_token
        self.consumed = 0

    def __iter__(self):
        return self

    def __len__(self):
        return (len(self.order) + self.stride - 1) // self.stride

    def __next__(self):
        if self.pos + self.mbs > len(self.order):
            raise StopIteration
        idx = self.order[self.pos:self.pos + self.mbs]
        self.pos += self.stride
        rows = [self.ds[i] for i in idx]
        sample = {k: torch.stack([r[k] for r in rows]) for k in rows[0]}
        batch = slice_for_context_parallel(make_batch(sample, pad_token=self.pad), self.mesh)
        return {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}


def finetune(cfg: ModelConfig, par: ParallelConfig, tc: TrainConfig, train_dataset, valid_dataset=None,
             mesh: Optional[Mesh] = None, device=None, end_of_epoch_callback: Optional[Callable] = None,
             pad_token: Optional[int] = None) -> Trainer:
    """Run ``tc.epochs`` epochs.  ``tc.pretrained_checkpoint`` (weights only) is loaded by the Trainer, which then
    refreshes the fp32 masters from the loaded weights."""
    trainer = Trainer(cfg, par, tc, mesh, device, dataset=train_dataset, valid_dataset=valid_dataset)
    epochs = tc.epochs or 1
    for epoch in range(epochs):
        it = EpochIterator(train_dataset, tc.micro_batch_size, trainer.mesh, trainer.device, epoch, seed=tc.seed,
                           keep_last=tc.keep_last, pad_token=pad_token)
        steps = len(it) // trainer.num_microbatches
        print_rank_0(f"working on epoch {epoch + 1}/{epochs}: {steps} iterations")
        trainer.data_iter = it
        for _ in range(steps):
            stats = trainer.train_step()
            if trainer.iteration % tc.log_interval == 0:
                print_rank_0(f" epoch {epoch + 1} iteration {trainer.iteration} | lm loss {float(stats.get('lm loss', 0)):.6E} | "
                             f"lr {stats['lr']:.3E}")
            if tc.save and tc.save_interval and trainer.iteration % tc.save_interval == 0:
                trainer.save()
        if valid_dataset is not None:
            ev = trainer.evaluate()
            print_rank_0(f" validation after epoch {epoch + 1} | lm loss {ev['lm loss']:.6E} | ppl {ev['ppl']:.6E}")
        if end_of_epoch_callback is not None:
            end_of_epoch_callback(trainer, epoch)
    if tc.save:
        trainer.save()
    return trainer

"""Training entry points: ``Trainer`` and ``pretrain``.

Contract of the reference's loop (linear_moe/training.py:51-180 ``pretrain``, :184-305 ``get_model``,
:307-379 ``train_step``, :382-554 ``training_log``, :566-698 ``train``, :701-820 ``evaluate``; the
entry scripts examples/*/pretrain_*.py provide ``model_provider``/``forward_step``/``loss_func``):

  zero grads -> forward/backward over the micro-batches (pipeline schedule) -> reduce grads ->
  optimizer step (unscale, clip, Adam, param gather) -> LR scheduler step -> log / eval / save / exit.

Extras kept from the reference: SIGTERM save-and-exit (``--exit-signal-handler``), ``--exit-interval``,
``--exit-duration-in-mins`` (max-reduced flag), NaN check, skipped-iteration accounting, a profiler
window (``--profile*``: NVTX ranges + cudaProfilerStart/Stop), TensorBoard scalars.  Added: tokens/s,
model-FLOPs utilisation, a host heartbeat watchdog.
"""
from __future__ import annotations

import math
import os
import signal
import sys
import time
from typing import Callable, Dict, Iterator, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config.model_config import ModelConfig, ParallelConfig, TrainConfig
from ..data.datasets import BatchIterator, SyntheticTokenDataset
from ..dist import collectives as C
from ..dist.mesh import Mesh, init_distributed, single_process_mesh
from ..models.moe import AuxLossTracker, MoEAuxLossAutoScaler
from ..models.transformer import CausalLM
from ..parallel.tensor_parallel import set_init_seed
from ..utils.memory import compute_weight_and_optimizer_memory, count_parameters, model_flops_per_token
from .optimizer import MixedPrecisionAdam, OptimizerParamScheduler
from .schedules import get_forward_backward_func, forward_backward_no_pipelining
from .timers import Timers
from .watchdog import Heartbeat


def print_rank_0(*a, **kw):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*a, **kw, flush=True)


def build_model(cfg: ModelConfig, mesh: Mesh, device, sequence_parallel: bool = False) -> List[CausalLM]:
    """One model chunk per virtual pipeline stage of this rank (training.py:184-305 ``get_model``)."""
    vpp = mesh.par.virtual_pipeline_model_parallel_size or 1
    from ..ops import fp8
    fp8.set_enabled(bool(cfg.fp8) and torch.device(device).type == "cuda")
    chunks = []
    for v in range(vpp):
        vs = v * mesh.pp + mesh.pp_rank
        m = CausalLM(cfg, mesh, pre_process=vs == 0, post_process=vs == vpp * mesh.pp - 1, vpp_rank=v,
                     sequence_parallel=sequence_parallel, device=device)
        chunks.append(m.to(device))
    return chunks


def masked_lm_loss(per_token: torch.Tensor, loss_mask: torch.Tensor, mesh: Mesh):
    """Masked mean over the whole (context-parallel) sequence.  Returns ``(loss for backward, loss for
    logging)``: the former is multiplied by the CP size because gradients are later averaged over dp*cp
    (pretrain_qwen.py:183-233)."""
    cp = mesh["cp"]
    s = (per_token.float() * loss_mask).sum()
    n = loss_mask.sum()
    if not cp.is_trivial:
        n = C.all_reduce_(n.clone(), cp)
        s_all = C.all_reduce(s, cp)
        loss = s_all / n.clamp(min=1.0)
        return loss * cp.size, loss.detach()
    loss = s / n.clamp(min=1.0)
    return loss, loss.detach()


class Trainer:
    def __init__(self, cfg: ModelConfig, par: ParallelConfig, tc: TrainConfig, mesh: Optional[Mesh] = None,
                 device: Optional[torch.device] = None, dataset=None, valid_dataset=None,
                 model_provider: Optional[Callable] = None, forward_step: Optional[Callable] = None):
        self.cfg, self.par, self.tc = cfg, par, tc
        self.mesh = mesh or single_process_mesh()
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        set_init_seed(tc.seed)
        if par.fused_comm and self.device.type == "cuda" and self.mesh.world_size > 1:
            from ..parallel import fused_comm
            fused_comm.set_timeout(par.fused_comm_timeout_s)
            fused_comm.init_workspaces(self.mesh, cfg, tc)
        torch.manual_seed(tc.seed + 100 * self.mesh.pp_rank + 10 * self.mesh.dp_rank + self.mesh.cp_rank)
        sp = par.sequence_parallel and par.tp > 1
        self.models = model_provider(cfg, self.mesh, self.device) if model_provider else \
            build_model(cfg, self.mesh, self.device, sp)
        self.model = self.models[0]
        wrapper = nn.ModuleList(self.models)
        self.optimizer = MixedPrecisionAdam(wrapper, self.mesh, tc, zero1=par.use_distributed_optimizer,
                                            sequence_parallel=sp, fused_comm=par.fused_comm,
                                            overlap_grad_reduce=par.overlap_grad_reduce)
        if par.overlap_grad_reduce and self.mesh.pp == 1 and len(self.models) == 1 and \
                any(b.fused is not None for b in self.optimizer.buffers):
            # a block's gradients are reduced while the backward pass of the blocks before it is still running
            getattr(self.model, "module", self.model).grad_ready_hook = self.optimizer.bucket_ready
        if par.overlap_param_gather and self.mesh.rank == 0:
            print("note: --overlap-param-gather has nothing to move: with the distributed optimizer the updated parameters are "
                  "broadcast by the fused Adam kernel itself (multimem stores), without it there is no parameter gather",
                  flush=True)
        self.scheduler = OptimizerParamScheduler(tc)
        self.timers = Timers(tc.timing_log_level, cuda=self.device.type == "cuda")
        self.iteration, self.consumed_samples = 0, 0
        self.custom_forward_step = forward_step
        dp = self.mesh.dp
        assert tc.global_batch_size % (tc.micro_batch_size * dp) == 0, \
            f"global batch {tc.global_batch_size} not divisible by micro batch {tc.micro_batch_size} x dp {dp}"
        self.num_microbatches = tc.global_batch_size // (tc.micro_batch_size * dp)
        self.global_batch_now = tc.global_batch_size
        if tc.rampup_batch_size:
            start, incr, _ = tc.rampup_batch_size
            unit = tc.micro_batch_size * dp
            assert start % unit == 0 and incr % unit == 0 and (tc.global_batch_size - start) % incr == 0 and incr > 0, \
                f"--rampup-batch-size {tc.rampup_batch_size}: start and increment must be multiples of micro batch x dp = " \
                f"{unit} and the increments must reach the global batch {tc.global_batch_size}"
        if dataset is None:
            dataset = SyntheticTokenDataset(cfg.vocab_size, tc.seq_length, seed=tc.seed)
        self.dataset, self.valid_dataset = dataset, valid_dataset
        self.data_iter = BatchIterator(dataset, tc.micro_batch_size, self.mesh, self.device, eod_token=tc.eod_token,
                                       eod_mask_loss=tc.eod_mask_loss, prefetch=tc.num_workers)
        self.writer = None
        if tc.tensorboard_dir and self.mesh.rank == self.mesh.world_size - 1:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.writer = SummaryWriter(tc.tensorboard_dir, max_queue=tc.tensorboard_queue_size)
            except Exception as e:                      # tensorboard is optional
                print_rank_0(f"tensorboard disabled: {e}")
        self._exit_signal = False
        if tc.exit_signal_handler:
            signal.signal(signal.SIGTERM, self._on_sigterm)
        self._t0 = time.time()
        self._log_acc: Dict[str, float] = {}
        self._log_n = 0
        self._nan_iters = 0
        self.heartbeat = Heartbeat(self.mesh, tc.heartbeat_interval_s, tc.heartbeat_timeout_s) \
            if tc.heartbeat_interval_s > 0 else None
        self.flops_per_token = model_flops_per_token(cfg, tc.seq_length)
        if tc.load and not self._has_checkpoint(tc.load):
            if tc.exit_on_missing_checkpoint:
                raise SystemExit(f"--exit-on-missing-checkpoint: no checkpoint under {tc.load}")
            print_rank_0(f"> no checkpoint under {tc.load}: starting from the initial weights")
        elif tc.load:
            self.load(tc.load, model_only=tc.finetune)
        elif tc.pretrained_checkpoint:
            self.load(tc.pretrained_checkpoint, model_only=True)
            self.optimizer.reload_model_params()

    # ------------------------------------------------------------------
    def _on_sigterm(self, *_):
        self._exit_signal = True

    def forward_step(self, batch, model: CausalLM, hidden_in):
        if self.custom_forward_step is not None:
            return self.custom_forward_step(batch, model, hidden_in)
        out = model(batch["tokens"], batch["labels"] if model.post_process else None, hidden_in=hidden_in)
        mesh = self.mesh

        def loss_fn(per_token):
            loss, log_loss = masked_lm_loss(per_token, batch["loss_mask"], mesh)
            if self.tc.check_for_nan_in_loss_and_grad and not torch.isfinite(log_loss):
                raise FloatingPointError(f"rank {mesh.rank}: non-finite loss at iteration {self.iteration}")
            return loss, {"lm loss": log_loss}
        return out, loss_fn

    def _run_schedule(self, forward_only: bool = False, data_iter=None):
        tc, mesh = self.tc, self.mesh
        data_iter = data_iter or self.data_iter
        fb = get_forward_backward_func(mesh)
        opt = None if forward_only else self.optimizer
        if mesh.pp == 1:
            return fb(self.forward_step, data_iter, self.model, self.num_microbatches, opt, forward_only)
        T = tc.seq_length // mesh.cp // (mesh.tp if (self.par.sequence_parallel and mesh.tp > 1) else 1)
        shape = (tc.micro_batch_size, T, self.cfg.hidden_size)
        if mesh.par.virtual_pipeline_model_parallel_size:
            iters = [data_iter] + [BatchIterator(self.dataset, tc.micro_batch_size, mesh, self.device,
                                                 consumed_samples=data_iter.consumed) for _ in self.models[1:]]
            logs = fb(self.forward_step, iters, self.models, self.num_microbatches, mesh, shape,
                      self.cfg.params_dtype, opt, forward_only)
            data_iter.consumed = iters[-1].consumed if len(iters) > 1 else data_iter.consumed
            return logs
        return fb(self.forward_step, data_iter, self.model, self.num_microbatches, mesh, shape,
                  self.cfg.params_dtype, opt, forward_only)

    def _check_kernels(self, where: str = ""):
        """Raise if a fused-communication kernel or a tcgen05 GEMM gave up on a bounded wait since the last check.
        Called every step between the gradient-norm read (which has synchronised the device) and the parameter
        update, and before a checkpoint is written, so a timed-out step never reaches the weights or the disk."""
        if self.device.type == "cuda":
            from ..parallel import fused_comm
            fused_comm.check_status(where or f"iteration {self.iteration + 1}")

    def _manual_gc(self):
        """``--manual-gc``: the cyclic collector is switched off and run by hand at the same step on every rank, so that a
        collection pause on one rank does not show up as waiting time in the other ranks' collectives."""
        import gc
        tc = self.tc
        if not tc.manual_gc:
            return
        if not getattr(self, "_gc_off", False):
            gc.collect()
            gc.disable()
            self._gc_off = True
        elif tc.manual_gc_interval and self.iteration % tc.manual_gc_interval == 0:
            gc.collect()

    def _ramped_global_batch(self, consumed: int) -> int:
        """``--rampup-batch-size start increment samples``: the global batch grows from ``start`` to the configured size
        in equal increments spread over the first ``samples`` samples (Megatron's ramp-up micro-batch calculator)."""
        tc = self.tc
        if not tc.rampup_batch_size:
            return tc.global_batch_size
        start, incr, ramp = tc.rampup_batch_size
        steps = (tc.global_batch_size - start) // incr
        if steps <= 0 or consumed >= ramp:
            return tc.global_batch_size
        return min(start + int(consumed / (ramp / steps)) * incr, tc.global_batch_size)

    def train_step(self) -> Dict[str, float]:
        tc, mesh = self.tc, self.mesh
        timers = self.timers
        self._manual_gc()
        self.global_batch_now = self._ramped_global_batch(self.consumed_samples)
        self.num_microbatches = self.global_batch_now // (tc.micro_batch_size * mesh.dp)
        for m in self.models:
            m.train()
        self.optimizer.zero_grad()
        MoEAuxLossAutoScaler.set_loss_scale((self.optimizer.loss_scale or 1.0) / self.num_microbatches)
        timers("forward-backward").start(barrier=tc.barrier_with_L1_time and tc.timing_log_level > 0)
        logs = self._run_schedule()
        timers("forward-backward").stop()
        for m in self.models:
            inner = getattr(m, "module", m)
            if getattr(inner, "offload", None) is not None:
                inner.offload.step_done()
        if tc.empty_unused_memory_level >= 2 and self.device.type == "cuda":
            torch.cuda.empty_cache()
        timers("all-grads-sync", 1).start()
        self.optimizer.reduce_grads()
        if self.device.type == "cuda":
            from ..parallel import fused_comm
            fused_comm.mark_step_sync()              # the reduction waits for every rank: all LASP slots are free again
        timers("all-grads-sync", 1).stop()
        timers("optimizer").start()
        lr, wd = self.scheduler.get_lr(), self.scheduler.get_wd()
        ok, grad_norm, _ = self.optimizer.step(lr, wd, pre_update=self._check_kernels)
        timers("optimizer").stop()
        if tc.empty_unused_memory_level >= 1 and self.device.type == "cuda":
            torch.cuda.empty_cache()
        if ok:
            self.scheduler.step(1)
        if self.cfg.test_mode:
            # --test-mode (attention.py:400-467, run every step there): replicated q / k norm weights must still agree
            # across the data- and tensor-parallel ranks
            for m in self.models:
                for mod in m.modules():
                    check = getattr(mod, "run_realtime_tests", None)
                    if check is not None and not check():
                        raise RuntimeError(f"--test-mode: replicated weights of {type(mod).__name__} differ between ranks "
                                           f"at iteration {self.iteration + 1}")
        self.iteration += 1
        self.consumed_samples += self.global_batch_now
        out = {"lr": lr, "grad_norm": grad_norm, "skipped": 0 if ok else 1}
        if mesh.is_last_stage and logs:
            keys = logs[0].keys()
            for k in keys:
                v = torch.stack([l[k].float() for l in logs]).mean()
                C.all_reduce_(v, mesh["dp"])
                out[k] = v / mesh.dp
        return out

    # ------------------------------------------------------------------
    def training_log(self, stats: Dict[str, float], elapsed_s: float):
        tc, mesh = self.tc, self.mesh
        for k, v in stats.items():
            if k in ("lr", "grad_norm", "skipped") or v is None:
                continue
            self._log_acc[k] = self._log_acc.get(k, 0.0) + float(v)
        self._log_n += 1
        self._log_acc["skipped"] = self._log_acc.get("skipped", 0.0) + stats.get("skipped", 0)
        if (self.writer is not None and tc.tensorboard_log_interval and self.iteration % tc.tensorboard_log_interval == 0
                and self.iteration % tc.log_interval != 0):
            # --tensorboard-log-interval: this step's values between two console lines (the console line writes averages)
            self.writer.add_scalar("learning-rate", stats["lr"], self.iteration)
            for k, v in stats.items():
                if k not in ("lr", "skipped") and v is not None:
                    self.writer.add_scalar("grad-norm" if k == "grad_norm" else k, float(v), self.iteration)
        if self.iteration % tc.log_interval != 0:
            return
        per_iter = elapsed_s / max(self._log_n, 1)
        tokens = self.global_batch_now * tc.seq_length
        tps = tokens / per_iter
        gpus = mesh.world_size
        mfu = None
        if self.device.type == "cuda":
            mfu = self.flops_per_token * tps / gpus / 2.25e15
        line = (f" iteration {self.iteration:8d}/{tc.train_iters:8d} | consumed samples: {self.consumed_samples:12d} |"
                f" elapsed time per iteration (ms): {per_iter * 1000:.1f} | tokens/s: {tps:.0f} |"
                f" tokens/s/gpu: {tps / gpus:.0f} | learning rate: {stats['lr']:.3E} |"
                f" global batch size: {self.global_batch_now:5d} |")
        for k, v in self._log_acc.items():
            if k != "skipped":
                line += f" {k}: {v / max(self._log_n, 1):.6E} |"
        if self.optimizer.loss_scale is not None:
            line += f" loss scale: {self.optimizer.loss_scale:.1f} |"
        if stats.get("grad_norm") is not None:
            line += f" grad norm: {stats['grad_norm']:.3f} |"
        if mfu is not None:
            line += f" MFU(bf16 dense peak): {mfu * 100:.1f}% |"
        line += f" number of skipped iterations: {int(self._log_acc.get('skipped', 0)):3d} |"
        line += f" number of nan iterations: {self._nan_iters:3d} |"
        aux = AuxLossTracker.pop()
        for k, v in aux.items():
            line += f" {k}: {float(v.sum()) / max(self.cfg.num_layers, 1) / max(self._log_n, 1):.4E} |"
            if tc.moe_per_layer_logging:
                per = (v / max(self._log_n, 1)).tolist()
                line += "".join(f" moe/{k}_layer_{i}: {x:.4E} |" for i, x in enumerate(per) if x != 0.0)
                if self.writer is not None:
                    for i, x in enumerate(per):
                        if x != 0.0:
                            self.writer.add_scalar(f"moe/{k}_layer_{i}", x, self.iteration)
        if mesh.rank == mesh.world_size - 1 or mesh.world_size == 1:
            print(line, flush=True)
        if tc.timing_log_level >= 0:
            tv = self.timers.collect()
            if tv:
                n = max(self._log_n, 1)
                print_rank_0("    timers (ms/iter): " + " | ".join(f"{k}: {v * 1000.0 / n:.2f}" for k, v in tv.items()))
                if tc.log_timers_to_tensorboard and self.writer is not None:
                    for k, v in tv.items():
                        self.writer.add_scalar(k + "-time", v / n, self.iteration)
        if self.writer is not None:
            it = self.iteration
            self.writer.add_scalar("learning-rate", stats["lr"], it)
            self.writer.add_scalar("batch-size", self.global_batch_now, it)
            self.writer.add_scalar("tokens-per-second", tps, it)
            for k, v in self._log_acc.items():
                self.writer.add_scalar(k, v / max(self._log_n, 1), it)
                self.writer.add_scalar(k + " vs samples", v / max(self._log_n, 1), self.consumed_samples)
            if stats.get("grad_norm") is not None:
                self.writer.add_scalar("grad-norm", stats["grad_norm"], it)
            if tc.log_memory_to_tensorboard and self.device.type == "cuda":
                self.writer.add_scalar("mem-allocated-bytes", torch.cuda.memory_allocated(), it)
                self.writer.add_scalar("mem-reserved-bytes", torch.cuda.memory_reserved(), it)
        if self.iteration == tc.log_interval and self.device.type == "cuda":
            print_rank_0(f"    memory (MB) | allocated: {torch.cuda.memory_allocated() / 2**20:.0f} | "
                         f"max allocated: {torch.cuda.max_memory_allocated() / 2**20:.0f} | "
                         f"reserved: {torch.cuda.memory_reserved() / 2**20:.0f}")
        self._log_acc, self._log_n = {}, 0

    @torch.no_grad()
    def evaluate(self, iters: Optional[int] = None) -> Dict[str, float]:
        tc = self.tc
        for m in self.models:
            m.eval()
        ds = self.valid_dataset or self.dataset
        it = BatchIterator(ds, tc.micro_batch_size, self.mesh, self.device, consumed_samples=1 << 20)
        total, n = 0.0, 0
        for _ in range(iters or tc.eval_iters):
            logs = self._run_schedule(forward_only=True, data_iter=it)
            for l in logs:
                total += float(l["lm loss"])
                n += 1
        t = torch.tensor([total, n], dtype=torch.float64, device=self.device)
        C.all_reduce_(t, self.mesh["world"])
        loss = (t[0] / t[1].clamp(min=1)).item()
        self._check_kernels("evaluation")
        for m in self.models:
            m.train()
        return {"lm loss": loss, "ppl": math.exp(min(20.0, loss))}

    # ------------------------------------------------------------------
    def save(self, path: Optional[str] = None):
        from ..ckpt.legacy import save_checkpoint
        path = path or self.tc.save
        if path:
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self._check_kernels("before checkpoint save")
            if self.tc.use_dist_ckpt:
                from ..ckpt.sharded import save_sharded
                save_sharded(path, self.iteration, self.models, self.cfg, self.mesh,
                             None if self.tc.no_save_optim else self.optimizer, layer_offsets=self._layer_offsets(),
                             extra={"consumed_samples": self.consumed_samples,
                                    "opt_param_scheduler": self.scheduler.state_dict(),
                                    "model_args": {k: (v if not isinstance(v, torch.dtype) else str(v))
                                                   for k, v in vars(self.cfg).items()}})
                return
            save_checkpoint(path, self.iteration, self.models, self.optimizer, self.scheduler, self.cfg, self.par,
                            self.tc, self.mesh, consumed_samples=self.consumed_samples)

    def _layer_offsets(self):
        """Global index of the first layer of every model chunk of this pipeline stage."""
        per = self.cfg.num_layers // (self.mesh.pp * len(self.models))
        return [(i * self.mesh.pp + self.mesh.pp_rank) * per for i in range(len(self.models))]

    @staticmethod
    def _has_checkpoint(path: str) -> bool:
        from ..ckpt import sharded
        return any(os.path.isfile(os.path.join(path, f)) for f in (sharded.TRACKER, "latest_checkpointed_iteration.txt"))

    def load(self, path: str, model_only: bool = False):
        from ..ckpt import sharded
        from ..ckpt.legacy import load_checkpoint
        has_sharded = os.path.isfile(os.path.join(path, sharded.TRACKER))
        if (self.tc.use_dist_ckpt or (self.tc.auto_detect_ckpt_format and has_sharded)) and has_sharded:
            opt = None if (model_only or self.tc.no_load_optim) else self.optimizer
            if opt is not None:
                opt.state_loaded = False
            it, extra = sharded.load_sharded(path, self.models, self.cfg, self.mesh, opt, layer_offsets=self._layer_offsets(),
                                             return_extra=True)
            if not model_only:
                self.iteration = it
                self.consumed_samples = int(extra.get("consumed_samples", 0))
                self.data_iter.consumed = self.consumed_samples
                if "opt_param_scheduler" in extra:
                    self.scheduler.load_state_dict(extra["opt_param_scheduler"])
            if not getattr(self.optimizer, "state_loaded", False):
                self.optimizer.reload_model_params()
            return
        it, consumed = load_checkpoint(path, self.models, None if (model_only or self.tc.no_load_optim) else self.optimizer,
                                       None if model_only else self.scheduler, self.mesh,
                                       load_rng=not (model_only or self.tc.no_load_rng))
        if not model_only:
            self.iteration, self.consumed_samples = it, consumed
            self.data_iter.consumed = consumed
        if not getattr(self.optimizer, "state_loaded", False):
            # weights only (pretrained / --no-load-optim / no optimizer file): derive the fp32 masters from them.
            # After a full resume the restored masters are kept bit for bit (finetune_utils.py:319-327 reloads only
            # on the pretrained-checkpoint path).
            self.optimizer.reload_model_params()

    # ------------------------------------------------------------------
    def _should_exit(self) -> Optional[str]:
        tc = self.tc
        if tc.exit_signal_handler:
            flag = torch.tensor([1 if self._exit_signal else 0], device=self.device)
            C.all_reduce_(flag, self.mesh["world"], op=dist.ReduceOp.MAX)
            if int(flag) > 0:
                return "signal"
        if tc.exit_duration_in_mins:
            mins = (time.time() - self._t0) / 60.0
            flag = torch.tensor([1 if mins > tc.exit_duration_in_mins else 0], device=self.device)
            C.all_reduce_(flag, self.mesh["world"], op=dist.ReduceOp.MAX)
            if int(flag) > 0:
                return "duration"
        if tc.exit_interval and self.iteration % tc.exit_interval == 0:
            return "interval"
        if tc.adlr_autoresume and self.iteration % max(tc.adlr_autoresume_interval, 1) == 0:
            from .watchdog import autoresume_termination_requested
            flag = torch.tensor([1 if (self.mesh.rank == 0 and autoresume_termination_requested()) else 0],
                                device=self.device)
            C.all_reduce_(flag, self.mesh["world"], op=dist.ReduceOp.MAX)
            if int(flag) > 0:
                return "autoresume"
        return None

    def train(self) -> Dict[str, float]:
        tc = self.tc
        last = {}
        t_prev = time.perf_counter()
        prof_on = False
        while self.iteration < tc.train_iters:
            if tc.profile and self.mesh.rank in tc.profile_ranks and self.device.type == "cuda":
                if self.iteration == tc.profile_step_start:
                    torch.cuda.cudart().cudaProfilerStart()
                    prof_on = True
                if self.iteration == tc.profile_step_end and prof_on:
                    torch.cuda.cudart().cudaProfilerStop()
                    prof_on = False
            if prof_on:
                torch.cuda.nvtx.range_push(f"iteration {self.iteration}")
            try:
                stats = self.train_step()
            except FloatingPointError:
                self._nan_iters += 1
                raise
            if prof_on:
                torch.cuda.nvtx.range_pop()
            if self.heartbeat is not None:
                self.heartbeat.beat(self.iteration)
            if self.iteration % tc.log_interval == 0:
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                now = time.perf_counter()
                self.training_log(stats, now - t_prev)
                t_prev = now
            else:
                self.training_log(stats, 0.0)
            last = stats
            if tc.eval_interval and self.iteration % tc.eval_interval == 0:
                ev = self.evaluate()
                print_rank_0(f" validation loss at iteration {self.iteration} | lm loss value: {ev['lm loss']:.6E} | "
                             f"lm loss PPL: {ev['ppl']:.6E} |")
                if self.writer is not None:
                    self.writer.add_scalar("lm loss validation", ev["lm loss"], self.iteration)
                    if tc.log_validation_ppl_to_tensorboard:
                        self.writer.add_scalar("lm loss validation ppl", ev["ppl"], self.iteration)
            if tc.save and tc.save_interval and self.iteration % tc.save_interval == 0:
                self.save()
            why = self._should_exit()
            if why:
                if tc.save:
                    self.save()
                print_rank_0(f"exiting program at iteration {self.iteration} ({why})")
                if why == "autoresume" and self.mesh.rank == 0:
                    from .watchdog import autoresume_request_resume
                    autoresume_request_resume()          # after the checkpoint is on disk
                break
        if self.heartbeat is not None:
            self.heartbeat.stop()
        return last


def pretrain(argv=None, dataset_provider: Optional[Callable] = None, model_provider: Optional[Callable] = None,
             forward_step: Optional[Callable] = None):
    """Command-line training entry (examples/*/pretrain_*.py:294-302)."""
    from ..config.arguments import parse_args
    from ..data.builders import build_datasets
    args, cfg, par, tc = parse_args(argv)
    if not torch.cuda.is_available():
        par.distributed_backend = "gloo"
    mesh = init_distributed(par)
    print_rank_0(f"> mesh: {mesh.describe()}")
    mem = compute_weight_and_optimizer_memory(cfg, par, verbose=mesh.rank == 0)
    train_ds, valid_ds = (dataset_provider or build_datasets)(args, cfg, tc)
    if tc.eod_mask_loss and tc.eod_token is None:
        # --eod-mask-loss: no loss on the token that follows an end-of-document token; the id comes from the tokenizer
        from ..data.tokenizer import build_tokenizer
        tok, _ = build_tokenizer(args.patch_tokenizer_type, args.tokenizer_model, cfg.vocab_size, args.extra_vocab_size)
        tc.eod_token = getattr(tok, "eod", None)
    trainer = Trainer(cfg, par, tc, mesh, dataset=train_ds, valid_dataset=valid_ds, model_provider=model_provider,
                      forward_step=forward_step)
    print_rank_0(f"> parameters on this rank: {count_parameters(trainer.models):,}")
    if tc.skip_train:
        stats = trainer.evaluate(tc.eval_iters) or {}
        if mesh.rank == 0 and stats:
            print_rank_0("validation: " + " | ".join(f"{k} {float(v):.6E}" for k, v in stats.items()))
        return trainer, stats
    stats = trainer.train()
    if tc.save:
        trainer.save()
        from ..ckpt.legacy import finalize_async_saves
        finalize_async_saves()
    return trainer, stats

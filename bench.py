"""Headline benchmark: training tokens/s of the LASP-2 Linear-Llama3-1B configuration.

Model (benchmark configuration "LASP-2 long-sequence Linear-Llama3 1B dense"): 16 layers of lightning
attention (per-head decay, chunk 64), hidden 2048, 16 heads x 128, SwiGLU ffn 8192, vocab 128256, bf16,
micro-batch 1, sequence parallel over all N GPUs of the node with LASP-2.  Per-GPU work is fixed at
16384 tokens (weak scaling): the sequence is 16384 x N, i.e. the named 131072-token sequence at N = 8.
Synthetic uniform token ids, N(0, 0.02) random-init weights.  One step = forward + backward + gradient
reduction over the sequence-parallel ranks + clip + Adam on fp32 masters.

  python bench.py --gpus 1 --steps K --warmup W
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

``--config`` selects another benchmark configuration together with its parallel layout (``LAYOUTS`` below); the default
is the configuration the headline number is quoted on.

Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with the batch already
on the device; ``e2e`` repeats the measurement through ``Trainer.train_step`` with, every step, the host->device
copy of that step's tokens/labels/mask from pinned memory and a device->host read of the loss.
``--impl reference`` would run the unmodified reference; it cannot be installed offline, so that arm prints why.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

TOKENS_PER_GPU = 16384
METRIC = "train tokens/s per 8xB200 box (LASP-2 Linear-Llama3-1B, lightning attention, 16384 tokens per GPU, seq 131072 at 8 GPUs)"

# Parallel layout, batch and metric of every benchmark configuration that ``--config`` accepts.  The default (and the
# configuration the headline number is quoted on) is the LASP-2 Linear-Llama3-1B one; the others weak-scale the number of
# sequences with the data-parallel size.  ``tp`` is capped by the number of GPUs.
LAYOUTS = {
    "bench-lasp2-llama3-1b": dict(kind="cp", metric=METRIC),
    "bench-a0.3b-2b-gla": dict(kind="ep", tp=1, mbs=8, seq=2048,
                               metric="train tokens/s (A0.3B-2B: 16 x GLA + 64-expert top-8 MoE, EP = N, 8 x 2048 tokens per GPU)"),
    "bench-a1b-7b-hybrid": dict(kind="ep", tp=2, mbs=2, seq=4096,
                                metric="train tokens/s (A1B-7B hybrid LLLN x 6: Gated DeltaNet + attention, 64-expert top-8 MoE, "
                                       "TP2 x EP N/2, 2 x 4096 tokens per data-parallel rank)"),
    "bench-mixtral-mamba2-fp8": dict(kind="ep", tp=2, mbs=1, seq=4096,
                                     metric="train tokens/s (Mixtral-shaped Mamba2 + attention hybrid, 8-expert top-2 MoE, e4m3 "
                                            "projections, TP2 x EP N/2, 4096 tokens per data-parallel rank)"),
}


def resolve_layout(config: str, world: int, zero1: bool = True, overlap: bool = False, tokens_per_gpu: int = TOKENS_PER_GPU):
    """Parallel layout and batch of a benchmark configuration on ``world`` GPUs: ``(layout entry, ParallelConfig keyword
    arguments, sequence length, micro batch, global batch, layout name)``."""
    layout = LAYOUTS.get(config, LAYOUTS["bench-lasp2-llama3-1b"])
    if layout["kind"] == "cp":                       # one sequence split over all GPUs (LASP-2)
        pkw = dict(context_parallel_size=world, use_distributed_optimizer=zero1, overlap_grad_reduce=overlap)
        return layout, pkw, tokens_per_gpu * world, 1, 1, f"sp{world} (LASP-2)"
    # tensor x expert parallel; the number of sequences scales with the data-parallel size
    tp = min(layout["tp"], world)
    pkw = dict(tensor_model_parallel_size=tp, sequence_parallel=tp > 1, expert_model_parallel_size=world // tp,
               use_distributed_optimizer=zero1 and world > tp, overlap_grad_reduce=overlap)
    return layout, pkw, layout["seq"], layout["mbs"], layout["mbs"] * (world // tp), f"tp{tp} ep{world // tp} dp{world // tp}"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--config", type=str, default="bench-lasp2-llama3-1b",
                   help="benchmark configuration: " + ", ".join(LAYOUTS) + " (preset, parallel layout and batch switch together)")
    p.add_argument("--tokens-per-gpu", type=int, default=TOKENS_PER_GPU)
    p.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (marks the result invalid)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--overlap-grad-reduce", action=argparse.BooleanOptionalAction, default=False,
                   help="reduce-scatter the gradients of a block while the backward pass of the blocks before it runs "
                        "(bitwise the same result; measured 2 - 3 ms per step slower than one reduce after backward at N = 2, "
                        "because the reduce kernel takes SM time and HBM bandwidth from the weight-gradient GEMMs)")
    p.add_argument("--zero1", action=argparse.BooleanOptionalAction, default=True,
                   help="distributed optimizer (ZeRO-1) through the fused NVLS kernels when N > 1 (the reference launchers default to DO=true)")
    return p.parse_args()


def reference_arm():
    if int(os.environ.get("RANK", "0")) != 0:          # launched as N ranks: one line, from rank 0
        return 0
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is not installable offline: its source tree has no setup.py/pyproject.toml and its "
                       "engines (megatron-core, transformer_engine, flash-linear-attention submodules, mamba_ssm, "
                       "grouped_gemm) are empty git links or absent from the image"}))
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm()
    import torch
    import torch.distributed as dist
    from linear_moe_b200.config.model_config import ParallelConfig, TrainConfig
    from linear_moe_b200.config.presets import get_preset
    from linear_moe_b200.dist.mesh import init_distributed
    from linear_moe_b200.bench.clocks import ClockSampler
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.parallel import fused_comm
    from linear_moe_b200.train.loop import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    layout, pkw, seq, mbs, gbs, layout_name = resolve_layout(args.config, world, args.zero1, args.overlap_grad_reduce,
                                                             args.tokens_per_gpu)
    par = ParallelConfig(distributed_backend="nccl", **pkw)
    mesh = init_distributed(par)
    dev = torch.device("cuda", torch.cuda.current_device())
    overrides = {}
    if args.layers is not None:
        base = get_preset(args.config)
        overrides["num_layers"] = args.layers
        if base.layer_type_list:
            overrides["layer_type_list"] = (base.layer_type_list * args.layers)[: args.layers]
        if base.hybrid_override_pattern:
            overrides["hybrid_override_pattern"] = (base.hybrid_override_pattern * args.layers)[: args.layers]
    cfg = get_preset(args.config, **overrides)
    tokens_per_step = gbs * seq
    tc = TrainConfig(micro_batch_size=mbs, global_batch_size=gbs, seq_length=seq, train_iters=10 ** 9, lr=1e-4, min_lr=1e-5,
                     lr_decay_style="cosine", lr_decay_iters=100000, lr_warmup_iters=100, weight_decay=0.1,
                     adam_beta1=0.9, adam_beta2=0.95, clip_grad=1.0, bf16=True, log_interval=10 ** 9, seed=1234,
                     check_for_nan_in_loss_and_grad=False,
                     manual_gc=os.environ.get("LMOE_BENCH_MANUAL_GC", "1") != "0")
    if world > 1:
        fused_comm.init_workspaces(mesh, cfg, tc)
    trainer = Trainer(cfg, par, tc, mesh, device=dev)
    n_params = sum(p.numel() for p in trainer.model.parameters())

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps):
        sync()
        K.reset_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.barrier()
        return float(ms) / steps, K.reset_launch_count() // max(steps, 1)

    # ---- device-resident batches (kernel-side number) ---------------------------------------
    resident = [next(trainer.data_iter) for _ in range(4)]
    torch.cuda.synchronize()

    class Cycle:
        def __init__(self, items):
            self.items, self.i = items, 0

        def __iter__(self):
            return self

        def __next__(self):
            self.i += 1
            return self.items[self.i % len(self.items)]
    real_iter = trainer.data_iter
    trainer.data_iter = Cycle(resident)
    for _ in range(max(args.warmup, 3)):
        trainer.train_step()
    sampler = ClockSampler(torch.cuda.current_device()) if mesh.rank == 0 else None
    ms_dev, launches = timed(trainer.train_step, args.steps)
    clocks = sampler.stop() if sampler is not None else None

    # ---- end to end: pinned host batch -> device every step, loss read back every step ----------
    e2e = None
    if not args.no_e2e:
        trainer.data_iter = real_iter
        h2d = sum(v.numel() * v.element_size() for v in resident[0].values())
        last = {}

        def e2e_step():
            st = trainer.train_step()                       # BatchIterator pins + copies this step's batch
            last["loss"] = float(st["lm loss"]) if "lm loss" in st else 0.0   # device -> host read
        for _ in range(2):
            e2e_step()
        ms_e2e, _ = timed(e2e_step, args.steps)
        e2e = {"value": tokens_per_step / (ms_e2e / 1000.0), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")}

    # ---- on-stream time of the fused LASP-2 exchange (push + wait for the other ranks + fold), one extra step ----
    lasp = None
    ws = fused_comm.lasp_workspace(mesh["cp"]) if world > 1 else None
    if ws is not None:
        trainer.data_iter = Cycle(resident)
        ws.timing = []
        trainer.train_step()
        torch.cuda.synchronize()
        us = [a.elapsed_time(b) * 1e3 for a, b in ws.timing]
        ws.timing = None
        t = torch.tensor([sum(us), float(len(us))], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        lasp = {"exchanges_per_step": int(t[1]), "us_per_exchange_max_over_ranks": float(t[0]) / max(float(t[1]), 1.0),
                "share_of_step": float(t[0]) / 1e3 / ms_dev,
                "note": "duration on the compute stream of the fused kernel that pushes the rank's state summary to every peer, "
                        "waits for theirs and folds them; it includes the skew between ranks and nothing of it is hidden"}

    if mesh.rank == 0:
        out = {
            "metric": layout["metric"], "value": tokens_per_step / (ms_dev / 1000.0), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "impl": "ours",
            "config": {"model": args.config, "global_batch": gbs, "seq_len": seq, "tokens_per_gpu": tokens_per_step // world,
                       "parallelism": layout_name + (" zero1" if par.use_distributed_optimizer else "") +
                       (" overlap-grad-reduce" if (args.zero1 and args.overlap_grad_reduce and world > 1) else ""), "params": n_params,
                       "layers": cfg.num_layers, "l2": "inputs larger than L2 (>= 16384 tokens x hidden bf16 activations and GBs of weights per GPU)",
                       "optimizer": "AdamW fp32 masters, clip 1.0", "valid": args.layers is None},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches * args.steps, "gpu_launches_per_step": launches,
        }
        if lasp is not None:
            out["lasp_exchange"] = lasp
        if clocks and clocks.get("sm_mhz"):
            out["ms_x_ghz"] = ms_dev * clocks["sm_mhz"] / 1e3      # clock-normalised step time, to compare runs
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

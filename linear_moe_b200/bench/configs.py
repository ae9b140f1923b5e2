"""Training-step throughput of the named model presets under a chosen parallel layout (secondary benchmarks; the
headline benchmark is ``bench.py`` at the repository root).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29544 \
      -m linear_moe_b200.bench.configs --preset bench-a0.3b-2b-gla --ep N --mbs 8 --seq 2048 [--tp 1] [--layers L]

Synthetic token ids, random-init weights, bf16, AdamW with fp32 masters (ZeRO-1 with ``--zero1``).  ``--steps`` steps are
timed with CUDA events after ``--warmup`` steps (barrier + synchronize on both sides, MAX over ranks); rank 0 prints one
JSON line with the job's aggregate tokens/s.  ``--layers`` shrinks the model (then ``"valid": false``).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--microbatches", type=int, default=1)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--zero1", action="store_true")
    ap.add_argument("--baseline-eager", action="store_true",
                    help="stand-in for the reference's NCCL + cuBLAS build: NCCL collectives instead of the fused peer-memory "
                         "kernels and library GEMMs instead of the tcgen05 dense kernel (same model, same step)")
    ap.add_argument("--torch-profile", type=str, default=None,
                    help="after the timed steps, run one more step under torch.profiler and write the per-operator CUDA-time "
                         "table (grouped by input shape) of rank 0 to this file")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    if a.baseline_eager:
        os.environ["LMOE_TCGEN05_GEMM"] = "0"
    from ..config.model_config import ParallelConfig, TrainConfig
    from ..config.presets import get_preset
    from ..dist.mesh import init_distributed
    from ..ops import cuda as K
    from ..ops import gemm
    from ..parallel import fused_comm
    from ..train.loop import Trainer
    world = int(os.environ.get("WORLD_SIZE", "1"))
    par = ParallelConfig(tensor_model_parallel_size=a.tp, sequence_parallel=a.tp > 1, expert_model_parallel_size=a.ep,
                         context_parallel_size=a.cp, use_distributed_optimizer=a.zero1, distributed_backend="nccl",
                         fused_comm=not a.baseline_eager, overlap_grad_reduce=False)
    mesh = init_distributed(par)
    dev = torch.device("cuda", torch.cuda.current_device())
    over = {}
    if a.layers is not None:
        base = get_preset(a.preset)
        over["num_layers"] = a.layers
        if base.layer_type_list:
            over["layer_type_list"] = (base.layer_type_list * a.layers)[: a.layers]
        if base.hybrid_override_pattern:
            over["hybrid_override_pattern"] = (base.hybrid_override_pattern * a.layers)[: a.layers]
    cfg = get_preset(a.preset, **over)
    gbs = a.mbs * mesh.dp * a.microbatches
    tc = TrainConfig(micro_batch_size=a.mbs, global_batch_size=gbs, seq_length=a.seq, train_iters=10 ** 9, lr=1e-4, min_lr=1e-5,
                     lr_decay_style="cosine", lr_decay_iters=100000, lr_warmup_iters=100, weight_decay=0.1, clip_grad=1.0,
                     bf16=True, log_interval=10 ** 9, seed=1234, check_for_nan_in_loss_and_grad=False,
                     manual_gc=os.environ.get("LMOE_BENCH_MANUAL_GC", "1") != "0")
    trainer = Trainer(cfg, par, tc, mesh, device=dev)
    n_params = sum(p.numel() for m in trainer.models for p in m.parameters())

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    last = None
    for _ in range(max(a.warmup, 1)):
        last = trainer.train_step()
    sync()
    K.reset_launch_count()
    from .clocks import ClockSampler
    sampler = ClockSampler(torch.cuda.current_device()) if mesh.rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        last = trainer.train_step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if sampler is not None else None
    launches = K.reset_launch_count() // a.steps
    fused_comm.check_status("bench configs")
    gemm.check_error()
    mem = torch.cuda.max_memory_allocated() / 2 ** 30
    if mesh.rank == 0:
        tokens = gbs * a.seq
        print(json.dumps({"preset": a.preset, "n_gpus": world, "parallelism": f"tp{a.tp} ep{a.ep} cp{a.cp} dp{mesh.dp}" +
                          (" zero1" if a.zero1 else ""), "tokens_per_step": tokens, "ms_per_step": float(ms),
                          "tokens_per_s": tokens / (float(ms) / 1e3), "params_this_rank": n_params, "layers": cfg.num_layers,
                          "loss": float(last["lm loss"]) if last and "lm loss" in last else None, "own_kernel_launches": launches,
                          "peak_mem_gib": round(mem, 1), "fp8": bool(cfg.fp8), "valid": a.layers is None,
                          "impl": "baseline-eager (NCCL + cuBLAS)" if a.baseline_eager else "ours", "clocks": clocks,
                          "global_batch": gbs, "seq_len": a.seq}))
    if a.torch_profile:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
            trainer.train_step()
            torch.cuda.synchronize()
        if mesh.rank == 0:
            with open(a.torch_profile, "w") as f:
                f.write(prof.key_averages(group_by_input_shape=True).table(sort_by="self_cuda_time_total", row_limit=80,
                                                                            max_name_column_width=48, max_shapes_column_width=100))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Timing of the fused compute + communication kernels against the NCCL + library-GEMM form of the same operator.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
      -m linear_moe_b200.bench.comm [--what all|tp|moe|lasp] [--iters 10]

One rank per GPU.  Every number is timed with CUDA events on the launching stream after 3 warm-up iterations, with a
barrier before each timed iteration, and reported as the MAX over ranks of the per-rank median.  The roofline of a fused
kernel is the slower of FLOPs / measured cuBLAS bf16 peak and NVLink bytes per GPU / 770 GB/s (measured peer copy).
"""
from __future__ import annotations

import argparse
import os
import statistics

import torch
import torch.distributed as dist

from .kernels import peaks

NVLINK_GBS = 770.0


def timeit(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def report(name, ms, flops=None, link_bytes=None):
    if dist.get_rank() != 0:
        return
    _, tf, kind = peaks()
    line = f"{name:58s} {ms * 1e3:9.1f} us"
    bound = 0.0
    if flops is not None:
        t = flops / ms / 1e9
        line += f" | {t:6.0f} TFLOPS/GPU"
        bound = max(bound, flops / (tf * 1e9))
    if link_bytes is not None:
        g = link_bytes / ms / 1e6
        line += f" | {g:5.0f} GB/s/GPU over NVLink"
        bound = max(bound, link_bytes / (NVLINK_GBS * 1e6))
    if bound > 0:
        line += f" | roofline {bound * 1e3:7.1f} us -> {bound / ms:4.2f} of it ({kind} GEMM peak, 770 GB/s link)"
    print(line, flush=True)


def bench_tp(mesh, iters):
    """Sequence-parallel column layer (all-gather -> GEMM) and row layer (GEMM -> reduce-scatter), the A1B-7B hybrid preset
    sizes: hidden 2048, per-rank tokens 4096 * 2 / W, ffn shard 2 * 1408 * 16 / W."""
    from .. import ops
    from ..dist import collectives as C
    from ..parallel import fused_comm
    g = mesh["tp"]
    W = g.size
    dev = torch.device("cuda", torch.cuda.current_device())
    B, T_loc, h = 1, 8192 // W, 2048
    f_loc = 8192 // W
    x = torch.randn(B, T_loc, h, device=dev).bfloat16()
    w1 = (0.02 * torch.randn(f_loc, h, device=dev)).bfloat16()
    w2 = (0.02 * torch.randn(h, f_loc, device=dev)).bfloat16()
    y = torch.randn(B, T_loc * W, f_loc, device=dev).bfloat16()
    fl = 2.0 * B * T_loc * W * h * f_loc
    link = (W - 1) * B * T_loc * h * 2.0                       # bytes one GPU must receive (AG) or send (RS)
    with torch.no_grad():
        t_nccl = timeit(lambda: torch.nn.functional.linear(C.all_gather_raw(x, g, dim=1), w1), iters)
        report(f"TP{W} all-gather (NCCL) + GEMM (cuBLAS)  [{T_loc * W}x{f_loc}x{h}]", t_nccl, fl, link)
        fused_comm._TP[g.name] = fused_comm.TpWorkspace(g, B * T_loc * max(h, f_loc), dev)
        t_f = timeit(lambda: ops.allgather_linear(x, w1, None, g, dim=1), iters)
        report(f"TP{W} all-gather -> GEMM fused (copier CTAs + local TMA)", t_f, fl, link)
        del fused_comm._TP[g.name]
        t_nccl = timeit(lambda: C.reduce_scatter_raw(torch.nn.functional.linear(y, w2)[0], g, dim=0), iters)
        report(f"TP{W} GEMM (cuBLAS) + reduce-scatter (NCCL)  [{T_loc * W}x{h}x{f_loc}]", t_nccl, fl, link)
        fused_comm._TP[g.name] = fused_comm.TpWorkspace(g, B * T_loc * max(h, f_loc), dev)
        t_f = timeit(lambda: ops.linear_reducescatter(y, w2, g, dim=1), iters)
        report(f"TP{W} GEMM -> reduce-scatter fused (peer-store epilogue + reduce)", t_f, fl, link)
        fused_comm.check_status("bench tp")


def bench_moe(mesh, iters):
    """Expert-parallel MoE layer core of the A0.3B-2B GLA preset: hidden 1024, expert ffn 896, 64 experts, top-8."""
    from ..config.model_config import ModelConfig
    from ..models.moe import MoELayer
    from ..parallel import fused_comm
    ep = mesh["ep"]
    W = ep.size
    dev = torch.device("cuda", torch.cuda.current_device())
    E = 64 if 64 % W == 0 else 8 * W
    cfg = ModelConfig(num_layers=2, hidden_size=1024, num_attention_heads=8, ffn_hidden_size=896, vocab_size=1024, num_experts=E,
                      moe_topk=8, moe_ffn_hidden_size=896, params_dtype=torch.bfloat16, moe_aux_loss_coeff=0.0)
    layer = MoELayer(cfg, mesh, 1, "layers.0.mlp", device=dev).to(dev)
    T = 8192
    x = torch.randn(1, T, 1024, device=dev).bfloat16()
    fl = 2.0 * T * 8 * 1024 * 3 * 896                          # expert FLOPs of this rank's share (balanced routing)
    link = 2.0 * T * 8 * 1024 * 2 * (W - 1) / W                # dispatch + combine bytes leaving one GPU
    with torch.no_grad():
        t_nccl = timeit(lambda: layer(x), iters)
        report(f"EP{W} MoE layer fwd, NCCL all-to-all path  [T={T}, top-8 of {E}]", t_nccl, fl, link)
        fused_comm._MOE[ep.name] = fused_comm.MoeWorkspace(ep, E, 1024, 3 * T * 8, dev)
        t_f = timeit(lambda: layer(x), iters)
        report(f"EP{W} MoE layer fwd, peer-memory push / pull path", t_f, fl, link)
    xg = x.clone().requires_grad_(True)

    def step():
        layer.zero_grad(set_to_none=True)
        xg.grad = None
        layer(xg).sum().backward()
    t_f = timeit(step, iters)
    report(f"EP{W} MoE layer fwd+bwd, peer-memory path", t_f, 3 * fl, 2 * link)
    del fused_comm._MOE[ep.name]
    t_nccl = timeit(step, iters)
    report(f"EP{W} MoE layer fwd+bwd, NCCL all-to-all path", t_nccl, 3 * fl, 2 * link)
    fused_comm.check_status("bench moe")


def bench_lasp(mesh, iters):
    """LASP-2 lightning attention of the LASP-2 Linear-Llama3-1B preset: 16 heads x 128, 16384 tokens per rank."""
    from ..parallel import fused_comm
    from ..parallel.lasp2 import lasp2
    cp = mesh["cp"]
    dev = torch.device("cuda", torch.cuda.current_device())
    B, T, H, D = 1, 16384, 16, 128
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev)).bfloat16()
    gdec = -torch.linspace(0.01, 0.3, H, device=dev)
    link = (cp.size - 1) * B * H * D * D * 4.0
    with torch.no_grad():
        q, k, v = qkv.split(D, dim=-1)
        t_nccl = timeit(lambda: lasp2("scalar", q, k, v, group=cp, g=gdec, scale=None), iters)
        report(f"CP{cp.size} lightning attention fwd, all-gather of states (NCCL)", t_nccl, None, link)
        fused_comm._LASP[cp.name] = fused_comm.LaspWorkspace(cp, B * H * D * D, dev)
        t_f = timeit(lambda: lasp2("scalar", q, k, v, group=cp, g=gdec, scale=None), iters)
        report(f"CP{cp.size} lightning attention fwd, exchange fused into the combine kernel", t_f, None, link)
        fused_comm.check_status("bench lasp")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="all")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    from ..config.model_config import ParallelConfig
    from ..dist.mesh import Mesh
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    if a.what in ("tp", "all") and world <= 8:
        bench_tp(Mesh(ParallelConfig(tensor_model_parallel_size=world, sequence_parallel=True)), a.iters)
    if a.what in ("moe", "all"):
        bench_moe(Mesh(ParallelConfig(expert_model_parallel_size=world)), a.iters)
    if a.what in ("lasp", "all"):
        bench_lasp(Mesh(ParallelConfig(context_parallel_size=world)), a.iters)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Multi-GPU tests of the fused compute+communication kernels (2 GPUs of one box, NCCL + symmetric memory).

Every rank checks the fused path against the same operator run on the whole sequence on its own GPU.
"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from dist_utils import run_distributed


def _need_gpus(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _lasp_worker(rank, world, D, decay, T):
    from linear_moe_b200 import ops
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.parallel import fused_comm
    from linear_moe_b200.parallel.lasp2 import lasp2
    dev = torch.device("cuda", rank)
    par = ParallelConfig(context_parallel_size=world)
    mesh = Mesh(par)
    B, H = 1, 4
    fused_comm._LASP[mesh["cp"].name] = fused_comm.LaspWorkspace(mesh["cp"], B * H * D * D, dev, spin_limit=2_000_000)
    torch.manual_seed(0)
    qkv = (0.5 * torch.randn(B, T * world, H, 3 * D, device=dev)).to(torch.bfloat16)
    go = torch.randn(B, T * world, H, D, device=dev).to(torch.bfloat16)
    g = -torch.tensor([0.01, 0.05, 0.2, 0.0], device=dev) if decay else None
    # whole sequence on this GPU
    full = qkv.clone().requires_grad_(True)
    q, k, v = full.split(D, dim=-1)
    o_ref, _ = ops.lsm_scalar(q, k, v, g, None, None, 64)
    o_ref.backward(go)
    # this rank's slice through the fused LASP-2 path, three calls in a row (slot/epoch bookkeeping)
    errs = []
    for it in range(3):
        loc = qkv[:, rank * T:(rank + 1) * T].clone().requires_grad_(True)
        ql, kl, vl = loc.split(D, dim=-1)
        o, _ = lasp2("scalar", ql, kl, vl, group=mesh["cp"], g=g, scale=None)
        o.backward(go[:, rank * T:(rank + 1) * T])
        torch.cuda.synchronize()
        fused_comm.check_status("lasp test")
        eo = (o.float() - o_ref[:, rank * T:(rank + 1) * T].float()).abs().max().item()
        eg = (loc.grad.float() - full.grad[:, rank * T:(rank + 1) * T].float()).abs().max().item()
        errs.append((eo, eg))
    scale_o = o_ref.float().abs().max().item()
    scale_g = full.grad.float().abs().max().item()
    return errs, scale_o, scale_g


@pytest.mark.parametrize("D,decay,T", [(128, True, 1024), (64, False, 300)])
def test_lasp2_fused_matches_single_gpu(D, decay, T):
    _need_gpus(2)
    outs = run_distributed(_lasp_worker, 2, backend="nccl", D=D, decay=decay, T=T)
    for errs, so, sg in outs:
        for eo, eg in errs:
            assert eo < 3e-2 * so, (errs, so)
            assert eg < 4e-2 * sg, (errs, sg)

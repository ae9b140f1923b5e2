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
    # four slots only: the six exchanges below pass through the slot-reuse guard (a stream-ordered catch-up of all ranks)
    fused_comm._LASP[mesh["cp"].name] = fused_comm.LaspWorkspace(mesh["cp"], B * H * D * D, dev, spin_limit=2_000_000, nslot=4)
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
    first = None
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
        # the exchange folds the ranks' summaries in a fixed order: repeated calls agree bit for bit
        if first is None:
            first = (o.detach().clone(), loc.grad.clone())
        else:
            assert torch.equal(o, first[0]) and torch.equal(loc.grad, first[1]), "fused LASP-2 is not run-to-run deterministic"
    scale_o = o_ref.float().abs().max().item()
    scale_g = full.grad.float().abs().max().item()
    return errs, scale_o, scale_g


def _lasp_gated_worker(rank, world, kind, D, T):
    """Data-dependent decays through the fused exchange: per-token scalar gates (``scalar``: Mamba2 SSD, simple GLA) and
    per-key-channel gates (``vector``: GLA, HGRN2, RWKV6)."""
    from linear_moe_b200 import ops
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.parallel import fused_comm
    from linear_moe_b200.parallel.lasp2 import lasp2
    dev = torch.device("cuda", rank)
    mesh = Mesh(ParallelConfig(context_parallel_size=world))
    B, H = 2, 3
    fused_comm._LASP[mesh["cp"].name] = fused_comm.LaspWorkspace(mesh["cp"], B * H * D * D, dev, spin_limit=2_000_000)
    torch.manual_seed(1)
    Tt = T * world
    qkv = (0.5 * torch.randn(B, Tt, H, 3 * D, device=dev)).to(torch.bfloat16)
    go = torch.randn(B, Tt, H, D, device=dev).to(torch.bfloat16)
    if kind == "scalar":
        gate = torch.nn.functional.logsigmoid(torch.randn(B, Tt, H, device=dev) + 3.0)
    else:
        gate = torch.nn.functional.logsigmoid(torch.randn(B, Tt, H, D, device=dev) + 3.0) / 4
    sl = slice(rank * T, (rank + 1) * T)

    def run(x, gt, group):
        q, k, v = x.split(D, dim=-1)
        if group is None:
            return (ops.lsm_scalar(q, k, v, gt, None, None, 64) if kind == "scalar"
                    else ops.lsm_vector(q, k, v, gt, None, None, None, 64))[0]
        return lasp2(kind, q, k, v, group=group, g=gt if kind == "scalar" else None, gk=gt if kind == "vector" else None)[0]
    full, gfull = qkv.clone().requires_grad_(True), gate.clone().requires_grad_(True)
    o_ref = run(full, gfull, None)
    o_ref.backward(go)
    K.reset_launch_count()
    loc, gloc = qkv[:, sl].clone().requires_grad_(True), gate[:, sl].clone().requires_grad_(True)
    calls0 = fused_comm.lasp_workspace(mesh["cp"]).calls
    o = run(loc, gloc, mesh["cp"])
    o.backward(go[:, sl])
    torch.cuda.synchronize()
    fused_comm.check_status("lasp gated test")
    assert fused_comm.lasp_workspace(mesh["cp"]).calls == calls0 + 2, "the fused exchange was not used"
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()
    return rel(o, o_ref[:, sl]), rel(loc.grad, full.grad[:, sl]), rel(gloc.grad, gfull.grad[:, sl])


@pytest.mark.parametrize("kind,D,T", [("scalar", 128, 512), ("vector", 128, 512), ("vector", 64, 200)])
def test_lasp2_fused_data_dependent_decay(kind, D, T):
    _need_gpus(2)
    outs = run_distributed(_lasp_gated_worker, 2, backend="nccl", kind=kind, D=D, T=T)
    for eo, eg, edecay in outs:
        assert eo < 2e-2 and eg < 3e-2 and edecay < 3e-2, (kind, eo, eg, edecay)


@pytest.mark.parametrize("D,decay,T", [(128, True, 1024), (64, False, 300)])
def test_lasp2_fused_matches_single_gpu(D, decay, T):
    _need_gpus(2)
    outs = run_distributed(_lasp_worker, 2, backend="nccl", D=D, decay=decay, T=T)
    for errs, so, sg in outs:
        for eo, eg in errs:
            assert eo < 3e-2 * so, (errs, so)
            assert eg < 4e-2 * sg, (errs, sg)


def _zero_worker(rank, world, multicast):
    from linear_moe_b200.config.model_config import ParallelConfig, TrainConfig
    from linear_moe_b200.config.presets import get_preset
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.parallel import fused_comm
    from linear_moe_b200.train.loop import Trainer
    dev = torch.device("cuda", rank)
    if not multicast:
        orig = fused_comm.ZeroBufferWorkspace.__init__
        fused_comm.ZeroBufferWorkspace.__init__ = lambda self, g, n, d, **kw: orig(self, g, n, d, use_multicast=False)
    cfg = get_preset("bench-lasp2-llama3-1b", num_layers=2, layer_type_list="LL", vocab_size=2048, hidden_size=256,
                     num_attention_heads=2, ffn_hidden_size=512)
    outs = {}
    for fused in (True, False, "no_overlap"):
        par = ParallelConfig(use_distributed_optimizer=True, fused_comm=bool(fused), overlap_grad_reduce=fused is True)
        mesh = Mesh(par)
        tc = TrainConfig(micro_batch_size=1, global_batch_size=world, seq_length=256, train_iters=4, bf16=True,
                         log_interval=1000, lr=1e-3, min_lr=1e-3, lr_decay_style="constant", seed=7)
        tr = Trainer(cfg, par, tc, mesh, device=dev)
        assert (tr.optimizer.buffers[0].fused is not None) == bool(fused)
        if fused is True:
            assert getattr(tr.model, "grad_ready_hook", None) is not None, "the bucketed reduce is not wired"
        losses = [float(tr.train_step()["lm loss"]) for _ in range(4)]
        if fused is True:
            fb = [b for b in tr.optimizer.buffers if b.fused is not None]
            assert any(tr.optimizer._layer_range(b, 0) is not None for b in fb), "no block maps to a gradient bucket"
            assert max(b.fused._next_slot for b in fb) > 2, "the reduce-scatter was not split into buckets"
        torch.cuda.synchronize()
        fused_comm.check_status("zero test")
        outs[fused] = (losses, torch.cat([b.params.float().cpu() for b in tr.optimizer.buffers]))
    # the bucketed reduce-scatter that overlaps the backward pass sums the same values in the same order as the single
    # launch after it: parameters must agree bit for bit
    assert torch.equal(outs[True][1], outs["no_overlap"][1]), "overlapped and non-overlapped fused ZeRO-1 differ"
    return outs[True][0], outs[False][0], (outs[True][1] - outs[False][1]).abs().max().item(), outs[False][1].abs().max().item()


@pytest.mark.parametrize("multicast", [True, False])
def test_zero1_fused_matches_nccl(multicast):
    """ZeRO-1 step through the fused NVLS kernels (multimem reduce / multimem store) or their peer-pointer variant
    equals the reduce-scatter / Adam / all-gather path on NCCL."""
    _need_gpus(2)
    outs = run_distributed(_zero_worker, 2, backend="nccl", multicast=multicast)
    for lf, ln, dmax, pmax in outs:
        assert all(abs(a - b) < 2e-2 for a, b in zip(lf, ln)), (lf, ln)
        assert dmax < 2e-2 * pmax + 4e-3, (dmax, pmax)
    assert outs[0][0][-1] < outs[0][0][0]


def _moe_worker(rank, world):
    from linear_moe_b200.config.model_config import ModelConfig, ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.models.moe import MoELayer
    from linear_moe_b200.ops import gemm
    from linear_moe_b200.parallel import fused_comm
    dev = torch.device("cuda", rank)
    mesh = Mesh(ParallelConfig(expert_model_parallel_size=world))
    cfg = ModelConfig(num_layers=2, hidden_size=256, num_attention_heads=2, ffn_hidden_size=512, vocab_size=1024,
                      num_experts=8, moe_topk=2, moe_ffn_hidden_size=128, params_dtype=torch.bfloat16)
    layer = MoELayer(cfg, mesh, 1, "layers.0.mlp", device=dev).to(dev)
    torch.manual_seed(100 + rank)                       # every rank routes its own tokens
    T = 700 + 40 * rank
    x = torch.randn(1, T, 256, device=dev).to(torch.bfloat16)
    go = torch.randn(1, T, 256, device=dev).to(torch.bfloat16)

    def run():
        xx = x.clone().requires_grad_(True)
        for p in layer.parameters():
            p.grad = None
        out = layer(xx)
        out.backward(go)
        torch.cuda.synchronize()
        return [out.float(), xx.grad.float()] + [p.grad.float() for p in layer.parameters()]

    ref = run()                                          # NCCL all-to-all path (no workspace yet)
    fused_comm._MOE[mesh["ep"].name] = fused_comm.MoeWorkspace(mesh["ep"], 8, 256, 4 * 800 * 2, dev)
    assert layer._fused_workspace(x.view(-1, 256)) is not None
    errs = []
    first = None
    for it in range(3):
        got = run()
        fused_comm.check_status("moe fused test")
        gemm.check_error()
        errs.append([((a - b).abs().max().item(), b.abs().max().item()) for a, b in zip(got, ref)])
        # rows are placed by prefix sums (no atomics) and every token sums its k expert outputs in slot order:
        # the layer's output and input gradient repeat bit for bit
        if first is None:
            first = got
        else:
            assert torch.equal(got[0], first[0]) and torch.equal(got[1], first[1]), "fused MoE exchange is not deterministic"
    return errs


def test_moe_fused_dispatch_combine_matches_nccl_path():
    _need_gpus(2)
    outs = run_distributed(_moe_worker, 2, backend="nccl")
    for errs in outs:
        for it in errs:
            for err, scale in it:
                assert err <= 3e-2 * scale + 1e-3, (err, scale)


def _tp_worker(rank, world, B, T_loc, h, f):
    from linear_moe_b200 import ops
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.ops import gemm
    from linear_moe_b200.parallel import fused_comm
    dev = torch.device("cuda", rank)
    mesh = Mesh(ParallelConfig(tensor_model_parallel_size=world, sequence_parallel=True))
    g = mesh["tp"]
    torch.manual_seed(5 + rank)
    x = torch.randn(B, T_loc, h, device=dev).to(torch.bfloat16)
    w1 = (0.05 * torch.randn(f, h, device=dev)).to(torch.bfloat16)          # column-parallel shard [f_loc, h]
    b1 = (0.1 * torch.randn(f, device=dev)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(h, f, device=dev)).to(torch.bfloat16)          # row-parallel shard [h, f_loc]
    go = torch.randn(B, T_loc, h, device=dev).to(torch.bfloat16)

    def run():
        ins = [t.clone().requires_grad_(True) for t in (x, w1, b1, w2)]
        y = ops.allgather_linear(ins[0], ins[1], ins[2], g, dim=1)         # [B, W*T_loc, f]
        z = ops.linear_reducescatter(torch.nn.functional.silu(y), ins[3], g, dim=1)
        z.backward(go)
        torch.cuda.synchronize()
        return [z.float(), y.float()] + [t.grad.float() for t in ins]

    ref = run()                                                             # NCCL collectives + cuBLAS
    fused_comm._TP[g.name] = fused_comm.TpWorkspace(g, B * T_loc * max(h, f), dev)
    errs = []
    for it in range(3):
        got = run()
        fused_comm.check_status("tp fused test")
        gemm.check_error()
        errs.append([((a - b).abs().max().item(), b.abs().max().item()) for a, b in zip(got, ref)])
    assert fused_comm._TP[g.name].ag_calls == 9 and fused_comm._TP[g.name].rs_calls == 6
    return errs


@pytest.mark.parametrize("B,T_loc,h,f", [(1, 512, 512, 1024), (2, 128, 256, 328)])
def test_tp_fused_allgather_gemm_and_gemm_reducescatter(B, T_loc, h, f):
    _need_gpus(2)
    outs = run_distributed(_tp_worker, 2, backend="nccl", B=B, T_loc=T_loc, h=h, f=f)
    for errs in outs:
        for it in errs:
            for err, scale in it:
                assert err <= 2e-2 * scale + 1e-3, (err, scale)


def _model_worker(rank, world, par_kw, overrides, steps):
    from linear_moe_b200.config.model_config import ParallelConfig, TrainConfig
    from linear_moe_b200.config.presets import get_preset
    from linear_moe_b200.data.datasets import SyntheticTokenDataset
    from linear_moe_b200.dist.mesh import Mesh, single_process_mesh
    from linear_moe_b200.ops import gemm
    from linear_moe_b200.parallel import fused_comm
    from linear_moe_b200.train.loop import Trainer
    dev = torch.device("cuda", rank)
    seq, gbs = 512, 2
    cfg = get_preset("bench-cpu-plumbing", params_dtype=torch.bfloat16, **overrides)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, num_samples=gbs, seed=0)

    def train(mesh, par):
        tc = TrainConfig(micro_batch_size=2 if mesh.dp == 1 else 1, global_batch_size=gbs, seq_length=seq, train_iters=steps,
                         lr=1e-3, min_lr=1e-3, lr_decay_style="constant", weight_decay=0.0, clip_grad=0.0,
                         log_interval=1, seed=0, bf16=True)
        tr = Trainer(cfg, par, tc, mesh, device=dev, dataset=ds)
        out = []
        for _ in range(steps):
            st = tr.train_step()
            out.append((float(st["lm loss"]), float(st["grad_norm"])))
        gemm.check_error()
        return out

    multi = train(Mesh(ParallelConfig(**par_kw)), ParallelConfig(**par_kw))
    used = dict(tp=sum(w.ag_calls for w in fused_comm._TP.values()), moe=sum(w.ep_push for w in fused_comm._MOE.values()),
                lasp=sum(w.calls for w in fused_comm._LASP.values()))
    single = train(single_process_mesh(), ParallelConfig()) if rank == 0 else None
    return multi, single, used


@pytest.mark.parametrize("name,par_kw,overrides,expect", [
    ("tp2_sp", dict(tensor_model_parallel_size=2, sequence_parallel=True), dict(layer_type_list="LN"), "tp moe"),
    ("ep2", dict(expert_model_parallel_size=2), dict(), "moe"),
    ("cp2_zero1", dict(context_parallel_size=2, use_distributed_optimizer=True),
     dict(la_module="lightning_attention", kv_channels=64), "lasp"),
])
def test_two_gpu_training_matches_one_gpu(name, par_kw, overrides, expect):
    """bf16 training steps of the small MoE model split over 2 GPUs (fused communication kernels on) against 1 GPU."""
    _need_gpus(2)
    outs = run_distributed(_model_worker, 2, backend="nccl", par_kw=par_kw, overrides=overrides, steps=3)
    multi, single, used = outs[0]
    for e in expect.split():
        assert used[e] > 0, f"the fused {e} path was not used: {used}"
    for (l, g), (l0, g0) in zip(multi, single):
        assert abs(l - l0) < 5e-2, (multi, single)
    assert abs(multi[0][1] - single[0][1]) < 0.1 * single[0][1], (multi, single)


def _resume_worker(rank, world, tmp):
    """Train 2 steps, checkpoint, train 2 more; a fresh trainer that loads the checkpoint reproduces steps 3-4."""
    from linear_moe_b200.config.model_config import ParallelConfig, TrainConfig
    from linear_moe_b200.config.presets import get_preset
    from linear_moe_b200.data.datasets import SyntheticTokenDataset
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.train.loop import Trainer
    dev = torch.device("cuda", rank)
    seq, gbs = 512, 4
    cfg = get_preset("bench-cpu-plumbing", params_dtype=torch.bfloat16, la_module="lightning_attention", kv_channels=64)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, num_samples=64, seed=0)
    par = ParallelConfig(context_parallel_size=2, use_distributed_optimizer=True)     # fused LASP-2 + fused ZeRO-1
    mesh = Mesh(par)

    def make():
        tc = TrainConfig(micro_batch_size=2, global_batch_size=gbs, seq_length=seq, train_iters=4, lr=1e-3, min_lr=1e-4,
                         lr_decay_style="cosine", lr_decay_iters=100, weight_decay=0.01, clip_grad=1.0, log_interval=1,
                         seed=0, bf16=True)
        return Trainer(cfg, par, tc, mesh, device=dev, dataset=ds)
    a = make()
    for _ in range(2):
        a.train_step()
    a.save(tmp)
    cont = [float(a.train_step()["lm loss"]) for _ in range(2)]
    b = make()
    b.load(tmp)
    assert b.iteration == 2
    resumed = [float(b.train_step()["lm loss"]) for _ in range(2)]
    return cont, resumed


def test_checkpoint_resume_with_fused_paths(tmp_path):
    _need_gpus(2)
    outs = run_distributed(_resume_worker, 2, backend="nccl", tmp=str(tmp_path / "ckpt"))
    cont, resumed = outs[0]
    for x, y in zip(cont, resumed):
        assert abs(x - y) < 2e-3, (cont, resumed)

"""Benchmark configuration #1: the CPU plumbing run.

2-layer basic linear attention (elu+1) + MoE (4 experts, top-2, ffn 512), hidden 256, 4 heads x 64,
vocab 32000, seq 512, micro-batch 2, fp32, Adam lr 1e-3, 10 steps, gloo world 2.  The loss must go
down and the logits after training must match the single-process run, for every way of splitting the
job over two ranks.
"""
import pytest
import torch

from linear_moe_b200.config.model_config import ParallelConfig, TrainConfig
from linear_moe_b200.config.presets import get_preset
from linear_moe_b200.data.datasets import SyntheticTokenDataset
from linear_moe_b200.dist import collectives as C
from linear_moe_b200.dist.mesh import Mesh, single_process_mesh
from linear_moe_b200.train.loop import Trainer

from dist_utils import run_distributed

STEPS = 10


def _train(mesh, par, overrides=None, steps=STEPS, seq=512, gbs=2):
    cfg = get_preset("bench-cpu-plumbing", **(overrides or {}))
    tc = TrainConfig(micro_batch_size=2 if mesh.dp == 1 else 1, global_batch_size=gbs, seq_length=seq,
                     train_iters=steps, lr=1e-3, min_lr=1e-3, lr_decay_style="constant", weight_decay=0.0,
                     clip_grad=0.0, log_interval=1000, seed=0)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, num_samples=gbs, seed=0)   # one fixed batch, repeated
    tr = Trainer(cfg, par, tc, mesh, device=torch.device("cpu"), dataset=ds)
    losses, gnorms = [], []
    for _ in range(steps):
        st = tr.train_step()
        gnorms.append(st["grad_norm"])
        if "lm loss" in st:
            losses.append(float(st["lm loss"]))
    # logits of the first sample after training, gathered to full [T, V] on every rank that has them
    tr.model.eval()
    sample = torch.stack([ds[0]["text"], ds[1]["text"]])[:, :-1]
    with torch.no_grad():
        logits = _full_logits(tr, sample, mesh)
    return losses, logits, gnorms


def _full_logits(tr, tokens, mesh):
    cp = mesh["cp"]
    if not cp.is_trivial:
        n = tokens.shape[1] // cp.size
        tokens = tokens[:, cp.rank * n:(cp.rank + 1) * n]
    if mesh.pp > 1:
        from linear_moe_b200.train.schedules import _send, _recv, _drain
        h = None
        if not mesh.is_first_stage:
            h = _recv((tokens.shape[0], tokens.shape[1], tr.cfg.hidden_size), torch.float32, "cpu",
                      mesh.prev_stage_rank, mesh)
        out = tr.model(tokens, None, hidden_in=h)
        if not mesh.is_last_stage:
            _send(out, mesh.next_stage_rank, mesh)
            _drain()
            return None
        logits = out
    else:
        logits = tr.model(tokens)
    if not cp.is_trivial:
        logits = C.all_gather_raw(logits.contiguous(), cp, dim=1)
    return logits[:, :64].clone()


def _worker(rank, world, par_kw, overrides):
    par = ParallelConfig(distributed_backend="gloo", **par_kw)
    mesh = Mesh(par)
    return _train(mesh, par, overrides)


@pytest.fixture(scope="module")
def single():
    return _train(single_process_mesh(), ParallelConfig())


def test_single_process_loss_decreases(single):
    losses, _, _ = single
    assert len(losses) == STEPS
    assert losses[-1] < losses[0] - 0.05, losses


@pytest.mark.parametrize("name,par_kw,overrides", [
    ("dp2", dict(), None),
    ("dp2_zero1", dict(use_distributed_optimizer=True), None),
    ("tp2_sp", dict(tensor_model_parallel_size=2, sequence_parallel=True), None),
    ("ep2", dict(expert_model_parallel_size=2), None),
    ("ep2_allgather_dispatcher", dict(expert_model_parallel_size=2), dict(moe_token_dispatcher_type="allgather")),
    ("tp2_sp_allgather_dispatcher", dict(tensor_model_parallel_size=2, sequence_parallel=True),
     dict(moe_token_dispatcher_type="allgather")),
    ("cp2_lasp2", dict(context_parallel_size=2), None),
    ("pp2", dict(pipeline_model_parallel_size=2), None),
])
def test_world2_matches_single_process(single, name, par_kw, overrides):
    ref_losses, ref_logits, ref_gn = single
    outs = run_distributed(_worker, 2, par_kw=par_kw, overrides=overrides)
    losses = next(o[0] for o in outs if o[0])
    logits = next(o[1] for o in outs if o[1] is not None)
    gn = outs[0][2]
    assert losses[-1] < losses[0] - 0.05
    # the first steps pin exact agreement of forward, backward and the reduced gradients; Adam then
    # amplifies fp32 reduction-order noise, so the 10-step trajectory gets a looser bound
    assert abs(losses[0] - ref_losses[0]) < 2e-5 and abs(losses[1] - ref_losses[1]) < 5e-5, (losses, ref_losses)
    assert abs(gn[0] - ref_gn[0]) < 1e-4 * ref_gn[0], (gn, ref_gn)
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=3e-3), (losses, ref_losses)
    rel = (logits - ref_logits).norm() / ref_logits.norm()
    assert rel < 2e-2, rel


def _train_vpp(mesh, par, steps=3, seq=128, gbs=4):
    cfg = get_preset("bench-cpu-plumbing", num_layers=4, layer_type_list="LLLL")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=gbs, seq_length=seq, train_iters=steps, lr=1e-3, min_lr=1e-3,
                     lr_decay_style="constant", weight_decay=0.0, clip_grad=0.0, log_interval=1000, seed=0)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, num_samples=gbs, seed=0)
    tr = Trainer(cfg, par, tc, mesh, device=torch.device("cpu"), dataset=ds)
    losses, gnorms = [], []
    for _ in range(steps):
        st = tr.train_step()
        gnorms.append(st["grad_norm"])
        if "lm loss" in st:
            losses.append(float(st["lm loss"]))
    return losses, gnorms


def _worker_vpp(rank, world, par_kw):
    par = ParallelConfig(distributed_backend="gloo", **par_kw)
    return _train_vpp(Mesh(par), par)


@pytest.mark.parametrize("par_kw", [
    dict(pipeline_model_parallel_size=2, virtual_pipeline_model_parallel_size=2),     # interleaved: 2 model chunks per stage
    dict(pipeline_model_parallel_size=2),                                             # 1F1B with 4 micro-batches in flight
])
def test_pipeline_schedules_match_single_process(par_kw):
    """Four layers on two pipeline stages (as two interleaved chunks per stage, or one), four micro-batches per step,
    against gradient accumulation in one process: same losses and gradient norms."""
    ref_losses, ref_gn = _train_vpp(single_process_mesh(), ParallelConfig())
    outs = run_distributed(_worker_vpp, 2, par_kw=par_kw)
    losses = next(o[0] for o in outs if o[0])
    gn = outs[0][1]
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=2e-4), (losses, ref_losses)
    assert torch.allclose(torch.tensor(gn), torch.tensor(ref_gn), rtol=2e-3), (gn, ref_gn)


def _train_shared(mesh, par, kw, steps=3, seq=64, gbs=4):
    cfg = get_preset("bench-cpu-plumbing", num_layers=4, num_experts=None, ffn_hidden_size=256, **kw)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=gbs, seq_length=seq, train_iters=steps, lr=3e-4, min_lr=3e-4,
                     lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, log_interval=1000, seed=0)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, num_samples=gbs, seed=0)
    tr = Trainer(cfg, par, tc, mesh, device=torch.device("cpu"), dataset=ds)
    losses, gnorms = [], []
    for _ in range(steps):
        st = tr.train_step()
        gnorms.append(st["grad_norm"])
        if "lm loss" in st:
            losses.append(float(st["lm loss"]))
    shared = {n: p.detach().clone() for m in tr.models for n, p in m.named_parameters()
              if getattr(p, "pp_shared_grad", None) is not None or "word_embeddings" in n or "lower_bounds" in n}
    return losses, gnorms, shared


def _worker_shared(rank, world, kw, par_kw):
    par = ParallelConfig(distributed_backend="gloo", **par_kw)
    return _train_shared(Mesh(par), par, kw)


@pytest.mark.parametrize("kw,par_kw", [
    (dict(tie_embeddings=True, layer_type_list="LLLL"), dict(pipeline_model_parallel_size=2)),
    (dict(la_module="hgrn2", la_feature_map=None, hgrn2_lower_bound=True, layer_type_list="LLLL"),
     dict(pipeline_model_parallel_size=2)),
    (dict(la_module="hgrn2", la_feature_map=None, hgrn2_lower_bound=True, layer_type_list="LLLL", tie_embeddings=True),
     dict(pipeline_model_parallel_size=2, virtual_pipeline_model_parallel_size=2)),
], ids=["tied_embeddings_pp2", "hgrn2_lower_bounds_pp2", "both_pp2_vpp2"])
def test_parameters_shared_across_pipeline_stages(kw, par_kw):
    """Tied input / output embeddings whose two uses sit on different pipeline stages, and HGRN2's lower-bound table that
    every stage (and interleaved model chunk) needs in full: the copies' gradients are summed, counted once in the
    gradient norm, and the copies stay equal while training matches the single-process run with clipping active."""
    ref_losses, ref_gn, ref_shared = _train_shared(single_process_mesh(), ParallelConfig(), kw)
    outs = run_distributed(_worker_shared, 2, kw=kw, par_kw=par_kw)
    losses = next(o[0] for o in outs if o[0])
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=3e-4), (losses, ref_losses)
    # the first step pins the gradients (fp32 accumulation order only); Adam's first updates then amplify rounding noise
    assert abs(outs[0][1][0] - ref_gn[0]) < 5e-4 * ref_gn[0], (outs[0][1], ref_gn)
    assert torch.allclose(torch.tensor(outs[0][1]), torch.tensor(ref_gn), rtol=2e-2), (outs[0][1], ref_gn)
    assert outs[1][1] == outs[0][1]
    if kw.get("tie_embeddings"):
        emb = next(v for n, v in outs[0][2].items() if "word_embeddings" in n)
        head = next(v for n, v in outs[1][2].items() if "output_layer" in n)
        assert torch.equal(emb, head)
        assert torch.allclose(emb, next(v for n, v in ref_shared.items() if "word_embeddings" in n), atol=2e-4)
    if kw.get("hgrn2_lower_bound"):
        tables = [v for o in outs for n, v in o[2].items() if "lower_bounds" in n]
        assert len(tables) >= 2 and all(torch.equal(t, tables[0]) for t in tables)
        assert tables[0].abs().max() > 0
        assert torch.allclose(tables[0], next(v for n, v in ref_shared.items() if "lower_bounds" in n), atol=2e-4)


def _train_rnn(mesh, par, la, steps=3, seq=64):
    cfg = get_preset("bench-cpu-plumbing", la_module=la, la_feature_map=None, num_experts=None, ffn_hidden_size=256,
                     hgrn2_lower_bound=la == "hgrn2")
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=seq, train_iters=steps, lr=1e-3, min_lr=1e-3,
                     lr_decay_style="constant", weight_decay=0.0, clip_grad=0.0, log_interval=1000, seed=0)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, num_samples=2, seed=0)
    tr = Trainer(cfg, par, tc, mesh, device=torch.device("cpu"), dataset=ds)
    out = [tr.train_step() for _ in range(steps)]
    return [float(o["lm loss"]) for o in out], [o["grad_norm"] for o in out]


def _worker_rnn(rank, world, la, sp=False):
    par = ParallelConfig(distributed_backend="gloo", tensor_model_parallel_size=2, sequence_parallel=sp)
    return _train_rnn(Mesh(par), par, la)


@pytest.mark.parametrize("la,sp", [("hgrn2", False), ("rwkv6", False), ("rwkv7", False),
                                   ("hgrn2", True), ("rwkv6", True), ("rwkv7", True)])
def test_linear_rnn_mixers_under_tensor_parallelism(la, sp):
    """HGRN2 / RWKV6 / RWKV7 with their heads split over two tensor-parallel ranks train like the single-process model
    (sharded projections, sliced per-head vectors, replicated low-rank mixers with completed gradients), with and without
    sequence parallelism (input gathered along T at the mixer's entry, output reduce-scattered)."""
    ref_losses, ref_gn = _train_rnn(single_process_mesh(), ParallelConfig(), la)
    outs = run_distributed(_worker_rnn, 2, la=la, sp=sp)
    losses, gn = outs[0]
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=2e-4), (losses, ref_losses)
    # the first step pins the gradients (fp32 reduction order only); Adam's first updates then amplify rounding noise
    assert abs(gn[0] - ref_gn[0]) < 5e-4 * ref_gn[0], (gn, ref_gn)
    assert torch.allclose(torch.tensor(gn), torch.tensor(ref_gn), rtol=2e-2), (gn, ref_gn)


def _worker_rnn_cp(rank, world, la):
    par = ParallelConfig(distributed_backend="gloo", context_parallel_size=2)
    return _train_rnn(Mesh(par), par, la)


@pytest.mark.parametrize("la", ["hgrn2", "rwkv6", "rwkv7"])
def test_linear_rnn_mixers_under_context_parallelism(la):
    """The same mixers with the sequence split over two ranks (token-shift halo from the rank before, LASP-2 exchange of
    the state summaries; RWKV7's transition is a matrix per head) train like the single-process model."""
    ref_losses, ref_gn = _train_rnn(single_process_mesh(), ParallelConfig(), la)
    outs = run_distributed(_worker_rnn_cp, 2, la=la)
    losses, gn = outs[0]
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=3e-4), (losses, ref_losses)
    assert abs(gn[0] - ref_gn[0]) < 1e-3 * ref_gn[0], (gn, ref_gn)


def _reduced_grads(mesh, par, kw, mbs=2):
    cfg = get_preset("bench-cpu-plumbing", **kw)
    tc = TrainConfig(micro_batch_size=mbs, global_batch_size=2, seq_length=64, train_iters=1, lr=1e-3, min_lr=1e-3,
                     lr_decay_style="constant", weight_decay=0.0, clip_grad=0.0, log_interval=1000, seed=0)
    ds = SyntheticTokenDataset(cfg.vocab_size, 64, num_samples=2, seed=0)
    tr = Trainer(cfg, par, tc, mesh, device=torch.device("cpu"), dataset=ds)
    for m in tr.models:
        m.train()
    tr.optimizer.zero_grad()
    tr._run_schedule()
    tr.optimizer.reduce_grads()
    return {n: (p.main_grad.clone().float(), bool(getattr(p, "tensor_parallel", False))) for n, p in tr.optimizer.named}


def _worker_reduced_grads(rank, world, kw, sp):
    par = ParallelConfig(distributed_backend="gloo", tensor_model_parallel_size=2, sequence_parallel=sp)
    return _reduced_grads(Mesh(par), par, kw)


_TP_GRAD_CASES = {
    "lightning": (dict(la_module="lightning_attention"), True),
    "retention_t2r": (dict(la_module="retention", la_feature_map="t2r"), True),
    "gla_groupnorm": (dict(la_module="gla", la_feature_map=None, la_output_norm="groupnorm"), True),
    "rebased": (dict(la_module="rebased", la_feature_map=None, kv_channels=16), True),
    "mom_gla": (dict(la_module="mom_gla", la_feature_map=None), True),
    "mom_gdn_nosp": (dict(la_module="mom_gated_deltanet", la_feature_map=None, num_experts=None, ffn_hidden_size=256), False),
    "attn_qk_layernorm": (dict(layer_type_list="NN", qk_layernorm=True), True),
    "mla": (dict(base_model="deepseek_v2", kv_lora_rank=32, q_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8,
                 v_head_dim=16, layer_type_list="NN", use_la_module=False), True),
    "mla_nosp": (dict(base_model="deepseek_v2", kv_lora_rank=32, q_lora_rank=None, qk_nope_head_dim=16, qk_rope_head_dim=8,
                      v_head_dim=16, layer_type_list="NN", use_la_module=False, num_experts=None, ffn_hidden_size=256), False),
}


@pytest.mark.parametrize("case", list(_TP_GRAD_CASES))
def test_replicated_parameter_gradients_under_tensor_parallelism(case):
    """After the gradient reduction, every parameter that is replicated over the tensor-parallel ranks holds, on both
    ranks, the gradient of the single-process model: parameters shared by all heads but applied to the rank's own heads
    (per-head output norms, q / k layer norms, learnable feature maps, MoM routing weights, MLA's shared rope key and
    replicated down-projections) get their partial gradients summed, and nothing is summed twice."""
    kw, sp = _TP_GRAD_CASES[case]
    ref = _reduced_grads(single_process_mesh(), ParallelConfig(), kw)
    outs = run_distributed(_worker_reduced_grads, 2, kw=kw, sp=sp)
    checked, bad = 0, []
    for n, (g0, sharded) in outs[0].items():
        g1, r = outs[1][n][0], ref[n][0]
        if sharded:
            assert g0.numel() * 2 == r.numel() or g0.shape != r.shape or r.dim() == 0, n
            continue
        assert g0.shape == r.shape, (n, g0.shape, r.shape)          # a sliced parameter that is not marked tensor_parallel
        if r.norm() < 1e-9:
            continue
        checked += 1
        e = max(((g - r).norm() / r.norm()).item() for g in (g0, g1))
        if e > 5e-3:
            bad.append((n, round(e, 4)))
    assert checked > 3 and not bad, bad


def _worker_cp_grads(rank, world, kw):
    par = ParallelConfig(distributed_backend="gloo", context_parallel_size=2)
    return _reduced_grads(Mesh(par), par, kw)


@pytest.mark.parametrize("case", ["gsa", "rwkv7", "mla", "based", "linear_attention_norm", "deltanet_conv", "mom_gla",
                                  "mom_gated_deltanet"])
def test_gradients_under_context_parallelism(case):
    """Every parameter's reduced gradient with the sequence split over two ranks equals the single-process gradient:
    gated slot attention (value-gated first pass + key-gated second pass through LASP-2), RWKV7 (matrix transition),
    MLA (gathered keys / values with rope offsets), Based and normalised linear attention (feature maps, normaliser
    column), DeltaNet with the short convolution's halo."""
    kw = {
        "gsa": dict(la_module="gsa", la_feature_map=None),
        "rwkv7": dict(la_module="rwkv7", la_feature_map=None),
        "mla": _TP_GRAD_CASES["mla"][0],
        "based": dict(la_module="based", la_feature_map=None, kv_channels=16),
        "linear_attention_norm": dict(la_module="linear_attention", la_feature_map="elu", la_do_feature_map_norm=True),
        "deltanet_conv": dict(la_module="deltanet", la_feature_map=None, use_short_conv=True),
        # mixture of memories: every memory's sub-sequence is carried across the ranks by LASP-2; the capacity is per
        # rank slice, so the comparison uses one that drops no token
        "mom_gla": dict(la_module="mom_gla", la_feature_map=None, mom_capacity=4.0),
        "mom_gated_deltanet": dict(la_module="mom_gated_deltanet", la_feature_map=None, mom_capacity=4.0),
    }[case]
    ref = _reduced_grads(single_process_mesh(), ParallelConfig(), kw)
    outs = run_distributed(_worker_cp_grads, 2, kw=kw)
    bad = []
    for n, (g0, _) in outs[0].items():
        r = ref[n][0]
        assert g0.shape == r.shape, n
        if r.norm() < 1e-9:
            continue
        e = max(((o[n][0] - r).norm() / r.norm()).item() for o in outs)
        if e > 5e-3:
            bad.append((n, round(e, 4)))
    assert not bad, bad


@pytest.mark.parametrize("kw", [
    dict(la_module="rwkv6", la_feature_map=None), dict(la_module="rwkv7", la_feature_map=None),
    dict(la_module="retention", la_feature_map="t2r"), dict(la_module="linear_attention", la_feature_map="elementwise_product"),
    dict(la_module="linear_attention", la_feature_map="polysketch"), dict(la_module="gla", la_feature_map="learnable_outer_product"),
    dict(la_module="mom_gla", la_feature_map=None), dict(la_module="gsa", la_feature_map=None),
    dict(la_module="mamba2", la_feature_map=None, hybrid_override_pattern="M-", num_layers=2, mamba_head_dim=16, mamba_d_state=16),
    dict(base_model="deepseek_v2", kv_lora_rank=32, q_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
         layer_type_list="NN", use_la_module=False),
], ids=lambda kw: kw.get("la_module", "mla") + "-" + str(kw.get("la_feature_map")))
def test_initial_weights_do_not_depend_on_the_global_generator(kw):
    """The trainer seeds the process-global generator differently on every data- and context-parallel rank (dropout), so
    a parameter drawn from it would differ between replicas: two builds under different global seeds must be equal."""
    from linear_moe_b200.models.transformer import CausalLM
    cfg = get_preset("bench-cpu-plumbing", **kw)
    torch.manual_seed(1)
    a = CausalLM(cfg).state_dict()
    torch.manual_seed(2)
    b = CausalLM(cfg).state_dict()
    diff = [n for n in a if not torch.equal(a[n], b[n])]
    assert not diff, diff


def test_bench_config_layouts():
    """``bench.py --config`` maps every benchmark configuration to a parallel layout that exists on 1, 2, 4 and 8 GPUs, and
    the headline configuration keeps 16384 tokens per GPU."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("lmoe_bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.config.presets import get_preset
    for name in bench.LAYOUTS:
        cfg = get_preset(name)
        for world in (1, 2, 4, 8):
            layout, pkw, seq, mbs, gbs, label = bench.resolve_layout(name, world)
            par = ParallelConfig(distributed_backend="gloo", **pkw)
            tp, ep, cp = par.tensor_model_parallel_size, par.expert_model_parallel_size, par.context_parallel_size
            assert world % (tp * cp) == 0 and (world // tp) % ep == 0, (name, world, label)
            dp = world // (tp * cp)
            assert gbs == mbs * dp and gbs * seq > 0
            if cfg.num_experts:
                assert cfg.num_experts % ep == 0
            if name == "bench-lasp2-llama3-1b":
                assert seq == 16384 * world and gbs == 1 and cp == world
    assert bench.resolve_layout("bench-a1b-7b-hybrid", 8)[5] == "tp2 ep4 dp4"


def test_workspace_guard_region_check():
    """``verify_canaries`` reports a workspace whose guard region lost its byte pattern (an overrun by a peer or a kernel)."""
    import pytest
    import torch
    from linear_moe_b200.parallel import fused_comm as fc
    saved = list(fc._CANARIES)
    try:
        fc._CANARIES.clear()
        numel = 100
        t = torch.zeros(numel + fc._CANARY_ELEMS, dtype=torch.float32)
        t[numel:].view(torch.uint8).fill_(fc._CANARY_BYTE)
        fc._CANARIES.append(("test:float32:100", t, numel))
        fc.verify_canaries()                                  # intact
        t[:numel].fill_(7.0)                                  # writes inside the workspace are fine
        fc.verify_canaries()
        t[numel + 3] = 1.0                                    # one element past the logical end
        with pytest.raises(RuntimeError, match="test:float32:100"):
            fc.verify_canaries()
    finally:
        fc._CANARIES[:] = saved


def test_memory_estimate_knows_the_expert_data_parallel_size():
    """Weights + optimizer estimate: the distributed optimizer shards dense state over the data-parallel ranks but expert
    state only over the expert-data-parallel ranks (none when EP uses up the data-parallel size)."""
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.config.presets import get_preset
    from linear_moe_b200.utils.memory import analytic_parameter_counts, compute_weight_and_optimizer_memory as est
    cfg = get_preset("bench-mixtral-mamba2-fp8")
    c = analytic_parameter_counts(cfg)
    par = ParallelConfig(tensor_model_parallel_size=2, expert_model_parallel_size=4, use_distributed_optimizer=True)
    got = est(cfg, par, world_size=8)                        # dp = 4, ep = 4 -> every expert shard lives on one rank only
    experts = c["experts"] / 4 / 2
    assert got > experts * 18.0                              # expert state is not sharded at all
    par16 = ParallelConfig(tensor_model_parallel_size=2, expert_model_parallel_size=4, use_distributed_optimizer=True)
    assert est(cfg, par16, world_size=16) < got              # twice the data-parallel size: expert state halves
    no_zero = ParallelConfig(tensor_model_parallel_size=2, expert_model_parallel_size=4)
    assert est(cfg, no_zero, world_size=8) > got


def test_direct_weight_gradient_accumulators_skip_the_zero_fill():
    """Weights whose gradient GEMM writes its fp32 accumulator directly are not cleared by ``zero_grad``; the three guards
    around that: (1) other accumulators are still cleared, (2) an ordinary autograd gradient arriving for such a weight
    clears the stale accumulator before adding, (3) a direct weight that saw no gradient in a step is cleared before the
    reduction."""
    import torch
    import torch.nn as nn
    from linear_moe_b200.config.model_config import TrainConfig
    from linear_moe_b200.dist.mesh import single_process_mesh
    from linear_moe_b200.train.optimizer import MixedPrecisionAdam
    torch.manual_seed(0)
    model = nn.ModuleList([nn.Sequential(nn.Linear(8, 16, bias=False), nn.Linear(16, 8, bias=False))])
    tc = TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=8, train_iters=4, lr=1e-2, min_lr=1e-2,
                     lr_decay_style="constant", clip_grad=0.0, weight_decay=0.0)
    opt = MixedPrecisionAdam(model, single_process_mesh(), tc)
    w0, w1 = model[0][0].weight, model[0][1].weight
    opt.zero_grad()
    # step 1: w0's gradient is written directly (what the weight-gradient GEMM does), w1's arrives through autograd
    assert w0._main_grad_fresh
    w0.main_grad.copy_(torch.full_like(w0.main_grad, 3.0))
    w0._main_grad_fresh, w0._direct_wgrad = False, True
    w1.grad = torch.ones_like(w1)
    opt._accumulate(w1)
    assert torch.all(w1.main_grad == 1.0)
    opt.zero_grad()
    assert torch.all(w0.main_grad == 3.0), "a direct weight's accumulator is cleared lazily"           # (skipped)
    assert torch.all(w1.main_grad == 0.0)                                                               # (1)
    # step 2: this time w0's gradient comes through autograd: the stale 3.0 must not be added to
    w0.grad = torch.full_like(w0, 2.0)
    opt._accumulate(w0)
    assert torch.all(w0.main_grad == 2.0)                                                               # (2)
    opt.zero_grad()
    # step 3: w0 gets no gradient at all: the reduction must not see step 2's values
    opt.reduce_grads()
    assert torch.all(w0.main_grad == 0.0)                                                               # (3)


def test_fp16_dynamic_loss_scale_skips_and_recovers():
    """fp16 training with the dynamic scaler: a scale that overflows the gradients skips the update (parameters and
    Adam state untouched, the step counted as skipped), halves after ``hysteresis`` overflows, and doubles again after
    ``loss_scale_window`` clean steps (training.py:390-417 semantics of skipped iterations)."""
    cfg = get_preset("bench-cpu-plumbing", num_experts=None, ffn_hidden_size=128, num_layers=1, layer_type_list="L",
                     params_dtype=torch.float16)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=32, train_iters=50, lr=1e-3, min_lr=1e-3,
                     lr_decay_style="constant", weight_decay=0.0, clip_grad=1.0, log_interval=1000, seed=0, fp16=True,
                     initial_loss_scale=2.0 ** 28, loss_scale_window=3, hysteresis=2, min_loss_scale=1.0)
    ds = SyntheticTokenDataset(cfg.vocab_size, 32, num_samples=4, seed=0)
    tr = Trainer(cfg, ParallelConfig(), tc, single_process_mesh(), device=torch.device("cpu"), dataset=ds)
    opt = tr.optimizer
    assert opt.dynamic_scale and opt.loss_scale == 2.0 ** 28
    scales, skipped = [], []
    for _ in range(30):
        before = [p.detach().clone() for _, p in opt.named]
        steps_before = opt.step_count
        st = tr.train_step()
        scales.append(opt.loss_scale)
        skipped.append(st["skipped"])
        moved = any(not torch.equal(a, p.detach()) for a, (_, p) in zip(before, opt.named))
        assert moved == (not st["skipped"]), "a skipped step must leave the weights alone, a clean step must move them"
        assert opt.step_count == steps_before + (0 if st["skipped"] else 1)
    assert skipped[0] == 1 and skipped[1] == 1                 # 2^28 overflows fp16 gradients
    # the scaler's rule, replayed on the observed overflow pattern
    scale, hyst, clean, want = 2.0 ** 28, 2, 0, []
    for sk in skipped:
        if sk:
            clean, hyst = 0, hyst - 1
            if hyst <= 0:
                scale = max(scale / 2.0, 1.0)
        else:
            clean += 1
            if clean >= 3:
                clean, hyst, scale = 0, 2, scale * 2.0
        want.append(scale)
    assert scales == want, (scales, want)
    assert 0 in skipped and any(b > a for a, b in zip(scales, scales[1:])), "the scale never recovered"
    assert opt.skipped_iters == sum(skipped) and tr.iteration == 30


@pytest.mark.parametrize("kw", [
    dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=1),
    dict(recompute_granularity="full", recompute_method="block", recompute_num_layers=1),
    dict(recompute_granularity="selective"),
    dict(moe_layer_recompute=True),
], ids=["full_uniform", "full_block", "selective", "moe_layer"])
def test_activation_recompute_keeps_loss_and_gradients(kw):
    """Every activation-recompute mode (hybrid_transformer_block.py:262-300, --moe-layer-recompute) is a memory trade
    only: same loss, same gradient for every parameter, with the router's jitter and auxiliary losses in play."""
    from linear_moe_b200.models.transformer import CausalLM
    base = dict(la_module="gla", la_feature_map=None, layer_type_list="LN", moe_aux_loss_coeff=0.01, moe_z_loss_coeff=1e-3)

    from linear_moe_b200.models.moe import AuxLossTracker

    def run(extra):
        torch.manual_seed(0)
        AuxLossTracker.values = {}
        m = CausalLM(get_preset("bench-cpu-plumbing", **base, **extra)).train()
        ids = torch.randint(0, 512, (2, 48), generator=torch.Generator().manual_seed(1))
        loss = m(ids, torch.roll(ids, -1, 1)).mean()
        loss.backward()
        logged = {k: v.tolist() for k, v in AuxLossTracker.pop().items()}
        return loss.item(), {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}, logged

    l0, g0, a0 = run({})
    l1, g1, a1 = run(kw)
    assert abs(l0 - l1) < 1e-6 and set(g0) == set(g1)
    assert a0 == a1 and a0["load_balancing_loss"][0] > 0, "the replayed forward pass must not be logged twice"
    for n in g0:
        assert torch.allclose(g0[n], g1[n], rtol=1e-4, atol=1e-6), n


def test_hidden_dropout_acts_in_training_only_and_attention_dropout_is_refused():
    from linear_moe_b200.config.model_config import ModelConfig
    from linear_moe_b200.models.transformer import CausalLM
    kw = dict(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, vocab_size=256)
    ids = torch.randint(0, 256, (2, 32), generator=torch.Generator().manual_seed(0))
    plain, drop = CausalLM(ModelConfig(**kw)), CausalLM(ModelConfig(hidden_dropout=0.2, **kw))
    drop.load_state_dict(plain.state_dict())
    with torch.no_grad():
        assert torch.equal(plain.eval()(ids), drop.eval()(ids))                  # evaluation: no dropout
        torch.manual_seed(1)
        a = drop.train()(ids)
        torch.manual_seed(1)
        b = drop(ids)
        torch.manual_seed(2)
        c = drop(ids)
    assert torch.equal(a, b) and not torch.equal(a, c) and not torch.allclose(a, plain.train()(ids), atol=1e-3)
    # full recompute replays the same masks: gradients equal those without recompute
    re = CausalLM(ModelConfig(hidden_dropout=0.2, recompute_granularity="full", recompute_method="uniform", **kw)).train()
    re.load_state_dict(plain.state_dict())
    grads = []
    for m in (drop.train(), re):
        m.zero_grad()
        torch.manual_seed(3)
        m(ids, torch.roll(ids, -1, 1)).mean().backward()
        grads.append([p.grad.clone() for p in m.parameters()])
    assert all(torch.allclose(x, y, rtol=1e-4, atol=1e-7) for x, y in zip(*grads))
    with pytest.raises(ValueError, match="attention-dropout"):
        ModelConfig(attention_dropout=0.1, **kw)


def test_sgd_matches_torch_sgd():
    """--optimizer sgd --sgd-momentum 0.9 with weight decay and clipping off: the flat-buffer update equals
    torch.optim.SGD on the same model and data, step for step."""
    from linear_moe_b200.config.model_config import ModelConfig
    from linear_moe_b200.models.transformer import CausalLM
    cfg = ModelConfig(num_layers=2, hidden_size=32, num_attention_heads=2, ffn_hidden_size=64, vocab_size=64)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=16, train_iters=4, lr=0.05, min_lr=0.05,
                     lr_decay_style="constant", weight_decay=0.01, clip_grad=0.0, log_interval=1000, seed=0,
                     optimizer="sgd", sgd_momentum=0.9)
    ds = SyntheticTokenDataset(cfg.vocab_size, 16, num_samples=8, seed=0)
    tr = Trainer(cfg, ParallelConfig(), tc, single_process_mesh(), device=torch.device("cpu"), dataset=ds)
    ref = CausalLM(cfg)
    ref.load_state_dict(tr.models[0].state_dict())
    decay = [p for n, p in ref.named_parameters() if p.dim() >= 2]
    plain = [p for n, p in ref.named_parameters() if p.dim() < 2]
    opt = torch.optim.SGD([{"params": decay, "weight_decay": 0.01}, {"params": plain, "weight_decay": 0.0}], lr=0.05, momentum=0.9)
    it = D_iter = iter(ds[i]["text"] for i in range(8))
    for step in range(4):
        st = tr.train_step()
        text = torch.stack([next(it), next(it)])
        opt.zero_grad()
        loss = ref.train()(text[:, :-1], text[:, 1:]).mean()
        loss.backward()
        opt.step()
        assert abs(float(st["lm loss"]) - loss.item()) < 1e-5, (step, float(st["lm loss"]), loss.item())
    a, b = tr.models[0].state_dict(), ref.state_dict()
    assert all(torch.allclose(a[k], b[k], rtol=1e-5, atol=1e-6) for k in a)


def _train_sgd(mesh, par, steps=3):
    cfg = get_preset("bench-cpu-plumbing", num_experts=None, ffn_hidden_size=128, num_layers=2, layer_type_list="LN")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=32, train_iters=steps, lr=0.02, min_lr=0.02,
                     lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, log_interval=1000, seed=0,
                     optimizer="sgd", sgd_momentum=0.9)
    ds = SyntheticTokenDataset(cfg.vocab_size, 32, num_samples=2, seed=0)
    tr = Trainer(cfg, par, tc, mesh, device=torch.device("cpu"), dataset=ds)
    out = [tr.train_step() for _ in range(steps)]
    return [float(o["lm loss"]) for o in out], [o["grad_norm"] for o in out]


def _worker_sgd(rank, world):
    par = ParallelConfig(distributed_backend="gloo", use_distributed_optimizer=True)
    return _train_sgd(Mesh(par), par)


def test_sgd_with_sharded_optimizer_state_matches_single_process():
    """SGD under ZeRO-1 on two data-parallel ranks (momentum buffers sharded, updated shards gathered) follows the
    single-process run with gradient accumulation."""
    ref_losses, ref_gn = _train_sgd(single_process_mesh(), ParallelConfig())
    losses, gn = run_distributed(_worker_sgd, 2)[0]
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=2e-4), (losses, ref_losses)
    assert torch.allclose(torch.tensor(gn), torch.tensor(ref_gn), rtol=2e-3), (gn, ref_gn)
    assert ref_losses[-1] < ref_losses[0]

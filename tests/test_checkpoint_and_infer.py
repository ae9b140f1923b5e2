"""Checkpoint layout, resharding rules, HF conversion, generation caches, datasets (all CPU)."""
import os

import numpy as np
import pytest
import torch

from linear_moe_b200.ckpt import hf_convert, legacy, reshard
from linear_moe_b200.config.model_config import ModelConfig, ParallelConfig, TrainConfig
from linear_moe_b200.dist.mesh import Mesh
from linear_moe_b200.models.transformer import CausalLM


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, vocab_size=512)
    base.update(kw)
    return ModelConfig(**base)


CASES = {
    "qwen2_moe_gqa": dict(base_model="qwen2", num_query_groups=2, add_qkv_bias=True, num_experts=4, moe_topk=2,
                          moe_ffn_hidden_size=64, enable_shared_expert=True, shared_moe_ffn_hidden_size=128),
    "hybrid_gla": dict(use_la_module=True, la_module="gla", layer_type_list="LN", num_experts=4, moe_ffn_hidden_size=64),
    "hybrid_gdn_conv": dict(use_la_module=True, la_module="gated_deltanet", layer_type_list="LN", use_short_conv=True),
    "mamba2": dict(use_la_module=True, la_module="mamba2", hybrid_override_pattern="M*", mamba_head_dim=16,
                   mamba_d_state=16, mamba_ngroups=2, base_model="mixtral", num_experts=4, moe_ffn_hidden_size=64),
    "deepseek_mla": dict(base_model="deepseek_v2", num_experts=4, moe_topk=2, moe_ffn_hidden_size=32,
                         enable_shared_expert=True, shared_moe_ffn_hidden_size=64, kv_lora_rank=32, qk_nope_head_dim=16,
                         qk_rope_head_dim=8, v_head_dim=16, q_lora_rank=24, moe_layer_freq=1),
    "rwkv6": dict(use_la_module=True, la_module="rwkv6", layer_type_list="LN"),
    "rwkv7": dict(use_la_module=True, la_module="rwkv7", layer_type_list="LL"),
    "hgrn2": dict(use_la_module=True, la_module="hgrn2", layer_type_list="LL", hgrn2_lower_bound=True),
    "gsa": dict(use_la_module=True, la_module="gsa", layer_type_list="LL"),
    "mom_gla": dict(use_la_module=True, la_module="mom_gla", layer_type_list="LL"),
    "mom_gdn": dict(use_la_module=True, la_module="mom_gated_deltanet", layer_type_list="LL"),
    "retention_t2r": dict(use_la_module=True, la_module="retention", la_feature_map="t2r", layer_type_list="LL"),
    "rebased": dict(use_la_module=True, la_module="rebased", layer_type_list="LL", kv_channels=16),
}


@pytest.mark.parametrize("name", list(CASES))
def test_reshard_rules_match_model_sharding(name):
    """A model built on TP rank r of 2 must hold exactly ``shard_state_dict(full, tp=2, tp_rank=r)``; same for EP."""
    cfg = _cfg(**CASES[name])
    full = CausalLM(cfg).state_dict()
    for tp, ep in ((2, 1), (1, 2)):
        if ep > 1 and not cfg.is_moe:
            continue
        par = ParallelConfig(tensor_model_parallel_size=tp, expert_model_parallel_size=ep)
        shards = {}
        for r in range(2):
            mesh = Mesh(par, world_size=2, rank=r, create_groups=False)
            sd = CausalLM(cfg, mesh, sequence_parallel=tp > 1).state_dict()
            t_r, e_r = (r, 0) if tp == 2 else (0, r)
            want = reshard.shard_state_dict(full, cfg, tp, 1, ep, t_r, 0, e_r)
            assert set(sd) == set(want)
            for k in sd:
                assert sd[k].shape == want[k].shape, (k, sd[k].shape, want[k].shape)
                assert torch.equal(sd[k], want[k]), k
            shards[(t_r, 0, e_r)] = sd
        merged = reshard.merge_state_dicts(shards, cfg, tp, 1, ep)
        for k in full:
            assert torch.equal(merged[k], full[k]), k


def test_pipeline_split_and_reshard_roundtrip():
    cfg = _cfg(num_layers=4, use_la_module=True, la_module="retention", layer_type_list="LLNL")
    full = CausalLM(cfg).state_dict()
    shards = {(t, p, 0): reshard.shard_state_dict(full, cfg, 2, 2, 1, t, p, 0) for t in range(2) for p in range(2)}
    assert "embedding.word_embeddings.weight" not in shards[(0, 1, 0)]
    assert "output_layer.weight" not in shards[(0, 0, 0)]
    again = reshard.reshard(shards, cfg, (2, 2, 1), (1, 4, 1))
    back = reshard.merge_state_dicts(again, cfg, 1, 4, 1)
    assert all(torch.equal(back[k], full[k]) for k in full)


@pytest.mark.parametrize("name", ["qwen2_moe_gqa", "deepseek_mla"])
def test_hf_roundtrip(name):
    cfg = _cfg(**CASES[name])
    sd = {k: v for k, v in CausalLM(cfg).state_dict().items()}
    hf = hf_convert.mcore_to_hf(sd, cfg)
    assert "model.layers.0.self_attn.o_proj.weight" in hf
    back = hf_convert.hf_to_mcore(hf, cfg)
    assert set(back) == set(sd)
    assert all(torch.equal(back[k], sd[k]) for k in sd)


def test_qkv_packing_is_group_major():
    H, G, hd, h = 4, 2, 3, 5
    q, k, v = torch.randn(H * hd, h), torch.randn(G * hd, h), torch.randn(G * hd, h)
    w = hf_convert.pack_qkv(q, k, v, G, hd)
    assert torch.equal(w[: 2 * hd], q[: 2 * hd]) and torch.equal(w[2 * hd:3 * hd], k[:hd])
    q2, k2, v2 = hf_convert.unpack_qkv(w, H, G, hd)
    assert torch.equal(q2, q) and torch.equal(k2, k) and torch.equal(v2, v)


def test_legacy_checkpoint_roundtrip(tmp_path):
    from linear_moe_b200.train.loop import Trainer
    cfg = _cfg(use_la_module=True, la_module="gla", layer_type_list="LN", num_experts=4, moe_ffn_hidden_size=64)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100,
                     save=str(tmp_path), lr=1e-3)
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    for _ in range(2):
        tr.train_step()
    tr.save()
    assert open(tmp_path / legacy.TRACKER).read() == "2"
    path = legacy.checkpoint_name(str(tmp_path), 2, False, 0, 0, 0, 1, 1)
    assert path.endswith("iter_0000002/mp_rank_00/model_optim_rng.pt")
    ck = torch.load(path, weights_only=False)
    assert ck["checkpoint_version"] == 3.0 and ck["iteration"] == 2
    keys = set(ck["model"])
    assert "decoder.layers.0.mlp.experts.local_experts.3.linear_fc1.weight" in keys
    assert "decoder.layers.0.self_attention.gk_proj.gk_proj.1.bias" in keys
    assert "embedding.word_embeddings.weight" in keys and "decoder.final_layernorm.weight" in keys
    tc2 = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100,
                      load=str(tmp_path), lr=1e-3)
    tr2 = Trainer(cfg, ParallelConfig(), tc2, device=torch.device("cpu"))
    assert tr2.iteration == 2
    a, b = tr.model.state_dict(), tr2.model.state_dict()
    assert all(torch.equal(a[k], b[k]) for k in a)
    s1, s2 = tr.train_step(), tr2.train_step()
    assert abs(float(s1["lm loss"]) - float(s2["lm loss"])) < 1e-5      # optimizer + data position restored


def test_zero1_optimizer_reshard():
    states = []
    for r in range(2):
        n = 256
        states.append({"step": 3, "loss_scale": None, "zero1": True, "buffers": [{
            "expert": False, "weight_decay": True, "shard": (r * n, (r + 1) * n), "numel": 512, "names": ["w"],
            "master": torch.arange(r * n, (r + 1) * n, dtype=torch.float32), "exp_avg": torch.ones(n) * r,
            "exp_avg_sq": torch.zeros(n)}]})
    new = reshard.reshard_optimizer_shards(states, 4)
    assert len(new) == 4 and new[3]["buffers"][0]["shard"] == (384, 512)
    assert torch.equal(torch.cat([s["buffers"][0]["master"] for s in new]), torch.arange(512, dtype=torch.float32))


@pytest.mark.parametrize("la", [None, "lightning_attention", "gla", "gated_deltanet", "hgrn2", "rwkv6", "mamba2",
                                "retention", "deltanet", "rwkv7", "gsa", "based", "rebased", "linear_attention_norm",
                                "mom_gla", "mom_gated_deltanet", "mla"])
def test_incremental_decoding_matches_full_forward(la):
    """Prefill + token-by-token decoding with the recurrent / KV caches gives the logits of one full forward."""
    torch.manual_seed(0)
    kw = dict(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, vocab_size=128, init_method_std=0.1)
    if la == "mamba2":
        kw.update(use_la_module=True, la_module=la, hybrid_override_pattern="M*", mamba_head_dim=16, mamba_d_state=16,
                  mamba_ngroups=2)
    elif la == "mla":
        kw.update(base_model="deepseek_v2", kv_lora_rank=32, q_lora_rank=24, qk_nope_head_dim=16, qk_rope_head_dim=8,
                  v_head_dim=16)
    elif la == "linear_attention_norm":
        kw.update(use_la_module=True, la_module="linear_attention", layer_type_list="LN", la_do_feature_map_norm=True)
    elif la in ("based", "rebased"):
        kw.update(use_la_module=True, la_module=la, layer_type_list="LN", kv_channels=8)
    elif la is not None:
        kw.update(use_la_module=True, la_module=la, layer_type_list="LN", use_short_conv=la == "gated_deltanet")
        if la.startswith("mom_"):
            kw.update(mom_capacity=float(kw.get("mom_num_memories", 4)))    # no token is dropped in the full forward either
    model = CausalLM(ModelConfig(**kw)).eval()
    ids = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        full = model(ids)
        caches = model.new_cache()
        parts = [model(ids[:, :5], caches=caches, position_offset=0)]
        for t in range(5, 12):
            parts.append(model(ids[:, t:t + 1], caches=caches, position_offset=t))
        inc = torch.cat(parts, dim=1)
    assert torch.allclose(full, inc, atol=2e-4, rtol=1e-3), (full - inc).abs().max()


def test_generation_api():
    from linear_moe_b200.data.tokenizer import NullTokenizer
    from linear_moe_b200.infer import generation as G
    torch.manual_seed(0)
    model = CausalLM(_cfg(vocab_size=64, use_la_module=True, la_module="retention", layer_type_list="LN")).eval()
    tok = NullTokenizer(64)
    texts, toks, lp = G.generate_and_post_process(model, tok, ["1 2 3", "4 5"], tokens_to_generate=6, top_k_sampling=1,
                                                  return_output_log_probs=True, use_eod_token_for_early_termination=False)
    assert len(toks[0]) == 9 and toks[0][:3] == [1, 2, 3] and toks[1][:2] == [4, 5]
    # greedy continuation equals argmax of a full forward on the generated prefix
    seq = torch.tensor([toks[1]])
    with torch.no_grad():
        nxt = model(seq[:, :-1])[0, -1].argmax().item()
    assert nxt == toks[1][-1]
    assert lp.shape == (2, 8) and torch.isfinite(lp).all()
    out, scores = G.beam_search(model, torch.tensor([[1, 2, 3]]), beam_size=3, max_new_tokens=4, eod=63)
    assert out.shape[0] == 1 and out[0, :3].tolist() == [1, 2, 3]
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0]])
    assert G.sample(logits, top_k=1).item() == 3
    assert set(G.modify_logits_for_top_k(logits, 2)[0].isinf().tolist()) == {True, False}
    assert G.modify_logits_for_top_p(logits, 0.5)[0, 0].isinf()


def test_indexed_dataset_and_index_builder(tmp_path):
    from linear_moe_b200.data import datasets as D
    from linear_moe_b200.utils import hostlib
    rng = np.random.RandomState(0)
    docs = [rng.randint(0, 1000, size=rng.randint(5, 40)).astype(np.int32) for _ in range(50)]
    prefix = str(tmp_path / "corpus")
    D.IndexedDataset.write(prefix, docs)
    ds = D.IndexedDataset(prefix)
    assert len(ds) == 50 and np.array_equal(ds.get(7), docs[7]) and np.array_equal(ds.get(7, 2, 3), docs[7][2:5])
    g = D.GPTDataset(ds, seq_length=16, num_samples=40, seed=1)
    flat = np.concatenate([docs[i] for i in g.doc_idx])
    for i in range(10):
        s = g.shuffle_idx[i]
        want = flat[s * 16: s * 16 + 17]
        assert np.array_equal(g[i]["text"].numpy(), want)
    lib = hostlib.load()
    if lib is not None:     # C++ builder equals the numpy definition
        sizes, doc_idx = np.asarray(ds.sizes), g.doc_idx
        a = hostlib.build_sample_idx(lib, sizes, doc_idx, 16, 30)
        hostlib._LIB, keep = None, hostlib._LIB
        hostlib._TRIED = True
        b = D.build_sample_idx(sizes, doc_idx, 16, 1, 16 * 30 + 1)
        hostlib._LIB = keep
        assert np.array_equal(a, b[: len(a)])
    batch = D.make_batch({"text": torch.arange(18)[None]}, eod_token=5, eod_mask_loss=True)
    assert batch["tokens"].shape == (1, 17) and batch["labels"][0, 5] == -100 and batch["loss_mask"][0, 5] == 0


def test_resume_keeps_fp32_masters_bitwise(tmp_path):
    """A full resume of a bf16 model restores the fp32 master weights exactly: re-deriving them from the bf16
    parameters would drop their low bits (the reference reloads masters only on the pretrained-checkpoint path)."""
    from linear_moe_b200.train.loop import Trainer
    cfg = _cfg(use_la_module=True, la_module="retention", layer_type_list="LN", params_dtype=torch.bfloat16)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100,
                     save=str(tmp_path), lr=1e-2, bf16=True)
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    for _ in range(2):
        tr.train_step()
    tr.save()
    masters = [b.master.clone() for b in tr.optimizer.buffers]
    assert any((m != m.bfloat16().float()).any() for m in masters), "masters must carry bits below bf16 for this test"
    tc2 = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100,
                      load=str(tmp_path), lr=1e-2, bf16=True)
    tr2 = Trainer(cfg, ParallelConfig(), tc2, device=torch.device("cpu"))
    for m, b in zip(masters, tr2.optimizer.buffers):
        assert torch.equal(m, b.master)
    # weights only: masters are derived from the parameters
    tc3 = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100,
                      load=str(tmp_path), lr=1e-2, bf16=True, no_load_optim=True)
    tr3 = Trainer(cfg, ParallelConfig(), tc3, device=torch.device("cpu"))
    for b in tr3.optimizer.buffers:
        assert torch.equal(b.master, b.shard_view(b.params).float())


def test_async_save_publishes_tracker_after_writers(tmp_path):
    """With --async-save the tracker file appears only once the writer threads have been joined (finalize)."""
    from linear_moe_b200.train.loop import Trainer
    cfg = _cfg(use_la_module=True, la_module="retention", layer_type_list="LN")
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100,
                     save=str(tmp_path), lr=1e-3, async_save=True)
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    tr.train_step()
    tr.save()
    assert legacy._PENDING_TRACKERS and not (tmp_path / legacy.TRACKER).exists()
    legacy.finalize_async_saves()
    assert open(tmp_path / legacy.TRACKER).read() == "1"
    assert (tmp_path / "iter_0000001" / "mp_rank_00" / "model_optim_rng.pt").exists()
    tr.train_step()
    tr.save()                                    # finalizes nothing pending, defers its own tracker again
    tr.save()                                    # the second save first publishes the first one's tracker
    assert open(tmp_path / legacy.TRACKER).read() == "2"
    legacy.finalize_async_saves()


def test_reference_te_style_norm_keys_are_mapped():
    sd = {"decoder.layers.0.self_attention.linear_qkv.layer_norm_weight": torch.ones(4),
          "decoder.layers.0.mlp.linear_fc1.layer_norm_weight": torch.zeros(4),
          "decoder.layers.0.mlp.linear_fc1.weight": torch.zeros(8, 4),
          "decoder.layers.0.mlp.linear_fc1._extra_state": None}
    out = legacy.from_reference_keys(sd)
    assert set(out) == {"decoder.layers.0.input_layernorm.weight", "decoder.layers.0.pre_mlp_layernorm.weight",
                        "decoder.layers.0.mlp.linear_fc1.weight"}


@pytest.mark.parametrize("name", ["qwen2_moe_gqa", "mamba2", "rwkv6", "rwkv7", "mom_gla"])
def test_sharded_checkpoint_reshard_on_load(tmp_path, name):
    """Sharded format: shards written under one (TP, PP, EP) layout are read under other layouts, every reader getting
    exactly its part of every tensor (no full merge)."""
    import json
    from types import SimpleNamespace
    from linear_moe_b200.ckpt import sharded
    if name not in CASES:
        pytest.skip(f"no case {name}")
    cfg = _cfg(**CASES[name])
    full = {k: v for k, v in CausalLM(cfg).state_dict().items() if not k.endswith("_extra_state")}
    src = (2, 2, 2) if cfg.is_moe else (2, 2, 1)
    tp, pp, ep = src
    n_layers = reshard.num_layer_entries(full)
    root = str(tmp_path)
    os.makedirs(os.path.join(root, "iter_0000007"), exist_ok=True)
    for t in range(tp):
        for p in range(pp):
            for e in range(ep):
                sd = reshard.shard_state_dict(full, cfg, tp, pp, ep, t, p, e)
                tensors, meta = sharded.describe(sd, cfg, tp, ep, t, e, layer_offset=p * (n_layers // pp))
                torch.save(tensors, sharded._shard_file(root, 7, t, p, e, "pt"))
                json.dump(meta, open(sharded._shard_file(root, 7, t, p, e, "json"), "w"))
    json.dump({"iteration": 7, "tp": tp, "pp": pp, "ep": ep, "step": None}, open(os.path.join(root, "iter_0000007", "metadata.json"), "w"))
    open(os.path.join(root, sharded.TRACKER), "w").write("7")
    rd = sharded.ShardReader(root)
    for dst in [(1, 1, 1), (4, 1, 1), (1, 2, 2 if cfg.is_moe else 1), (2, 1, 4 if cfg.is_moe else 1)]:
        t2, p2, e2 = dst
        if cfg.is_moe and cfg.num_experts % e2:
            continue
        for t in range(t2):
            for p in range(p2):
                for e in range(e2):
                    want_sd = reshard.shard_state_dict(full, cfg, t2, p2, e2, t, p, e)
                    off = p * (n_layers // p2)
                    for k, v in want_sd.items():
                        g = sharded._global_name(k, off)
                        gshape = sharded._global_shape(g, v.shape, cfg, t2, e2)
                        assert list(gshape) == list(full[g].shape), (g, gshape, full[g].shape)
                        got = rd.read(g, sharded.index_map(g, gshape, cfg, t2, e2, t, e), v.shape)
                        assert torch.equal(got, v), (dst, k)


def test_sharded_checkpoint_trainer_roundtrip_with_optimizer(tmp_path):
    """save_sharded / load_sharded through a Trainer: weights, fp32 masters and Adam moments come back bit for bit."""
    from linear_moe_b200.ckpt import sharded
    from linear_moe_b200.train.loop import Trainer
    cfg = _cfg(use_la_module=True, la_module="gla", layer_type_list="LN", num_experts=4, moe_ffn_hidden_size=64,
               params_dtype=torch.bfloat16)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100, lr=1e-2, bf16=True)
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    for _ in range(2):
        tr.train_step()
    sharded.save_sharded(str(tmp_path), tr.iteration, tr.models, cfg, tr.mesh, tr.optimizer)
    tr2 = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    it = sharded.load_sharded(str(tmp_path), tr2.models, cfg, tr2.mesh, tr2.optimizer)
    assert it == 2 and tr2.optimizer.step_count == tr.optimizer.step_count
    a, b = tr.model.state_dict(), tr2.model.state_dict()
    assert all(torch.equal(a[k], b[k]) for k in a if torch.is_tensor(a[k]))
    for x, y in zip(tr.optimizer.buffers, tr2.optimizer.buffers):
        for kind in ("master", "exp_avg", "exp_avg_sq"):
            u, v = getattr(x, kind), getattr(y, kind)
            used = max(s.start + s.numel for s in x.slots)
            assert torch.equal(u[:used], v[:used]), kind


def test_use_dist_ckpt_flag_resumes_training(tmp_path):
    """--use-dist-ckpt: Trainer.save / Trainer(load=...) go through the sharded format and the resumed run continues
    with the same loss as the original."""
    from linear_moe_b200.train.loop import Trainer
    cfg = _cfg(use_la_module=True, la_module="retention", layer_type_list="LN")
    kw = dict(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, log_interval=100, lr=1e-3, use_dist_ckpt=True)
    tr = Trainer(cfg, ParallelConfig(), TrainConfig(save=str(tmp_path), **kw), device=torch.device("cpu"))
    for _ in range(2):
        tr.train_step()
    tr.save()
    assert (tmp_path / "latest_sharded_iteration.txt").read_text() == "2"
    tr2 = Trainer(cfg, ParallelConfig(), TrainConfig(load=str(tmp_path), **kw), device=torch.device("cpu"))
    assert tr2.iteration == 2 and tr2.consumed_samples == tr.consumed_samples
    s1, s2 = tr.train_step(), tr2.train_step()
    assert abs(float(s1["lm loss"]) - float(s2["lm loss"])) < 1e-5


def _generate_worker(rank, world, par_kw):
    from linear_moe_b200.infer import generation as G
    from linear_moe_b200.infer.lm_eval_adaptor import EvalHarnessAdaptor
    par = ParallelConfig(distributed_backend="gloo", **par_kw)
    mesh = Mesh(par) if world > 1 else None
    return _generate(mesh)


def _generate(mesh):
    from linear_moe_b200.infer import generation as G
    from linear_moe_b200.infer.lm_eval_adaptor import EvalHarnessAdaptor
    from linear_moe_b200.models.transformer import CausalLM
    cfg = _cfg(num_layers=4, use_la_module=True, la_module="gla", layer_type_list="LNLN", num_query_groups=2)
    if mesh is not None and mesh.pp > 1:
        model = CausalLM(cfg, mesh, pre_process=mesh.is_first_stage, post_process=mesh.is_last_stage)
    else:
        model = CausalLM(cfg, mesh)
    torch.manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (2, 24))
    tokens = torch.cat([prompts[:, :10], torch.zeros(2, 14, dtype=torch.long)], 1)
    toks, _, lp = G.generate_tokens(model, tokens.clone(), torch.tensor([6, 10]), top_k=1, return_log_probs=True)
    scores = G.score_tokens(model, prompts)

    class Tok:
        eod = 0

        def encode(self, s):
            return [int(x) for x in s.split()]

        def decode(self, t):
            return " ".join(str(x) for x in t)
    ad = EvalHarnessAdaptor(model, Tok(), max_length=64)
    ll = ad.loglikelihood([("1 2 3 4 5", "6 7 8"), ("9 8 7", "6 5")])
    return toks, lp, scores, ll


@pytest.mark.parametrize("par_kw", [dict(pipeline_model_parallel_size=2), dict(tensor_model_parallel_size=2)])
def test_generation_and_eval_across_pipeline_and_tensor_parallel_ranks(par_kw):
    """Greedy generation, token scoring and the evaluation adaptor give the same result on two pipeline stages or two
    tensor-parallel ranks as in one process, on EVERY rank (sampled tokens / log-probs are handed back by the last
    stage; vocabulary-parallel logits are gathered)."""
    from dist_utils import run_distributed
    ref_toks, ref_lp, ref_scores, ref_ll = _generate(None)
    outs = run_distributed(_generate_worker, 2, par_kw=par_kw)
    for toks, lp, scores, ll in outs:
        assert torch.equal(toks, ref_toks)
        assert torch.allclose(lp, ref_lp, atol=1e-4)
        assert torch.allclose(scores, ref_scores, atol=1e-4)
        assert all(abs(a[0] - b[0]) < 1e-3 and a[1] == b[1] for a, b in zip(ll, ref_ll))

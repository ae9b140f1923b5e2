"""Argument surface, fine-tuning loop, lm-eval adaptor, preprocessing, layer patterns, failure detection (CPU)."""
import json
import os
import time

import pytest
import torch

from linear_moe_b200.config.arguments import build_parser, parse_args
from linear_moe_b200.config.model_config import ModelConfig, ParallelConfig, TrainConfig
from linear_moe_b200.config.presets import PRESETS, get_preset
from linear_moe_b200.models.layout import allocate_mamba_pattern, expand_layer_pattern, split_for_pipeline


def test_reference_flags_are_accepted():
    argv = ("--num-layers 4 --hidden-size 64 --num-attention-heads 4 --ffn-hidden-size 128 --seq-length 128 "
            "--max-position-embeddings 128 --micro-batch-size 1 --global-batch-size 8 --lr 1e-4 --min-lr 1e-5 "
            "--lr-decay-style cosine --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 "
            "--init-method-std 0.008 --attention-dropout 0.0 --hidden-dropout 0.0 --train-iters 10 --lr-warmup-iters 2 "
            "--log-interval 10 --eval-interval 100000 --eval-iters 10 --save-interval 100 --tensorboard-queue-size 1000 "
            "--log-timers-to-tensorboard --log-batch-size-to-tensorboard --log-validation-ppl-to-tensorboard "
            "--tensor-model-parallel-size 2 --pipeline-model-parallel-size 1 --context-parallel-size 1 --no-load-optim "
            "--no-load-rng --num-workers 8 --extra-vocab-size 293 --patch-tokenizer-type Qwen2Tokenizer "
            "--dataset LLama-Pretrain-Idxmap --swiglu --normalization RMSNorm --norm-epsilon 1e-6 "
            "--use-rotary-position-embeddings --no-rope-fusion --position-embedding-type rope "
            "--untie-embeddings-and-output-weights --disable-bias-linear --add-qkv-bias --group-query-attention "
            "--num-query-groups 4 --rotary-percent 1.0 --rotary-base 1000000 --rotary-seq-len-interpolation-factor 1 "
            "--no-create-attention-mask-in-dataloader --bf16 --use-distributed-optimizer --sequence-parallel "
            "--recompute-activations --moe-router-topk 2 --num-experts 8 --moe-aux-loss-coeff 1e-2 "
            "--expert-model-parallel-size 2 --moe-router-load-balancing-type aux_loss --moe-ffn-hidden-size 64 "
            "--enable-shared-expert --shared-moe-ffn-hidden-size 128 --use-la-module --la-module gated_deltanet "
            "--la-mode chunk --base-model qwen2 --la-feature-map elu --la-output-norm rmsnorm --la-gate-fn swish "
            "--layer-type-list LLLN --transformer-impl transformer_engine --use-mcore-models --use-flash-attn "
            "--fp8-hybrid --fp8-amax-history-len 1024 --fp8-amax-compute-algo max --moe-token-dropping "
            "--moe-train-capacity-factor 1.25 --top-k 5 --temperature 0.7 --out-seq-length 32 "
            "--cpu-offloading --cpu-offloading-num-layers 2 --cuda-graph-decode").split()
    args, cfg, par, tc = parse_args(argv)
    assert cfg.la_module == "gated_deltanet" and cfg.layer_type_list == "LLLN" and cfg.num_experts == 8
    assert cfg.vocab_size % (128 * 2) == 0 and not cfg.add_bias_linear and cfg.add_qkv_bias and not cfg.tie_embeddings
    assert par.tp == 2 and par.ep == 2 and par.sequence_parallel and par.use_distributed_optimizer
    assert cfg.recompute_granularity == "selective" and cfg.fp8 == "rowwise" and tc.bf16
    assert cfg.cpu_offloading and cfg.cpu_offloading_num_layers == 2 and args.cuda_graph_decode
    assert cfg.params_dtype == torch.bfloat16 and cfg.moe_token_dropping and cfg.moe_train_capacity_factor == 1.25
    names = {a.dest for a in build_parser()._actions}
    for flag in ("la_tie_feature_map_qk", "gla_la_gate_low_rank_dim", "rwkv6_la_proj_low_rank_dim", "expand_k", "a_num",
                 "megatron_hybrid_mamba_method", "hybrid_override_pattern", "kv_lora_rank", "text_generate_input_file",
                 "repetition_penalty", "max_padding_length", "keep_last", "sliding_window", "mom_num_memories"):
        assert flag in names, flag


def test_presets_build():
    for name in PRESETS:
        cfg = get_preset(name)
        specs = cfg.layer_types()
        assert len(specs) >= cfg.num_layers


def test_layer_patterns():
    cfg = ModelConfig(num_layers=4, use_la_module=True, la_module="gla", layer_type_list="LLLN", num_experts=4)
    s = expand_layer_pattern(cfg)
    assert [x.mixer for x in s] == ["lsm", "lsm", "lsm", "attn"] and all(x.ffn == "moe" for x in s)
    assert [x.index for x in split_for_pipeline(s, 2, 1)] == [2, 3]            # hybrid patterns are PP-sliced
    m = ModelConfig(num_layers=4, use_la_module=True, la_module="mamba2", hybrid_override_pattern="MM*M")
    assert "".join(x.symbol for x in expand_layer_pattern(m)) == "M-M-*-M-"     # default: an FFN block after each mixer
    lit = m.replace(megatron_hybrid_mamba_method=True, hybrid_override_pattern="M-*-")
    assert "".join(x.symbol for x in expand_layer_pattern(lit)) == "M-*-"
    auto = allocate_mamba_pattern(8, 0.25, 0.25)
    assert auto.count("*") == 2 and auto.count("-") == 2
    ds = ModelConfig(num_layers=3, base_model="deepseek_v2", num_experts=4, moe_layer_freq=1)
    assert [x.ffn for x in expand_layer_pattern(ds)] == ["mlp", "moe", "moe"] and expand_layer_pattern(ds)[0].mixer == "mla"


def test_finetune_and_eval_adaptor(tmp_path):
    from linear_moe_b200.data.datasets import RawJsonDataset
    from linear_moe_b200.data.tokenizer import NullTokenizer
    from linear_moe_b200.infer.lm_eval_adaptor import EvalHarnessAdaptor, LinearMoeOpenCompassModel
    from linear_moe_b200.train.finetune import finetune
    rows = [{"instruction": " ".join(str((i * 7 + j) % 50) for j in range(5)), "input": "",
             "output": " ".join(str((i + j) % 50) for j in range(4))} for i in range(16)]
    path = tmp_path / "sft.json"
    path.write_text(json.dumps(rows))
    tok = NullTokenizer(64)
    ds = RawJsonDataset([str(path)], tok, max_padding_length=16, sft=True)
    item = ds[0]
    assert item["text"].shape == (17,) and (item["labels_full"][:5] == -100).all() and item["labels_full"][5] >= 0
    cfg = ModelConfig(num_layers=2, hidden_size=32, num_attention_heads=2, ffn_hidden_size=64, vocab_size=64,
                      use_la_module=True, la_module="linear_attention", layer_type_list="LN")
    tc = TrainConfig(micro_batch_size=4, global_batch_size=4, seq_length=16, epochs=3, lr=3e-3, min_lr=3e-3,
                     lr_decay_style="constant", log_interval=1000, weight_decay=0.0)
    first = {}
    tr = finetune(cfg, ParallelConfig(), tc, ds, end_of_epoch_callback=lambda t, e: first.setdefault(e, t.iteration))
    assert tr.iteration == 12 and first[0] == 4
    ad = EvalHarnessAdaptor(tr.model, tok, max_length=32)
    res = ad.loglikelihood([("1 2 3", "4 5"), ("", "7")])
    assert len(res) == 2 and all(r[0] < 0 for r in res)
    assert len(ad.loglikelihood_rolling([("1 2 3 4 5 6 7 8",)])) == 1
    assert isinstance(ad.generate_until([("1 2 3", {"max_gen_toks": 4, "until": []})])[0], str)
    assert LinearMoeOpenCompassModel(tr.model, tok).get_ppl(["1 2 3 4"])[0] > 0


def test_preprocess(tmp_path):
    from linear_moe_b200.data import preprocess
    from linear_moe_b200.data.datasets import IndexedDataset
    src = tmp_path / "in.jsonl"
    src.write_text("\n".join(json.dumps({"text": " ".join(str(i + j) for j in range(6))}) for i in range(10)))
    preprocess.main(["--input", str(src), "--output-prefix", str(tmp_path / "out"), "--append-eod", "--vocab-size", "100"])
    ds = IndexedDataset(str(tmp_path / "out_text_document"))
    assert len(ds) == 10 and ds.get(3).tolist() == [3, 4, 5, 6, 7, 8, 99]


def test_heartbeat_detects_a_silent_rank():
    """Host-side failure detection: a rank that stops beating is reported; nothing touches a GPU."""
    from linear_moe_b200.train.watchdog import CommTimeout, Heartbeat, raise_on_comm_status

    class Store(dict):
        def set(self, k, v): self[k] = v.encode()
        def check(self, ks): return all(k in self for k in ks)

    class M:
        world_size = 3
        def __init__(self, r): self.rank = r
    store, now = Store(), [100.0]
    hb = [Heartbeat(M(r), 0.0, 5.0, store=store, clock=lambda: now[0]) for r in range(3)]
    for h in hb:
        h.beat(1)
    assert hb[0].check() == []
    now[0] = 104.0
    hb[0].beat(2), hb[1].beat(2)            # rank 2 went silent
    now[0] = 107.0
    assert hb[0].check() == [2] and hb[1].check() == [2]
    with pytest.raises(CommTimeout):
        raise_on_comm_status(torch.tensor([(7 << 24) | (3 << 16) | 1]), "lasp")
    raise_on_comm_status(torch.tensor([0]), "ok")


def test_convert_checkpoint_cli_roundtrip(tmp_path):
    """HF -> Megatron layout split over TP2 x EP2 -> merged back to HF through the example CLI gives the same tensors."""
    import subprocess
    import sys
    import torch
    from linear_moe_b200.ckpt import hf_convert
    from linear_moe_b200.config.model_config import ModelConfig
    from linear_moe_b200.models.transformer import CausalLM
    flags = ["--base-model", "qwen2", "--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--group-query-attention",
             "--num-query-groups", "2", "--ffn-hidden-size", "128", "--num-experts", "4", "--moe-router-topk", "2",
             "--moe-ffn-hidden-size", "32", "--vocab-size", "256", "--patch-tokenizer-type", "NullTokenizer", "--swiglu",
             "--untie-embeddings-and-output-weights", "--disable-bias-linear", "--seq-length", "32", "--max-position-embeddings", "32",
             "--micro-batch-size", "1", "--global-batch-size", "1", "--train-iters", "1"]
    from linear_moe_b200.config.arguments import parse_args
    _, cfg, _, _ = parse_args(flags)
    model = CausalLM(cfg)
    hf = hf_convert.mcore_to_hf({k: v.detach() for k, v in model.state_dict().items()}, cfg)
    hf_dir, ck, back = tmp_path / "hf", tmp_path / "ck", tmp_path / "back"
    hf_dir.mkdir()
    torch.save(hf, hf_dir / "pytorch_model.bin")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = os.path.join(root, "examples", "convert_checkpoint.py")
    subprocess.run([sys.executable, cli, "--direction", "hf2mcore", "--load", str(hf_dir), "--save", str(ck),
                    "--target-tp", "2", "--target-ep", "2", *flags], check=True, capture_output=True)
    assert (ck / "latest_checkpointed_iteration.txt").read_text() == "release"
    subprocess.run([sys.executable, cli, "--direction", "mcore2hf", "--load", str(ck), "--save", str(back),
                    "--source-tp", "2", "--source-ep", "2", *flags], check=True, capture_output=True)
    out = torch.load(back / "pytorch_model.bin")
    assert set(out) == set(hf)
    for k in hf:
        assert torch.equal(out[k], hf[k]), k


@pytest.mark.parametrize("base,size,la,pattern", [
    ("qwen2", "A0.3B", "gla", "LLLLLLLLLLLL"), ("qwen2", "A1B", "gated_deltanet", "LLLNLLLNLLLNLLLN"), ("qwen2", "7B", "none", ""),
    ("qwen2", "0.5Boriginal", "none", ""), ("qwen2", "72B", "linear_attention", "L" * 80),
    ("llama3", "1B", "lasp2", "LLLLLLLLLLLLLLLL"), ("llama3", "8B", "retention", "LLLN" * 8),
    ("mixtral", "Small", "rwkv6", "LLLLLLLL"), ("mixtral", "8x7B", "mamba2", "M-" * 16),
    ("deepseek_v2", "A2.4B", "hgrn2", "L" * 27), ("deepseek_v2", "A21B", "none", ""),
])
def test_launcher_flags_parse_into_the_model(base, size, la, pattern):
    """``examples/run_pretrain.sh`` in dry-run mode prints the flags it would pass; every model-size block of every
    backbone parses and yields the architecture the block names (the reference has one launcher per backbone)."""
    import os
    import subprocess
    from linear_moe_b200.config.arguments import parse_args
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, DRY_RUN="1", BASE_MODEL=base, MODEL_SIZE=size, LA_MODULE=la, LAYER_TYPE_LIST=pattern or "L",
               TP="2", EP="2", SP="true", PR="bf16")
    out = subprocess.run(["bash", os.path.join(root, "examples", "run_pretrain.sh")], env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    _, cfg, par, tc = parse_args(out.stdout.split())
    assert cfg.base_model == base and par.tp == 2 and par.ep == 2 and par.sequence_parallel
    assert cfg.vocab_size % (128 * 2) == 0
    assert cfg.normalization == ("LayerNorm" if base == "mixtral" else "RMSNorm")
    assert cfg.add_qkv_bias == (base == "qwen2") and not cfg.add_bias_linear and not cfg.tie_embeddings
    kinds = cfg.layer_types()
    if la == "none":
        assert not cfg.use_la_module and all(s.symbol == "N" and s.mixer in ("attn", "mla") for s in kinds)
    elif la == "mamba2":
        # without --megatron-hybrid-mamba-method every mixer block is followed by its own MLP block (the reference's default)
        assert [s.symbol for s in kinds if s.symbol != "-"] == [c for c in pattern if c != "-"]
    else:
        assert cfg.la_module == la and len(kinds) == cfg.num_layers
    if base == "deepseek_v2":
        assert cfg.kv_lora_rank == 512 and all(s.mixer == "mla" for s in kinds if s.symbol == "N")


def test_evaluation_launcher_builds_on_the_training_blocks():
    import os
    import subprocess
    from linear_moe_b200.config.arguments import build_parser, configs_from_args
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, DRY_RUN_EVAL="1", CKPT="/ckpt", VALID_DATA="/data/valid.json", BASE_MODEL="llama3",
               MODEL_SIZE="0.3B", LA_MODULE="lasp2", LAYER_TYPE_LIST="L" * 12, GPUS="2", TP="2", BATCH_SIZE="4")
    out = subprocess.run(["bash", os.path.join(root, "examples", "run_evaluate.sh")], env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    words = out.stdout.split()
    assert words[0].endswith("evaluate.py")
    p = build_parser()
    p.add_argument("--lm-eval-tasks", type=str, default=None)
    cfg, par, tc = configs_from_args(p.parse_args(words[1:]))
    assert cfg.la_module == "lasp2" and par.tp == 2 and tc.load == "/ckpt" and tc.no_load_optim and tc.eval_iters == 10
    assert tc.valid_data == ["/data/valid.json"] and tc.dataset == "LLama-Pretrain-Raw" and tc.global_batch_size == 4


def test_autoresume_checkpoints_and_exits(tmp_path, monkeypatch):
    """``--adlr-autoresume``: at the next check after the scheduler's auto-resume service (a fake ``userlib.auto_resume``
    here) or the stand-in file asks for termination, the run writes a checkpoint, asks to be queued again and stops."""
    import sys
    import types
    from linear_moe_b200.config.model_config import ModelConfig, ParallelConfig, TrainConfig
    from linear_moe_b200.train.loop import Trainer
    calls = {"asked": 0, "resume": 0}

    class AutoResume:
        @staticmethod
        def termination_requested():
            calls["asked"] += 1
            return calls["asked"] >= 2

        @staticmethod
        def request_resume():
            calls["resume"] += 1
    pkg, mod = types.ModuleType("userlib"), types.ModuleType("userlib.auto_resume")
    mod.AutoResume = AutoResume
    pkg.auto_resume = mod
    monkeypatch.setitem(sys.modules, "userlib", pkg)
    monkeypatch.setitem(sys.modules, "userlib.auto_resume", mod)
    cfg = ModelConfig(num_layers=1, hidden_size=32, num_attention_heads=2, ffn_hidden_size=64, vocab_size=64)
    kw = dict(micro_batch_size=1, global_batch_size=1, seq_length=16, train_iters=20, log_interval=100, lr=1e-3,
              adlr_autoresume=True, adlr_autoresume_interval=3)
    tr = Trainer(cfg, ParallelConfig(), TrainConfig(save=str(tmp_path / "a"), **kw), device=torch.device("cpu"))
    tr.train()
    assert tr.iteration == 6 and calls == {"asked": 2, "resume": 1}
    assert (tmp_path / "a" / "latest_checkpointed_iteration.txt").read_text().strip() == "6"
    # without the service: the file named by LMOE_AUTORESUME_FILE
    monkeypatch.delitem(sys.modules, "userlib")
    monkeypatch.delitem(sys.modules, "userlib.auto_resume")
    stop = tmp_path / "stop"
    monkeypatch.setenv("LMOE_AUTORESUME_FILE", str(stop))
    tr2 = Trainer(cfg, ParallelConfig(), TrainConfig(save=str(tmp_path / "b"), **kw), device=torch.device("cpu"))
    stop.write_text("")
    tr2.train()
    assert tr2.iteration == 3


def test_sample_based_schedule_and_checkpoint_flags(tmp_path):
    """Megatron's general training flags beyond the reference's launchers: sample-based run length and warm-up, warm-up
    as a fraction, --finetune (weights only, counters at 0), --exit-on-missing-checkpoint, --ckpt-format, --mock-data."""
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train.loop import Trainer
    base = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "64", "--seq-length", "16", "--micro-batch-size", "2", "--global-batch-size", "4", "--lr", "1e-3"]
    _, _, _, tc = parse_args(base + ["--train-samples", "400", "--lr-decay-samples", "320", "--lr-warmup-samples", "40"])
    assert (tc.train_iters, tc.lr_decay_iters, tc.lr_warmup_iters) == (100, 80, 10)
    _, _, _, tc = parse_args(base + ["--train-iters", "200", "--lr-warmup-fraction", "0.05", "--ckpt-format", "torch_dist",
                                     "--mock-data", "--tp-comm-overlap", "--log-throughput",
                                     "--accumulate-allreduce-grads-in-fp32"])
    assert tc.lr_warmup_iters == 10 and tc.use_dist_ckpt and tc.dataset == "Synthetic"
    # a run to fine-tune from
    _, cfg, _, tc = parse_args(base + ["--train-iters", "3", "--save", str(tmp_path / "ck"), "--log-interval", "100"])
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    for _ in range(3):
        tr.train_step()
    tr.save()
    _, cfg, _, tc = parse_args(base + ["--train-iters", "3", "--load", str(tmp_path / "ck"), "--finetune"])
    assert tc.no_load_optim and tc.no_load_rng
    ft = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    assert ft.iteration == 0 and ft.consumed_samples == 0 and ft.optimizer.step_count == 0
    a, b = tr.models[0].state_dict(), ft.models[0].state_dict()
    assert all(torch.equal(a[k], b[k]) for k in a)
    _, cfg, _, tc = parse_args(base + ["--load", str(tmp_path / "ck")])
    assert Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu")).iteration == 3
    # nothing to load
    _, cfg, _, tc = parse_args(base + ["--load", str(tmp_path / "nothing")])
    assert Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu")).iteration == 0
    _, cfg, _, tc = parse_args(base + ["--load", str(tmp_path / "nothing"), "--exit-on-missing-checkpoint"])
    with pytest.raises(SystemExit):
        Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))


def test_resume_takes_the_schedule_from_the_command_line_or_the_checkpoint(tmp_path):
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train.loop import Trainer
    base = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "64", "--seq-length", "16", "--micro-batch-size", "1", "--train-iters", "40",
            "--lr-decay-style", "cosine", "--lr-warmup-iters", "2", "--log-interval", "100"]
    _, cfg, _, tc = parse_args(base + ["--lr", "1e-3", "--min-lr", "1e-4", "--save", str(tmp_path)])
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    for _ in range(5):
        tr.train_step()
    tr.save()
    want_ckpt = tr.scheduler.get_lr()
    _, cfg, _, tc = parse_args(base + ["--lr", "5e-4", "--min-lr", "5e-5", "--load", str(tmp_path)])
    cli = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    assert cli.scheduler.num_steps == 5 and abs(cli.scheduler.get_lr() - want_ckpt / 2) < 1e-9
    _, cfg, _, tc = parse_args(base + ["--lr", "5e-4", "--min-lr", "5e-5", "--load", str(tmp_path),
                                      "--use-checkpoint-opt_param-scheduler"])
    kept = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    assert abs(kept.scheduler.get_lr() - want_ckpt) < 1e-12


def test_batch_size_rampup(tmp_path):
    """--rampup-batch-size 2 2 12 with a global batch of 6: batches 2 (samples 0-5), 4 (6-11), then 6; the sample
    counter, the number of micro-batches and the data position follow, also across a resume."""
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train.loop import Trainer
    base = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "64", "--seq-length", "16", "--micro-batch-size", "1", "--global-batch-size", "6", "--lr", "1e-3",
            "--train-iters", "9", "--log-interval", "100", "--rampup-batch-size", "2", "2", "12", "--save", str(tmp_path)]
    _, cfg, _, tc = parse_args(base)
    assert tc.rampup_batch_size == (2, 2, 12)
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    seen = []
    for _ in range(7):
        tr.train_step()
        seen.append((tr.global_batch_now, tr.num_microbatches, tr.consumed_samples))
    assert [s[0] for s in seen] == [2, 2, 2, 4, 4, 6, 6]
    assert [s[1] for s in seen] == [2, 2, 2, 4, 4, 6, 6] and seen[-1][2] == 26 and tr.data_iter.consumed == 26
    tr.save()
    _, cfg, _, tc = parse_args(base + ["--load", str(tmp_path)])
    again = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    a, b = tr.train_step(), again.train_step()
    assert again.consumed_samples == 32 and abs(float(a["lm loss"]) - float(b["lm loss"])) < 1e-6
    with pytest.raises(AssertionError):
        _, cfg, _, tc = parse_args(base[:-6] + ["--rampup-batch-size", "2", "3", "12"])
        Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))


def test_megatron_moe_flag_spellings(capsys):
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train.loop import Trainer
    base = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "64", "--seq-length", "16", "--micro-batch-size", "2", "--num-experts", "4", "--moe-router-topk", "2",
            "--moe-ffn-hidden-size", "32", "--moe-aux-loss-coeff", "0.01", "--base-model", "mixtral"]
    _, cfg, _, tc = parse_args(base + ["--moe-expert-capacity-factor", "1.5", "--moe-router-pre-softmax",
                                       "--moe-per-layer-logging", "--train-iters", "2", "--log-interval", "1"])
    assert cfg.moe_token_dropping and cfg.moe_train_capacity_factor == 1.5 and cfg.moe_eval_capacity_factor == 1.5
    assert cfg.moe_router_order == "softmax_topk" and tc.moe_per_layer_logging
    _, plain, _, _ = parse_args(base)
    assert plain.moe_router_order == "topk_softmax" and not plain.moe_token_dropping
    Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu")).train()
    out = capsys.readouterr().out
    assert "moe/load_balancing_loss_layer_0:" in out and "moe/load_balancing_loss_layer_1:" in out


def test_logging_and_loader_flags_have_readers(tmp_path, monkeypatch):
    """--tensorboard-log-interval, --log-timers-to-tensorboard, --num-workers, --test-mode and --num-shared-experts all
    change behaviour (none is accepted and ignored)."""
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train import loop as L
    written = []

    class Writer:
        def __init__(self, *a, **k):
            pass

        def add_scalar(self, name, value, step):
            written.append((name, step))

        def flush(self):
            pass

        def close(self):
            pass
    import torch.utils.tensorboard as tb
    monkeypatch.setattr(tb, "SummaryWriter", Writer)
    base = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "64", "--seq-length", "16", "--micro-batch-size", "2", "--train-iters", "6", "--lr", "1e-3",
            "--qk-layernorm", "--test-mode", "--num-workers", "2", "--log-interval", "4", "--tensorboard-dir", str(tmp_path),
            "--tensorboard-log-interval", "2", "--log-timers-to-tensorboard", "--timing-log-level", "1"]
    _, cfg, par, tc = parse_args(base)
    assert cfg.test_mode and tc.num_workers == 2 and tc.tensorboard_log_interval == 2
    tr = L.Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    assert tr.data_iter.prefetch == 2
    tr.train()
    steps = sorted({s for n, s in written if n == "learning-rate"})
    assert steps == [2, 4, 6], steps                           # every 2nd step, the console step 4 included once
    assert any(n.endswith("-time") for n, _ in written)
    # --test-mode notices replicated weights that drifted apart (here: a check that is made to fail)
    monkeypatch.setattr(type(tr.models[0].decoder.layers[0].self_attention), "run_realtime_tests", lambda self: False)
    with pytest.raises(RuntimeError, match="test-mode"):
        tr.train_step()
    _, ds, _, _ = parse_args(["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--num-experts", "4",
                              "--moe-ffn-hidden-size", "24", "--enable-shared-expert", "--num-shared-experts", "2"])
    assert ds.shared_moe_ffn_hidden_size == 48


def test_compatibility_only_flags_are_named_once(capsys):
    from linear_moe_b200.config.arguments import NO_EFFECT, build_parser, parse_args
    base = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2"]
    parse_args(base)
    assert "without effect" not in capsys.readouterr().out
    parse_args(base + ["--use-flash-attn", "--transformer-impl", "transformer_engine", "--vision-tower", "clip"])
    out = capsys.readouterr().out
    assert out.count("without effect here") == 1
    assert all(f in out for f in ("--use-flash-attn", "--transformer-impl", "--vision-tower"))
    dests = {a.dest for a in build_parser()._actions}
    assert NO_EFFECT <= dests, sorted(NO_EFFECT - dests)


def test_use_checkpoint_args_restores_the_architecture(tmp_path, capsys):
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train.loop import Trainer
    arch = ["--num-layers", "2", "--hidden-size", "48", "--num-attention-heads", "4", "--ffn-hidden-size", "96",
            "--vocab-size", "128", "--use-la-module", "--la-module", "retention", "--layer-type-list", "LN",
            "--group-query-attention", "--num-query-groups", "2"]
    run = ["--seq-length", "16", "--micro-batch-size", "1", "--train-iters", "1", "--log-interval", "100"]
    _, cfg, _, tc = parse_args(arch + run + ["--save", str(tmp_path)])
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    tr.train_step()
    tr.save()
    # a command line with another architecture, and a run-time switch of its own
    other = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--recompute-granularity", "full",
             "--recompute-method", "uniform"]
    _, got, _, tc2 = parse_args(other + run + ["--load", str(tmp_path), "--use-checkpoint-args"])
    assert "--use-checkpoint-args: from the checkpoint" in capsys.readouterr().out
    for k in ("num_layers", "hidden_size", "num_attention_heads", "num_query_groups", "ffn_hidden_size", "vocab_size",
              "la_module", "layer_type_list"):
        assert getattr(got, k) == getattr(cfg, k), k
    assert got.recompute_granularity == "full"                       # how it runs stays with the command line
    again = Trainer(got, ParallelConfig(), tc2, device=torch.device("cpu"))
    a, b = tr.models[0].state_dict(), again.models[0].state_dict()
    assert again.iteration == 1 and all(torch.equal(a[k], b[k]) for k in a)
    _, plain, _, _ = parse_args(other + run + ["--load", str(tmp_path)])
    assert plain.hidden_size == 32


def test_use_checkpoint_args_reads_the_sharded_format_too(tmp_path):
    from linear_moe_b200.config.arguments import parse_args
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.train.loop import Trainer
    arch = ["--num-layers", "2", "--hidden-size", "48", "--num-attention-heads", "4", "--ffn-hidden-size", "96", "--vocab-size", "128"]
    run = ["--seq-length", "16", "--micro-batch-size", "1", "--train-iters", "1", "--log-interval", "100", "--use-dist-ckpt"]
    _, cfg, _, tc = parse_args(arch + run + ["--save", str(tmp_path)])
    tr = Trainer(cfg, ParallelConfig(), tc, device=torch.device("cpu"))
    tr.train_step()
    tr.save()
    _, got, _, tc2 = parse_args(["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2"] + run +
                                ["--load", str(tmp_path), "--use-checkpoint-args"])
    assert (got.num_layers, got.hidden_size, got.ffn_hidden_size, got.vocab_size) == (2, 48, 96, cfg.vocab_size)
    assert Trainer(got, ParallelConfig(), tc2, device=torch.device("cpu")).iteration == 1


def test_skip_train_only_evaluates(capsys):
    from linear_moe_b200.train.loop import pretrain
    argv = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "64", "--seq-length", "16", "--micro-batch-size", "2", "--train-iters", "5", "--eval-iters", "2",
            "--skip-train", "--log-interval", "100"]
    trainer, stats = pretrain(argv)
    assert trainer.iteration == 0 and "lm loss" in stats and float(stats["lm loss"]) > 0
    assert "validation:" in capsys.readouterr().out


def test_window_size_spelling():
    from linear_moe_b200.config.arguments import parse_args
    b = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2"]
    assert parse_args(b + ["--window-size", "7,0"])[1].sliding_window == 8          # 7 earlier tokens + the current one
    assert parse_args(b + ["--window-size=-1,0"])[1].sliding_window is None         # no window
    assert parse_args(b + ["--sliding-window", "16", "--window-size", "3,0"])[1].sliding_window == 16
    with pytest.raises(ValueError, match="RIGHT = 0"):
        parse_args(b + ["--window-size", "7,3"])


def test_pretrain_cli_on_an_indexed_corpus_with_cache_and_read_ahead(tmp_path):
    """The whole data path through the command line: json lines -> tokenised .bin / .idx -> training with the index cache,
    the read-ahead thread, the native gather and --eod-mask-loss."""
    import json
    import os
    from linear_moe_b200.data import preprocess
    from linear_moe_b200.train.loop import pretrain
    rng = torch.Generator().manual_seed(0)
    src = tmp_path / "docs.jsonl"
    with open(src, "w") as f:
        for _ in range(40):
            n = int(torch.randint(5, 60, (1,), generator=rng))
            f.write(json.dumps({"text": " ".join(str(int(t)) for t in torch.randint(0, 100, (n,), generator=rng))}) + "\n")
    preprocess.main(["--input", str(src), "--output-prefix", str(tmp_path / "corpus"), "--patch-tokenizer-type", "NullTokenizer",
                     "--vocab-size", "128", "--append-eod"])
    prefix = next(str(tmp_path / p[:-4]) for p in os.listdir(tmp_path) if p.endswith(".idx"))
    argv = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "2", "--ffn-hidden-size", "64",
            "--vocab-size", "128", "--patch-tokenizer-type", "NullTokenizer", "--seq-length", "16", "--micro-batch-size", "2",
            "--global-batch-size", "4", "--train-iters", "4", "--lr", "1e-3", "--log-interval", "100", "--eval-interval", "1000",
            "--dataset", "LLama-Pretrain-Idxmap", "--data-path", prefix, "--split", "90,10,0",
            "--data-cache-path", str(tmp_path / "cache"), "--num-workers", "2", "--eod-mask-loss"]
    trainer, stats = pretrain(argv)
    assert trainer.iteration == 4 and trainer.consumed_samples == 16 and float(stats["lm loss"]) > 0
    assert trainer.tc.eod_token == 127 and trainer.data_iter.prefetch == 2
    assert len(os.listdir(tmp_path / "cache")) >= 3
    trainer.data_iter._shutdown()

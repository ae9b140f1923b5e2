"""Command-line front end that accepts the reference's flag names.

The reference adds ~95 flags on top of Megatron's base parser
(linear_moe/arguments.py:64-604) and its launchers pass ~120 flags in total
(examples/linear_moe_qwen2/run_pretrain_qwen.sh:388-449,
examples/linear_moe_mixtral/run_pretrain_mistral.sh:272-331,
examples/linear_moe_deepseek_v2/run_pretrain_deepseek.sh:307-366).
This module accepts the same spelling for every one of those flags and turns the
namespace into the three typed dataclasses of :mod:`model_config`.  Flags that
selected between library back ends in the reference (``--transformer-impl``,
``--use-flash-attn``, ``--moe-megablocks``, ``--no-rope-fusion`` ...) are accepted
and recorded but select nothing: there is one code path.
"""
from __future__ import annotations

import argparse
import os
from typing import Optional, Sequence, Tuple

import torch

from .model_config import LA_MODULES, ModelConfig, ParallelConfig, TrainConfig

_TOKENIZERS = (
    "JiebaBPETokenizer", "BloomTokenizerFromHF", "ChatGLMTokenizerFromHF", "GLM10BZHTokenizerFromHF",
    "IcetkGLM130BTokenizer", "OPTTokenizer", "LLamaTokenizer", "LLama2Tokenizer", "LLama3Tokenizer",
    "FalconTokenizer", "StarcoderTokenizerFromHF", "QwenTokenizer", "Qwen2Tokenizer", "QwenVLTokenizer",
    "YiTokenizer", "MistralTokenizer", "BloomTokenizerFromCustom", "VicunaTokenizerFromHF",
    "DeepSeekV2Tokenizer", "NullTokenizer",
)


def _flag(g, *names, **kw):
    g.add_argument(*names, **kw)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("linear_moe_b200", allow_abbrev=False)

    g = p.add_argument_group("network")
    _flag(g, "--num-layers", type=int, default=2)
    _flag(g, "--hidden-size", type=int, default=256)
    _flag(g, "--ffn-hidden-size", "--intermediate-size", type=int, default=None, dest="ffn_hidden_size")
    _flag(g, "--num-attention-heads", type=int, default=4)
    _flag(g, "--kv-channels", type=int, default=None)
    _flag(g, "--group-query-attention", action="store_true")
    _flag(g, "--num-query-groups", "--n-head-kv", type=int, default=None, dest="num_query_groups")
    _flag(g, "--max-position-embeddings", type=int, default=4096)
    _flag(g, "--position-embedding-type", type=str, default="rope",
          choices=["learned_absolute", "rope", "none"])
    _flag(g, "--use-rotary-position-embeddings", action="store_true")
    _flag(g, "--no-position-embedding", action="store_true")
    _flag(g, "--rotary-base", type=float, default=10000.0)
    _flag(g, "--rotary-percent", type=float, default=1.0)
    _flag(g, "--rotary-interleaved", action="store_true")
    _flag(g, "--rotary-seq-len-interpolation-factor", type=float, default=None)
    _flag(g, "--rotary-scaling-factor", "--rotary-scale-factor", type=float, default=1.0,
          dest="rotary_scaling_factor")
    _flag(g, "--normalization", type=str, default="RMSNorm", choices=["RMSNorm", "LayerNorm"])
    _flag(g, "--norm-epsilon", type=float, default=1e-6)
    _flag(g, "--swiglu", action="store_true")
    _flag(g, "--glu-activation", type=str, default=None)
    _flag(g, "--disable-bias-linear", action="store_true")
    _flag(g, "--disable-bias-linear-fc", action="store_true")
    _flag(g, "--disable-bias-attn-fc", action="store_true")
    _flag(g, "--add-qkv-bias", action="store_true")
    _flag(g, "--untie-embeddings-and-output-weights", action="store_true")
    _flag(g, "--init-method-std", type=float, default=0.02)
    _flag(g, "--attention-dropout", type=float, default=0.0)
    _flag(g, "--hidden-dropout", type=float, default=0.0)
    _flag(g, "--qk-layernorm", action="store_true")
    _flag(g, "--sliding-window", type=int, default=None)
    _flag(g, "--window-size", type=str, default=None, metavar="LEFT,RIGHT",
          help="Megatron's spelling of the attention window: LEFT earlier tokens plus the current one (RIGHT must be 0 for "
               "causal attention); the same as --sliding-window LEFT+1")
    _flag(g, "--apply-query-key-layer-scaling", action="store_true")
    _flag(g, "--vocab-size", type=int, default=None)
    _flag(g, "--extra-vocab-size", type=int, default=0)
    _flag(g, "--make-vocab-size-divisible-by", type=int, default=128)
    _flag(g, "--transformer-type", type=str, default="megatron")
    _flag(g, "--transformer-impl", type=str, default="local")
    _flag(g, "--use-mcore-models", action="store_true")
    _flag(g, "--use-flash-attn", action="store_true")
    _flag(g, "--no-rope-fusion", action="store_true")
    _flag(g, "--no-bias-swiglu-fusion", action="store_true")
    _flag(g, "--no-masked-softmax-fusion", action="store_true")
    _flag(g, "--no-create-attention-mask-in-dataloader", action="store_true")
    _flag(g, "--disable-parallel-output", action="store_true")
    _flag(g, "--attention-head-type", type=str, default=None)
    _flag(g, "--use-alibi-mask", action="store_true")
    _flag(g, "--use-normhead", action="store_true")
    _flag(g, "--embed-layernorm", action="store_true")
    _flag(g, "--position-encoding-2d", action="store_true")
    _flag(g, "--use-llama2-rotary-position-embeddings", action="store_true")
    _flag(g, "--use-mistral-rotary-position-embeddings", action="store_true")
    _flag(g, "--test-mode", action="store_true")

    g = p.add_argument_group("linear sequence modeling")
    _flag(g, "--use-la-module", action="store_true")
    _flag(g, "--la-module", type=str, default=None, choices=list(LA_MODULES))
    _flag(g, "--la-mode", type=str, default="chunk")
    _flag(g, "--base-model", type=str, default="qwen2")
    _flag(g, "--layer-type-list", type=str, default=None)
    _flag(g, "--hybrid-override-pattern", type=str, default=None)
    _flag(g, "--hybrid-attention-ratio", type=float, default=0.0)
    _flag(g, "--hybrid-mlp-ratio", type=float, default=0.0)
    _flag(g, "--megatron-hybrid-mamba-method", action="store_true")
    _flag(g, "--la-feature-map", type=str, default=None)
    _flag(g, "--la-tie-feature-map-qk", action="store_true")
    _flag(g, "--la-norm-q", action="store_true")
    _flag(g, "--la-norm-k", action="store_true")
    _flag(g, "--la-do-feature-map-norm", action="store_true")
    _flag(g, "--la-checkpointing", action="store_true")
    _flag(g, "--la-output-norm", type=str, default="rmsnorm")
    # store_false, as in the reference (arguments.py:553-556): passing it switches affine OFF
    _flag(g, "--la-elementwise-affine", action="store_false")
    _flag(g, "--la-norm-eps", type=float, default=1e-5)
    _flag(g, "--la-chunk-size", type=int, default=64)
    _flag(g, "--gla-la-gate-logit-normalizer", type=int, default=16)
    _flag(g, "--gla-la-gate-low-rank-dim", type=int, default=16)
    _flag(g, "--gla-la-clamp-min", type=float, default=None)
    _flag(g, "--rwkv6-la-proj-low-rank-dim", type=int, default=32)
    _flag(g, "--rwkv6-la-gate-low-rank-dim", type=int, default=64)
    _flag(g, "--rwkv7-la-decay-low-rank-dim", type=int, default=64)
    _flag(g, "--rwkv7-la-gate-low-rank-dim", type=int, default=128)
    _flag(g, "--rwkv7-la-a-low-rank-dim", type=int, default=64)
    _flag(g, "--la-gate-fn", type=str, default="swish")
    _flag(g, "--expand-k", type=float, default=1.0)
    _flag(g, "--expand-v", type=float, default=1.0)
    _flag(g, "--use-cache", action="store_true")
    _flag(g, "--mix-type", type=str, default=None)
    _flag(g, "--a-pooling", action="store_true")
    _flag(g, "--a-num", type=int, default=None)
    _flag(g, "--use-short-conv", action="store_true")
    _flag(g, "--no-short-conv", action="store_true")
    _flag(g, "--conv-size", type=int, default=4)
    _flag(g, "--gsa-num-slots", type=int, default=64)
    _flag(g, "--mamba-d-state", type=int, default=128)
    _flag(g, "--mamba-head-dim", type=int, default=64)
    _flag(g, "--mamba-ngroups", type=int, default=8)
    _flag(g, "--mamba-expand", type=int, default=2)
    _flag(g, "--mamba-chunk-size", type=int, default=128)
    # The reference has these only as dataclass defaults (transformer_config.py:103-109).
    _flag(g, "--mom-num-memories", type=int, default=4)
    _flag(g, "--mom-topk", type=int, default=2)
    _flag(g, "--mom-capacity", type=float, default=1.0)
    _flag(g, "--mom-shared-mem", action=argparse.BooleanOptionalAction, default=True)

    g = p.add_argument_group("moe")
    _flag(g, "--num-experts", type=int, default=None)
    _flag(g, "--moe-router-topk", "--moe-topk", type=int, default=2, dest="moe_topk")
    _flag(g, "--moe-ffn-hidden-size", type=int, default=None)
    _flag(g, "--shared-moe-ffn-hidden-size", type=int, default=None)
    _flag(g, "--enable-shared-expert", action="store_true")
    _flag(g, "--num-shared-experts", type=int, default=None)
    _flag(g, "--moe-layer-freq", type=int, default=1)
    _flag(g, "--expert-interval", type=int, default=1)
    _flag(g, "--moe-router-load-balancing-type", type=str, default="aux_loss",
          choices=["aux_loss", "sinkhorn", "none"])
    _flag(g, "--moe-aux-loss-coeff", "--moe-loss-coeff", type=float, default=0.0, dest="moe_aux_loss_coeff")
    _flag(g, "--moe-z-loss-coeff", "--z-loss-weight", type=float, default=0.0, dest="moe_z_loss_coeff")
    _flag(g, "--moe-input-jitter-eps", type=float, default=None)
    _flag(g, "--moe-token-dropping", action="store_true")
    _flag(g, "--moe-expert-capacity-factor", type=float, default=None,
          help="Megatron's spelling (the reference's router reads config.moe_expert_capacity_factor, router.py:238): sets "
               "the training and evaluation capacity factors and switches token dropping on")
    _flag(g, "--moe-router-pre-softmax", action="store_true", help="softmax over all experts before the top-k selection")
    _flag(g, "--moe-per-layer-logging", action="store_true", help="log the auxiliary losses of every MoE layer")
    _flag(g, "--moe-train-capacity-factor", type=float, default=None)
    _flag(g, "--moe-eval-capacity-factor", type=float, default=None)
    _flag(g, "--moe-min-capacity", type=int, default=4)
    _flag(g, "--moe-pad-expert-input-to-capacity", action="store_true")
    _flag(g, "--moe-token-drop-policy", type=str, default="probs", choices=["probs", "position"])
    _flag(g, "--moe-token-dispatcher-type", type=str, default="alltoall", choices=["alltoall", "allgather"])
    _flag(g, "--moe-grouped-gemm", action="store_true")
    _flag(g, "--moe-megablocks", action="store_true")
    _flag(g, "--moe-layer-recompute", action="store_true")
    _flag(g, "--moe", action="store_true")
    _flag(g, "--use-tutel", action="store_true")
    _flag(g, "--router-type", type=str, default="topk")
    _flag(g, "--moe-input-feature-slicing", action="store_true")
    _flag(g, "--expert-tensor-parallelism", action="store_true")

    g = p.add_argument_group("mla")
    _flag(g, "--q-lora-rank", type=int, default=None)
    _flag(g, "--kv-lora-rank", type=int, default=512)
    _flag(g, "--qk-nope-head-dim", type=int, default=128)
    _flag(g, "--qk-rope-head-dim", type=int, default=64)
    _flag(g, "--v-head-dim", type=int, default=128)

    g = p.add_argument_group("parallel")
    _flag(g, "--tensor-model-parallel-size", type=int, default=1)
    _flag(g, "--pipeline-model-parallel-size", type=int, default=1)
    _flag(g, "--num-layers-per-virtual-pipeline-stage", type=int, default=None)
    _flag(g, "--context-parallel-size", type=int, default=1)
    _flag(g, "--expert-model-parallel-size", "--moe-expert-parallel-size", type=int, default=1,
          dest="expert_model_parallel_size")
    _flag(g, "--sequence-parallel", action="store_true")
    _flag(g, "--use-distributed-optimizer", action="store_true")
    _flag(g, "--overlap-grad-reduce", action=argparse.BooleanOptionalAction, default=False)
    _flag(g, "--overlap-param-gather", action=argparse.BooleanOptionalAction, default=False)
    _flag(g, "--distributed-backend", type=str, default="nccl", choices=["nccl", "gloo"])
    _flag(g, "--distributed-timeout-minutes", type=int, default=10)
    _flag(g, "--no-fused-comm", action="store_true")
    _flag(g, "--fused-comm-timeout-s", type=float, default=20.0)
    _flag(g, "--local-rank", "--local_rank", type=int, default=None, dest="local_rank")

    g = p.add_argument_group("training")
    _flag(g, "--micro-batch-size", type=int, default=1)
    _flag(g, "--global-batch-size", type=int, default=None)
    _flag(g, "--seq-length", type=int, default=2048)
    _flag(g, "--train-iters", type=int, default=10)
    _flag(g, "--lr", type=float, default=1e-4)
    _flag(g, "--min-lr", type=float, default=1e-5)
    _flag(g, "--lr-decay-style", type=str, default="cosine",
          choices=["constant", "linear", "cosine", "inverse-square-root"])
    _flag(g, "--lr-decay-iters", type=int, default=None)
    _flag(g, "--lr-warmup-iters", type=int, default=0)
    _flag(g, "--lr-warmup-fraction", type=float, default=None, help="warm-up as a fraction of the decay span")
    _flag(g, "--train-samples", type=int, default=None, help="sample-based run length (with a constant global batch)")
    _flag(g, "--lr-decay-samples", type=int, default=None)
    _flag(g, "--lr-warmup-samples", type=int, default=0)
    _flag(g, "--skip-train", action="store_true", help="evaluate only")
    _flag(g, "--optimizer", type=str, default="adam", choices=["adam", "sgd"])
    _flag(g, "--sgd-momentum", type=float, default=0.9)
    _flag(g, "--rampup-batch-size", type=int, nargs=3, default=None, metavar=("START", "INCREMENT", "SAMPLES"),
          help="grow the global batch from START by INCREMENT to --global-batch-size over the first SAMPLES samples")
    _flag(g, "--empty-unused-memory-level", type=int, default=0, choices=[0, 1, 2],
          help="release the caching allocator's free blocks every step (1: after the step, 2: also after backward)")
    _flag(g, "--lr-warmup-init", type=float, default=0.0)
    _flag(g, "--weight-decay", type=float, default=0.1)
    _flag(g, "--start-weight-decay", type=float, default=None)
    _flag(g, "--end-weight-decay", type=float, default=None)
    _flag(g, "--weight-decay-incr-style", type=str, default="constant")
    _flag(g, "--adam-beta1", type=float, default=0.9)
    _flag(g, "--adam-beta2", type=float, default=0.95)
    _flag(g, "--adam-eps", type=float, default=1e-8)
    _flag(g, "--clip-grad", type=float, default=1.0)
    _flag(g, "--bf16", action="store_true")
    _flag(g, "--fp16", action="store_true")
    _flag(g, "--fp8-hybrid", action="store_true")
    _flag(g, "--fp8-format", type=str, default=None)
    _flag(g, "--fp8-amax-history-len", type=int, default=1024)
    _flag(g, "--fp8-amax-compute-algo", type=str, default="max")
    _flag(g, "--loss-scale", type=float, default=None)
    _flag(g, "--initial-loss-scale", type=float, default=2.0 ** 32)
    _flag(g, "--min-loss-scale", type=float, default=1.0)
    _flag(g, "--loss-scale-window", type=int, default=1000)
    _flag(g, "--hysteresis", type=int, default=2)
    _flag(g, "--seed", type=int, default=1234)
    _flag(g, "--recompute-activations", action="store_true")
    _flag(g, "--recompute-granularity", type=str, default=None, choices=["full", "selective"])
    _flag(g, "--recompute-method", type=str, default=None, choices=["uniform", "block"])
    _flag(g, "--recompute-num-layers", type=int, default=1)
    _flag(g, "--cuda-graph-decode", action="store_true",
          help="generation: replay one-token steps from a CUDA graph (models with fixed-size caches)")
    _flag(g, "--cpu-offloading", action="store_true")
    _flag(g, "--cpu-offloading-num-layers", type=int, default=0)
    _flag(g, "--train-mode", type=str, default="pretrain", choices=["pretrain", "finetune"])
    _flag(g, "--check-for-nan-in-loss-and-grad", action=argparse.BooleanOptionalAction, default=True)
    _flag(g, "--exit-interval", type=int, default=None)
    _flag(g, "--adlr-autoresume", action="store_true",
          help="checkpoint and exit when the cluster's auto-resume service (or the file named by LMOE_AUTORESUME_FILE) asks")
    _flag(g, "--adlr-autoresume-interval", type=int, default=1000)
    _flag(g, "--manual-gc", action="store_true")
    _flag(g, "--manual-gc-interval", type=int, default=0)
    _flag(g, "--exit-duration-in-mins", type=float, default=None)
    _flag(g, "--exit-signal-handler", action="store_true")
    _flag(g, "--heartbeat-interval-s", type=float, default=0.0)
    _flag(g, "--heartbeat-timeout-s", type=float, default=60.0)
    _flag(g, "--max-tokens-to-oom", type=int, default=12000)

    g = p.add_argument_group("logging")
    _flag(g, "--log-interval", type=int, default=10)
    _flag(g, "--eval-interval", type=int, default=100000)
    _flag(g, "--eval-iters", type=int, default=10)
    _flag(g, "--tensorboard-dir", type=str, default=None)
    _flag(g, "--tensorboard-log-interval", type=int, default=10)
    _flag(g, "--tensorboard-queue-size", type=int, default=1000)
    _flag(g, "--log-timers-to-tensorboard", action="store_true")
    _flag(g, "--log-batch-size-to-tensorboard", action="store_true")
    _flag(g, "--log-validation-ppl-to-tensorboard", action="store_true")
    _flag(g, "--log-memory-to-tensorboard", action="store_true")
    _flag(g, "--timing-log-level", type=int, default=0, choices=[0, 1, 2])
    _flag(g, "--barrier-with-L1-time", action=argparse.BooleanOptionalAction, default=True)
    _flag(g, "--transformer-timers", action="store_true")
    _flag(g, "--preset", type=str, default=None)            # model architecture from config/presets.py instead of flags
    _flag(g, "--profile", action="store_true")
    _flag(g, "--profile-step-start", type=int, default=10)
    _flag(g, "--profile-step-end", type=int, default=12)
    _flag(g, "--profile-ranks", type=int, nargs="+", default=[0])

    g = p.add_argument_group("checkpointing")
    _flag(g, "--save", type=str, default=None)
    _flag(g, "--load", type=str, default=None)
    _flag(g, "--save-interval", type=int, default=None)
    _flag(g, "--pretrained-checkpoint", type=str, default=None)
    _flag(g, "--no-load-optim", action="store_true")
    _flag(g, "--override-opt_param-scheduler", action="store_true", dest="override_opt_param_scheduler",
          help="on resume take the learning-rate schedule from the command line (the default), without the note")
    _flag(g, "--use-checkpoint-opt_param-scheduler", action="store_true", dest="use_checkpoint_opt_param_scheduler",
          help="on resume take the learning-rate schedule stored in the checkpoint")
    _flag(g, "--finetune", action="store_true",
          help="load the weights only and start from iteration 0 (no optimizer state, no random state)")
    _flag(g, "--exit-on-missing-checkpoint", action="store_true", help="stop when --load names no checkpoint")
    _flag(g, "--ckpt-format", type=str, default=None, choices=["torch", "torch_dist"],
          help="torch = the legacy mp_rank layout, torch_dist = the sharded format (same as --use-dist-ckpt)")
    # accepted for launcher compatibility; what they ask for is always on here
    _flag(g, "--accumulate-allreduce-grads-in-fp32", action="store_true", help="gradients are accumulated and reduced in fp32")
    _flag(g, "--tp-comm-overlap", action="store_true", help="the fused all-gather / reduce-scatter GEMMs overlap by construction")
    _flag(g, "--log-throughput", action="store_true", help="tokens/s and model FLOP/s utilisation are always in the log line")
    _flag(g, "--mock-data", action="store_true", help="same as --dataset Synthetic")
    _flag(g, "--attention-softmax-in-fp32", action="store_true", help="the attention kernels always take the softmax in fp32")
    _flag(g, "--use-cpu-initialization", action="store_true",
          help="initial weights depend on (seed, parameter name) only, so every parallel layout starts from the same model")
    _flag(g, "--no-load-rng", action="store_true")
    _flag(g, "--no-save-optim", action="store_true")
    _flag(g, "--no-save-rng", action="store_true")
    _flag(g, "--async-save", action="store_true")
    _flag(g, "--use-dist-ckpt", action="store_true")
    _flag(g, "--dist-ckpt-format", type=str, default="torch_dist", choices=["torch_dist", "zarr"])
    _flag(g, "--auto-detect-ckpt-format", action="store_true")
    _flag(g, "--use-checkpoint-args", action="store_true")
    _flag(g, "--convert-checkpoint-from-megatron-to-transformers", action="store_true")

    g = p.add_argument_group("data")
    _flag(g, "--dataset", type=str, default="Synthetic",
          choices=["Synthetic", "LLama-Pretrain-Idxmap", "LLama-Pretrain-Raw", "LLama-SFT"])
    _flag(g, "--data-path", "--data-dir", type=str, nargs="*", default=None, dest="data_path")
    _flag(g, "--train-data", "--train-data-path", type=str, nargs="*", default=None, dest="train_data")
    _flag(g, "--valid-data", "--valid-data-path", type=str, nargs="*", default=None, dest="valid_data")
    _flag(g, "--split", type=str, default="99,1,0")
    _flag(g, "--max-padding-length", type=int, default=None)
    _flag(g, "--num-workers", type=int, default=0)
    _flag(g, "--data-cache-path", type=str, default=None, help="folder for the dataset index arrays (built once, then memory-mapped)")
    _flag(g, "--epochs", type=int, default=None)
    _flag(g, "--keep-last", action="store_true")
    _flag(g, "--eod-mask-loss", action="store_true")
    _flag(g, "--tokenizer-type", type=str, default="NullTokenizer")
    _flag(g, "--patch-tokenizer-type", type=str, default="NullTokenizer", choices=list(_TOKENIZERS))
    _flag(g, "--tokenizer-model", "--load-tokenizer", type=str, default=None, dest="tokenizer_model")
    _flag(g, "--source-seq-len", type=int, default=None)
    _flag(g, "--target-seq-len", type=int, default=None)

    g = p.add_argument_group("generation / evaluation")
    _flag(g, "--top-p", type=float, default=0.0)
    _flag(g, "--top-k", type=int, default=0)
    _flag(g, "--temperature", type=float, default=1.0)
    _flag(g, "--out-seq-length", type=int, default=1024)
    _flag(g, "--generation-length", type=int, default=None)
    _flag(g, "--repetition-penalty", "--repetition_penalty", type=float, default=1.0, dest="repetition_penalty")
    _flag(g, "--verbosity", type=str, default="INFO", help="logging verbosity of the evaluation harness adaptor")
    _flag(g, "--text-generate-input-file", type=str, default="")
    _flag(g, "--text-generate-output-file", type=str, default="")
    _flag(g, "--text-generate-gt-file", type=str, default="")
    _flag(g, "--time", action="store_true")
    _flag(g, "--input-len", type=int, default=1)
    _flag(g, "--eval-dev", action="store_true")
    _flag(g, "--eval-fp32", action="store_true")
    _flag(g, "--task-list", type=str, default="all")
    _flag(g, "--num-fewshot", type=int, default=None)
    _flag(g, "--adaptive-seq-len", action="store_true")

    # Multimodal leftovers of the reference's parser (arguments.py:270-330): no data path reaches
    # them (linear_moe/data/__init__.py:23-27 has the imports commented out); accepted, unused.
    g = p.add_argument_group("vestigial")
    for name in ("--mm-use-im-start-end", "--mm-use-im-patch-token", "--tune-mm-mlp-adapter",
                 "--freeze-clip-vision-tower", "--freeze-llm", "--cvcuda-image-processing"):
        _flag(g, name, action="store_true")
    for name in ("--image-folder", "--vision-tower", "--image-aspect-ratio", "--version",
                 "--mm-projector-type"):
        _flag(g, name, type=str, default=None)
    for name in ("--mm-vision-select-layer", "--image-size", "--patch-size"):
        _flag(g, name, type=int, default=None)
    return p


def get_patch_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    """Compatibility hook with the reference's name (arguments.py:64): returns a parser that
    already knows every patch flag."""
    return parser


def pad_vocab(vocab: int, divisible_by: int, tp: int) -> int:
    """Round the vocabulary up so that it splits evenly over TP ranks
    (tokenizer/__init__.py:17-31 ``_vocab_size_with_padding``)."""
    mult = divisible_by * tp
    return (vocab + mult - 1) // mult * mult


def configs_from_args(args: argparse.Namespace) -> Tuple[ModelConfig, ParallelConfig, TrainConfig]:
    if getattr(args, "window_size", None) and args.sliding_window is None:
        left, _, right = args.window_size.partition(",")
        if int(right or 0) != 0:
            raise ValueError("--window-size: causal attention takes RIGHT = 0")
        args.sliding_window = None if int(left) < 0 else int(left) + 1
    if args.moe_expert_capacity_factor is not None:
        args.moe_token_dropping = True
        if args.moe_train_capacity_factor is None:
            args.moe_train_capacity_factor = args.moe_expert_capacity_factor
        if args.moe_eval_capacity_factor is None:
            args.moe_eval_capacity_factor = args.moe_expert_capacity_factor
    dtype = torch.bfloat16 if args.bf16 else torch.float16 if args.fp16 else torch.float32
    vocab = args.vocab_size if args.vocab_size is not None else 32000
    vocab = pad_vocab(vocab + args.extra_vocab_size, args.make_vocab_size_divisible_by,
                      args.tensor_model_parallel_size)
    pos = args.position_embedding_type
    if args.no_position_embedding:
        pos = "none"
    recompute = args.recompute_granularity
    if args.recompute_activations and recompute is None:
        recompute = "selective"
    use_conv = args.use_short_conv and not args.no_short_conv
    ffn = args.ffn_hidden_size if args.ffn_hidden_size is not None else 4 * args.hidden_size
    model = ModelConfig(
        base_model=args.base_model, num_layers=args.num_layers, hidden_size=args.hidden_size,
        num_attention_heads=args.num_attention_heads,
        num_query_groups=args.num_query_groups if (args.group_query_attention or args.num_query_groups) else None,
        kv_channels=args.kv_channels, ffn_hidden_size=ffn, vocab_size=vocab,
        max_position_embeddings=args.max_position_embeddings, normalization=args.normalization,
        norm_eps=args.norm_epsilon, swiglu=args.swiglu or args.glu_activation == "swiglu" or True,
        add_bias_linear=not (args.disable_bias_linear or args.disable_bias_linear_fc),
        add_qkv_bias=args.add_qkv_bias and not args.disable_bias_attn_fc,
        tie_embeddings=not args.untie_embeddings_and_output_weights,
        init_method_std=args.init_method_std, hidden_dropout=args.hidden_dropout,
        attention_dropout=args.attention_dropout, qk_layernorm=args.qk_layernorm,
        sliding_window=args.sliding_window, position_embedding_type=pos,
        rotary_base=args.rotary_base, rotary_percent=args.rotary_percent,
        rotary_interleaved=args.rotary_interleaved, rotary_scaling_factor=args.rotary_scaling_factor,
        rotary_seq_len_interpolation_factor=args.rotary_seq_len_interpolation_factor,
        use_la_module=args.use_la_module, la_module=args.la_module, layer_type_list=args.layer_type_list,
        hybrid_override_pattern=args.hybrid_override_pattern,
        megatron_hybrid_mamba_method=args.megatron_hybrid_mamba_method,
        hybrid_attention_ratio=args.hybrid_attention_ratio, hybrid_mlp_ratio=args.hybrid_mlp_ratio,
        la_mode=args.la_mode, la_feature_map=args.la_feature_map,
        la_tie_feature_map_qk=args.la_tie_feature_map_qk, la_norm_q=args.la_norm_q, la_norm_k=args.la_norm_k,
        la_do_feature_map_norm=args.la_do_feature_map_norm, la_checkpointing=args.la_checkpointing,
        la_output_norm=args.la_output_norm, la_elementwise_affine=args.la_elementwise_affine,
        la_norm_eps=args.la_norm_eps, la_gate_fn=args.la_gate_fn, la_chunk_size=args.la_chunk_size,
        expand_k=args.expand_k, expand_v=args.expand_v,
        gla_la_gate_logit_normalizer=args.gla_la_gate_logit_normalizer,
        gla_la_gate_low_rank_dim=args.gla_la_gate_low_rank_dim, gla_la_clamp_min=args.gla_la_clamp_min,
        rwkv6_la_proj_low_rank_dim=args.rwkv6_la_proj_low_rank_dim,
        rwkv6_la_gate_low_rank_dim=args.rwkv6_la_gate_low_rank_dim,
        rwkv7_la_decay_low_rank_dim=args.rwkv7_la_decay_low_rank_dim,
        rwkv7_la_gate_low_rank_dim=args.rwkv7_la_gate_low_rank_dim,
        rwkv7_la_a_low_rank_dim=args.rwkv7_la_a_low_rank_dim,
        gsa_num_slots=args.gsa_num_slots, use_short_conv=use_conv, conv_size=args.conv_size,
        mamba_d_state=args.mamba_d_state, mamba_head_dim=args.mamba_head_dim,
        mamba_ngroups=args.mamba_ngroups, mamba_expand=args.mamba_expand,
        mamba_chunk_size=args.mamba_chunk_size,
        mom_num_memories=args.mom_num_memories, mom_topk=args.mom_topk, mom_capacity=args.mom_capacity,
        mom_shared_mem=args.mom_shared_mem,
        num_experts=args.num_experts, moe_topk=args.moe_topk, moe_ffn_hidden_size=args.moe_ffn_hidden_size,
        shared_moe_ffn_hidden_size=args.shared_moe_ffn_hidden_size,
        enable_shared_expert=args.enable_shared_expert, num_shared_experts=args.num_shared_experts,
        moe_layer_freq=args.moe_layer_freq, expert_interval=args.expert_interval,
        moe_router_load_balancing_type=args.moe_router_load_balancing_type,
        moe_router_order="softmax_topk" if args.moe_router_pre_softmax else None,
        moe_aux_loss_coeff=args.moe_aux_loss_coeff, moe_z_loss_coeff=args.moe_z_loss_coeff,
        moe_input_jitter_eps=args.moe_input_jitter_eps, moe_token_dropping=args.moe_token_dropping,
        moe_train_capacity_factor=args.moe_train_capacity_factor,
        moe_eval_capacity_factor=args.moe_eval_capacity_factor, moe_min_capacity=args.moe_min_capacity,
        moe_pad_expert_input_to_capacity=args.moe_pad_expert_input_to_capacity,
        moe_token_drop_policy=args.moe_token_drop_policy,
        moe_token_dispatcher_type=args.moe_token_dispatcher_type,
        moe_layer_recompute=args.moe_layer_recompute,
        q_lora_rank=args.q_lora_rank, kv_lora_rank=args.kv_lora_rank,
        qk_nope_head_dim=args.qk_nope_head_dim, qk_rope_head_dim=args.qk_rope_head_dim,
        v_head_dim=args.v_head_dim, params_dtype=dtype,
        fp8="rowwise" if (args.fp8_hybrid or args.fp8_format) else None,
        recompute_granularity=recompute, recompute_method=args.recompute_method,
        recompute_num_layers=args.recompute_num_layers, test_mode=args.test_mode,
        cpu_offloading=args.cpu_offloading, cpu_offloading_num_layers=args.cpu_offloading_num_layers,
    )
    vpp = None
    if args.num_layers_per_virtual_pipeline_stage:
        per_stage = args.num_layers // args.pipeline_model_parallel_size
        vpp = per_stage // args.num_layers_per_virtual_pipeline_stage
    par = ParallelConfig(
        tensor_model_parallel_size=args.tensor_model_parallel_size,
        pipeline_model_parallel_size=args.pipeline_model_parallel_size,
        virtual_pipeline_model_parallel_size=vpp,
        context_parallel_size=args.context_parallel_size,
        expert_model_parallel_size=args.expert_model_parallel_size,
        sequence_parallel=args.sequence_parallel and args.tensor_model_parallel_size > 1,
        use_distributed_optimizer=args.use_distributed_optimizer,
        overlap_grad_reduce=args.overlap_grad_reduce, overlap_param_gather=args.overlap_param_gather,
        distributed_backend=args.distributed_backend,
        distributed_timeout_minutes=args.distributed_timeout_minutes,
        fused_comm=not args.no_fused_comm, fused_comm_timeout_s=args.fused_comm_timeout_s,
    )
    gbs = args.global_batch_size if args.global_batch_size is not None else args.micro_batch_size
    if args.train_samples is not None:              # sample-based schedule: the global batch is constant, so iterations
        args.train_iters = args.train_samples // gbs
        if args.lr_decay_samples is not None:
            args.lr_decay_iters = args.lr_decay_samples // gbs
        if args.lr_warmup_samples:
            args.lr_warmup_iters = args.lr_warmup_samples // gbs
    if args.lr_warmup_fraction is not None:
        span = args.lr_decay_iters if args.lr_decay_iters is not None else args.train_iters
        args.lr_warmup_iters = int(args.lr_warmup_fraction * span)
    if args.finetune:
        args.no_load_optim = args.no_load_rng = True
    if args.ckpt_format == "torch_dist":
        args.use_dist_ckpt = True
    if args.mock_data:
        args.dataset = "Synthetic"
    train = TrainConfig(
        micro_batch_size=args.micro_batch_size, global_batch_size=gbs, seq_length=args.seq_length,
        train_iters=args.train_iters, lr=args.lr, min_lr=args.min_lr, lr_decay_style=args.lr_decay_style,
        lr_decay_iters=args.lr_decay_iters, lr_warmup_iters=args.lr_warmup_iters,
        lr_warmup_init=args.lr_warmup_init, weight_decay=args.weight_decay,
        start_weight_decay=args.start_weight_decay, end_weight_decay=args.end_weight_decay,
        weight_decay_incr_style=args.weight_decay_incr_style, adam_beta1=args.adam_beta1,
        adam_beta2=args.adam_beta2, adam_eps=args.adam_eps, clip_grad=args.clip_grad, bf16=args.bf16,
        fp16=args.fp16, loss_scale=args.loss_scale, initial_loss_scale=args.initial_loss_scale,
        min_loss_scale=args.min_loss_scale, loss_scale_window=args.loss_scale_window,
        hysteresis=args.hysteresis, seed=args.seed, log_interval=args.log_interval,
        eval_interval=args.eval_interval, eval_iters=args.eval_iters, save_interval=args.save_interval,
        save=args.save, load=args.load, pretrained_checkpoint=args.pretrained_checkpoint,
        no_load_optim=args.no_load_optim, no_load_rng=args.no_load_rng, no_save_optim=args.no_save_optim,
        no_save_rng=args.no_save_rng, async_save=args.async_save, use_dist_ckpt=args.use_dist_ckpt,
        auto_detect_ckpt_format=args.auto_detect_ckpt_format, tensorboard_dir=args.tensorboard_dir,
        tensorboard_log_interval=args.tensorboard_log_interval, tensorboard_queue_size=args.tensorboard_queue_size,
        log_timers_to_tensorboard=args.log_timers_to_tensorboard,
        log_memory_to_tensorboard=args.log_memory_to_tensorboard,
        log_validation_ppl_to_tensorboard=args.log_validation_ppl_to_tensorboard,
        timing_log_level=args.timing_log_level, barrier_with_L1_time=args.barrier_with_L1_time,
        exit_interval=args.exit_interval, exit_duration_in_mins=args.exit_duration_in_mins,
        optimizer=args.optimizer, sgd_momentum=args.sgd_momentum, moe_per_layer_logging=args.moe_per_layer_logging,
        rampup_batch_size=tuple(args.rampup_batch_size) if args.rampup_batch_size else None,
        override_opt_param_scheduler=args.override_opt_param_scheduler,
        use_checkpoint_opt_param_scheduler=args.use_checkpoint_opt_param_scheduler,
        finetune=args.finetune, exit_on_missing_checkpoint=args.exit_on_missing_checkpoint, skip_train=args.skip_train,
        empty_unused_memory_level=args.empty_unused_memory_level,
        adlr_autoresume=args.adlr_autoresume, adlr_autoresume_interval=args.adlr_autoresume_interval,
        manual_gc=args.manual_gc, manual_gc_interval=args.manual_gc_interval,
        exit_signal_handler=args.exit_signal_handler,
        check_for_nan_in_loss_and_grad=args.check_for_nan_in_loss_and_grad, profile=args.profile,
        profile_step_start=args.profile_step_start, profile_step_end=args.profile_step_end,
        profile_ranks=list(args.profile_ranks), dataset=args.dataset, data_path=args.data_path,
        train_data=args.train_data, valid_data=args.valid_data, split=args.split,
        max_padding_length=args.max_padding_length, num_workers=args.num_workers, epochs=args.epochs,
        keep_last=args.keep_last, eod_mask_loss=args.eod_mask_loss,
        heartbeat_interval_s=args.heartbeat_interval_s, heartbeat_timeout_s=args.heartbeat_timeout_s,
    )
    if getattr(args, "preset", None):
        # a named preset replaces the architecture flags (parallelism, precision and training flags still apply)
        from .presets import get_preset
        model = get_preset(args.preset, params_dtype=dtype, fp8=model.fp8 or None)
    return model, par, train


# Flags of the reference's launchers that select something this framework has one form of (a fused kernel that is always
# used, a Megatron code path that does not exist here) or that the reference itself never reads (its multimodal and
# vestigial model switches).  They parse, and a run that sets one says so once instead of silently ignoring it.
NO_EFFECT = frozenset("""
use_rotary_position_embeddings apply_query_key_layer_scaling transformer_type transformer_impl use_mcore_models
use_flash_attn no_rope_fusion no_bias_swiglu_fusion no_masked_softmax_fusion no_create_attention_mask_in_dataloader
disable_parallel_output attention_head_type use_alibi_mask use_normhead embed_layernorm position_encoding_2d
use_llama2_rotary_position_embeddings use_mistral_rotary_position_embeddings use_cache mix_type a_pooling a_num
moe_grouped_gemm moe_megablocks moe use_tutel router_type moe_input_feature_slicing expert_tensor_parallelism
fp8_amax_history_len fp8_amax_compute_algo train_mode max_tokens_to_oom log_batch_size_to_tensorboard transformer_timers
dist_ckpt_format tokenizer_type source_seq_len target_seq_len generation_length text_generate_gt_file
time input_len eval_dev eval_fp32 adaptive_seq_len mm_use_im_start_end mm_use_im_patch_token tune_mm_mlp_adapter
freeze_clip_vision_tower freeze_llm cvcuda_image_processing image_folder vision_tower image_aspect_ratio version
mm_projector_type mm_vision_select_layer image_size patch_size la_checkpointing moe_pad_expert_input_to_capacity
""".split())


def flags_without_effect(parser: argparse.ArgumentParser, args: argparse.Namespace):
    """Option strings of the ``NO_EFFECT`` flags that the command line set to something other than their default."""
    out = []
    for a in parser._actions:
        if a.dest in NO_EFFECT and a.option_strings and getattr(args, a.dest, a.default) != a.default:
            out.append(a.option_strings[0])
    return sorted(out)


# what --use-checkpoint-args does NOT take from the checkpoint: how the model is run, not what it is
_RUNTIME_FIELDS = frozenset("""params_dtype recompute_granularity recompute_method recompute_num_layers moe_layer_recompute
cpu_offloading cpu_offloading_num_layers cross_entropy_chunk test_mode fp8 la_mode hidden_dropout attention_dropout
moe_token_dispatcher_type""".split())


def apply_checkpoint_args(model: ModelConfig, load: str) -> ModelConfig:
    """``--use-checkpoint-args``: the architecture (every model field a checkpoint stores, except the run-time switches)
    comes from the checkpoint under ``load`` instead of the command line."""
    import dataclasses
    from ..ckpt.legacy import read_checkpoint_args
    stored = read_checkpoint_args(load)
    if stored is None:
        return model
    take = {}
    for f in dataclasses.fields(ModelConfig):
        if f.name in _RUNTIME_FIELDS or not hasattr(stored, f.name):
            continue
        v = getattr(stored, f.name)
        if v != getattr(model, f.name):
            take[f.name] = v
    if take and int(os.environ.get("RANK", "0")) == 0:
        print("> --use-checkpoint-args: from the checkpoint: " + ", ".join(f"{k}={v}" for k, v in sorted(take.items())),
              flush=True)
    return model.replace(**take) if take else model


def parse_args(argv: Optional[Sequence[str]] = None):
    """Parse ``argv`` → ``(namespace, ModelConfig, ParallelConfig, TrainConfig)``."""
    parser = build_parser()
    args = parser.parse_args(argv)
    ignored = flags_without_effect(parser, args)
    if ignored and int(os.environ.get("RANK", "0")) == 0:
        print("> accepted for launcher compatibility, without effect here: " + " ".join(ignored), flush=True)
    model, par, train = configs_from_args(args)
    if args.use_checkpoint_args and args.load:
        model = apply_checkpoint_args(model, args.load)
    return args, model, par, train

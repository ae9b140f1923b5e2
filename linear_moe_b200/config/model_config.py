"""Typed configuration for models, parallel layout and training.

The reference keeps one flat ``argparse.Namespace`` that is copied field-by-name
into a per-family ``TransformerConfig`` subclass
(linear_moe/arguments.py:23-61, linear_moe/model/qwen2/transformer_config.py:19-115,
linear_moe/model/deepseek_v2/transformer_config.py:6-90) and read back through a
global ``get_args()``.  Here the same information lives in three explicit
dataclasses that are passed down the constructor chain; nothing is global.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

LA_MODULES = (
    "linear_attention", "lightning_attention", "retention", "gla", "deltanet",
    "gated_deltanet", "gsa", "based", "rebased", "hgrn2", "rwkv6", "rwkv7",
    "mamba2", "lasp2", "mom_gla", "mom_gated_deltanet", "mom_linear_attention",
)
BASE_MODELS = ("qwen2", "llama3", "mixtral", "deepseek_v2")


@dataclass
class ModelConfig:
    # ---- backbone -------------------------------------------------------
    base_model: str = "qwen2"
    num_layers: int = 2
    hidden_size: int = 256
    num_attention_heads: int = 4
    num_query_groups: Optional[int] = None        # GQA groups for 'N' layers
    kv_channels: Optional[int] = None             # head dim
    ffn_hidden_size: int = 1024
    vocab_size: int = 32000                       # already padded
    max_position_embeddings: int = 4096
    normalization: str = "RMSNorm"                # RMSNorm | LayerNorm
    norm_eps: float = 1e-6
    swiglu: bool = True
    add_bias_linear: bool = False
    add_qkv_bias: bool = False
    tie_embeddings: bool = False
    init_method_std: float = 0.02
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    qk_layernorm: bool = False
    sliding_window: Optional[int] = None
    # ---- positional -----------------------------------------------------
    position_embedding_type: str = "rope"         # rope | none
    rotary_base: float = 10000.0
    rotary_percent: float = 1.0
    rotary_interleaved: bool = False
    rotary_scaling_factor: float = 1.0            # YaRN factor (deepseek_v2)
    rotary_seq_len_interpolation_factor: Optional[float] = None
    # ---- token mixer layout --------------------------------------------
    use_la_module: bool = False
    la_module: Optional[str] = None
    layer_type_list: Optional[str] = None         # e.g. "LLLNLLLN"
    hybrid_override_pattern: Optional[str] = None  # e.g. "MMM*MMM*" / "M-M-*-"
    megatron_hybrid_mamba_method: bool = False
    hybrid_attention_ratio: float = 0.0
    hybrid_mlp_ratio: float = 0.0
    # ---- LSM hyper-parameters ------------------------------------------
    la_mode: str = "chunk"                        # chunk | fused_chunk | fused_recurrent | parallel
    la_feature_map: Optional[str] = None
    la_tie_feature_map_qk: bool = False
    la_norm_q: bool = False
    la_norm_k: bool = False
    la_do_feature_map_norm: bool = False
    la_checkpointing: bool = False
    la_output_norm: str = "rmsnorm"               # rmsnorm | identity | groupnorm
    la_elementwise_affine: bool = True
    la_norm_eps: float = 1e-5
    la_gate_fn: str = "swish"
    la_chunk_size: int = 64
    expand_k: float = 1.0
    expand_v: float = 1.0
    gla_la_gate_logit_normalizer: int = 16
    gla_la_gate_low_rank_dim: int = 16
    gla_la_clamp_min: Optional[float] = None
    rwkv6_la_proj_low_rank_dim: int = 32
    rwkv6_la_gate_low_rank_dim: int = 64
    rwkv7_la_decay_low_rank_dim: int = 64
    rwkv7_la_gate_low_rank_dim: int = 128
    rwkv7_la_a_low_rank_dim: int = 64
    hgrn2_lower_bound: bool = False
    deltanet_qk_activation: str = "silu"
    deltanet_qk_norm: str = "l2"
    gsa_num_slots: int = 64
    use_short_conv: bool = False                  # reference GDN has none; config #3 asks for it
    conv_size: int = 4
    # ---- Mamba2 ---------------------------------------------------------
    mamba_d_state: int = 128
    mamba_head_dim: int = 64
    mamba_ngroups: int = 8
    mamba_expand: int = 2
    mamba_d_conv: int = 4
    mamba_chunk_size: int = 128
    # ---- Mixture of memories -------------------------------------------
    mom_num_memories: int = 4
    mom_topk: int = 2
    mom_capacity: float = 1.0
    mom_shared_mem: bool = True
    # ---- MoE ------------------------------------------------------------
    num_experts: Optional[int] = None
    moe_topk: int = 2
    moe_ffn_hidden_size: Optional[int] = None
    shared_moe_ffn_hidden_size: Optional[int] = None
    enable_shared_expert: bool = False
    shared_expert_gate: bool = True               # qwen2: sigmoid gate; deepseek: none
    num_shared_experts: Optional[int] = None
    moe_layer_freq: int = 1                       # deepseek: layers < freq are dense
    expert_interval: int = 1
    moe_router_order: Optional[str] = None        # softmax_topk | topk_softmax (None → by family)
    moe_router_load_balancing_type: str = "aux_loss"  # aux_loss | sinkhorn | none
    moe_aux_loss_coeff: float = 0.0
    moe_z_loss_coeff: float = 0.0
    moe_input_jitter_eps: Optional[float] = None
    moe_token_dropping: bool = False
    moe_train_capacity_factor: Optional[float] = None
    moe_eval_capacity_factor: Optional[float] = None
    moe_min_capacity: int = 4
    moe_pad_expert_input_to_capacity: bool = False
    moe_token_drop_policy: str = "probs"          # probs | position
    moe_token_dispatcher_type: str = "alltoall"   # alltoall | allgather
    moe_grouped_gemm: bool = True
    moe_layer_recompute: bool = False
    # ---- MLA (deepseek_v2) ---------------------------------------------
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    # ---- precision / memory --------------------------------------------
    params_dtype: torch.dtype = torch.float32
    fp8: Optional[str] = None                     # None | "rowwise": e4m3 GEMMs, one current-amax scale per operand row (ops/fp8.py)
    recompute_granularity: Optional[str] = None   # None | selective | full
    recompute_method: Optional[str] = None        # uniform | block
    recompute_num_layers: int = 1
    cpu_offloading: bool = False                  # activations of the first cpu_offloading_num_layers blocks go to pinned host memory
    cpu_offloading_num_layers: int = 0
    cross_entropy_chunk: int = 4096               # tokens per fused LM-head+CE chunk
    test_mode: bool = False

    def __post_init__(self):
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.base_model not in BASE_MODELS:
            raise ValueError(f"unknown base model {self.base_model!r}")
        if self.la_module is not None and self.la_module not in LA_MODULES:
            raise ValueError(f"unknown --la-module {self.la_module!r}")
        if (self.enable_shared_expert and self.shared_moe_ffn_hidden_size is None and self.num_shared_experts
                and self.moe_ffn_hidden_size):
            # DeepSeek-V2 counts shared experts: their fused width is the count times the routed experts' width
            self.shared_moe_ffn_hidden_size = self.num_shared_experts * self.moe_ffn_hidden_size
        if self.attention_dropout and self.attention_dropout > 0.0:
            raise ValueError("--attention-dropout > 0 is not available: the attention kernels never materialise the "
                             "probabilities it would act on (the reference's launchers train with 0.0); use --hidden-dropout")
        if self.moe_router_order is None:
            # Qwen2/DeepSeek: softmax then top-k (qwen2/moe/router.py:70-71);
            # Mixtral/Llama3: top-k then softmax (mixtral/moe/router.py:159-160).
            self.moe_router_order = (
                "softmax_topk" if self.base_model in ("qwen2", "deepseek_v2") else "topk_softmax")
        if self.num_experts is not None and self.moe_ffn_hidden_size is None:
            self.moe_ffn_hidden_size = self.ffn_hidden_size
        if self.base_model == "deepseek_v2":
            self.shared_expert_gate = False

    # -- derived ----------------------------------------------------------
    @property
    def is_moe(self) -> bool:
        return self.num_experts is not None and self.num_experts > 0

    @property
    def key_dim(self) -> int:
        return int(self.hidden_size * self.expand_k)

    @property
    def value_dim(self) -> int:
        return int(self.hidden_size * self.expand_v)

    def layer_types(self) -> List[str]:
        """Explicit per-layer token-mixer list.

        'L' = linear (LSM) layer, 'N' = softmax attention layer
        (hybrid_transformer_block.py:144-165); for Mamba stacks 'M' = Mamba2
        mixer, '*' = softmax attention, '-' = MLP/MoE (ssm.py:117-157).
        """
        from ..models.layout import expand_layer_pattern
        return expand_layer_pattern(self)

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)


@dataclass
class ParallelConfig:
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1                # LASP-2 / AG-KV sequence-parallel axis
    expert_model_parallel_size: int = 1
    sequence_parallel: bool = False               # Megatron-style SP inside TP regions
    use_distributed_optimizer: bool = False
    overlap_grad_reduce: bool = False             # bucketed gradient reduce-scatter during backward (bitwise equal; off as in Megatron)
    overlap_param_gather: bool = False            # accepted; the parameter all-gather is part of the fused Adam + broadcast kernel
    distributed_backend: str = "nccl"
    distributed_timeout_minutes: int = 10
    fused_comm: bool = True                       # P2P/NVLS kernels instead of NCCL where available
    fused_comm_timeout_s: float = 20.0            # how long a fused kernel waits for a peer before it reports a timeout

    @property
    def tp(self): return self.tensor_model_parallel_size
    @property
    def pp(self): return self.pipeline_model_parallel_size
    @property
    def cp(self): return self.context_parallel_size
    @property
    def ep(self): return self.expert_model_parallel_size


@dataclass
class TrainConfig:
    micro_batch_size: int = 1
    global_batch_size: int = 1
    seq_length: int = 2048
    train_iters: int = 10
    lr: float = 1e-4
    min_lr: float = 1e-5
    lr_decay_style: str = "cosine"                # constant | linear | cosine | inverse-square-root
    lr_decay_iters: Optional[int] = None
    lr_warmup_iters: int = 0
    lr_warmup_init: float = 0.0
    weight_decay: float = 0.1
    start_weight_decay: Optional[float] = None
    end_weight_decay: Optional[float] = None
    weight_decay_incr_style: str = "constant"
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    bf16: bool = False
    fp16: bool = False
    loss_scale: Optional[float] = None
    initial_loss_scale: float = 2.0 ** 32
    min_loss_scale: float = 1.0
    loss_scale_window: int = 1000
    hysteresis: int = 2
    seed: int = 1234
    log_interval: int = 10
    eval_interval: int = 100000
    eval_iters: int = 10
    save_interval: Optional[int] = None
    save: Optional[str] = None
    load: Optional[str] = None
    pretrained_checkpoint: Optional[str] = None
    no_load_optim: bool = False
    no_load_rng: bool = False
    no_save_optim: bool = False
    no_save_rng: bool = False
    async_save: bool = False
    use_dist_ckpt: bool = False                   # sharded checkpoint format with reshard-on-load (ckpt/sharded.py)
    auto_detect_ckpt_format: bool = False         # on load, take whichever format the directory holds
    tensorboard_dir: Optional[str] = None
    tensorboard_log_interval: int = 10
    tensorboard_queue_size: int = 1000
    log_timers_to_tensorboard: bool = False
    log_memory_to_tensorboard: bool = False
    log_validation_ppl_to_tensorboard: bool = False
    timing_log_level: int = 0
    barrier_with_L1_time: bool = True
    exit_interval: Optional[int] = None
    exit_duration_in_mins: Optional[float] = None
    optimizer: str = "adam"                       # adam | sgd
    sgd_momentum: float = 0.9
    eod_token: Optional[int] = None               # the tokenizer's end-of-document id, for --eod-mask-loss
    moe_per_layer_logging: bool = False           # the auxiliary losses of every MoE layer in the log line and TensorBoard
    rampup_batch_size: Optional[Tuple[int, int, int]] = None     # --rampup-batch-size start increment ramp-up-samples
    override_opt_param_scheduler: bool = False
    use_checkpoint_opt_param_scheduler: bool = False
    finetune: bool = False                        # --finetune: weights only, iteration and sample counters start at 0
    exit_on_missing_checkpoint: bool = False
    skip_train: bool = False
    empty_unused_memory_level: int = 0
    adlr_autoresume: bool = False                 # --adlr-autoresume: ask the scheduler's auto-resume service every interval
    adlr_autoresume_interval: int = 1000
    manual_gc: bool = False                       # --manual-gc: Python's collector off, collected by hand every manual_gc_interval steps
    manual_gc_interval: int = 0                   # 0 = only at evaluation / checkpoint time
    exit_signal_handler: bool = False
    check_for_nan_in_loss_and_grad: bool = True
    profile: bool = False
    profile_step_start: int = 10
    profile_step_end: int = 12
    profile_ranks: List[int] = field(default_factory=lambda: [0])
    dataset: str = "Synthetic"                    # Synthetic | LLama-Pretrain-Idxmap | LLama-Pretrain-Raw | LLama-SFT
    data_path: Optional[List[str]] = None
    train_data: Optional[List[str]] = None
    valid_data: Optional[List[str]] = None
    split: str = "99,1,0"
    max_padding_length: Optional[int] = None
    num_workers: int = 0
    epochs: Optional[int] = None
    keep_last: bool = False
    eod_mask_loss: bool = False
    heartbeat_interval_s: float = 0.0             # >0 starts the host watchdog
    heartbeat_timeout_s: float = 60.0

"""Named model presets.

The reference encodes model sizes as shell ``if`` blocks in its launchers
(examples/linear_moe_qwen2/run_pretrain_qwen.sh:126-290,
examples/linear_moe_llama3/run_pretrain_mcore_llama.sh:136-179,
examples/linear_moe_mixtral/run_pretrain_mistral.sh:140-168,
examples/linear_moe_deepseek_v2/run_pretrain_deepseek.sh:136-209).  Here they are
plain dictionaries of :class:`ModelConfig` overrides, plus the five benchmark
configurations this framework is measured on.
"""
from __future__ import annotations

from typing import Dict

import torch

from .model_config import ModelConfig

_QWEN2 = dict(base_model="qwen2", add_qkv_bias=True, norm_eps=1e-6, rotary_base=1e6, swiglu=True)
_LLAMA3 = dict(base_model="llama3", norm_eps=1e-5, rotary_base=5e5, swiglu=True)
_MIXTRAL = dict(base_model="mixtral", norm_eps=1e-5, rotary_base=1e6, swiglu=True, sliding_window=4096,
                init_method_std=0.006)
_DSV2 = dict(base_model="deepseek_v2", norm_eps=1e-6, rotary_base=1e4, swiglu=True, rotary_scaling_factor=40,
             kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)

PRESETS: Dict[str, dict] = {
    # ---- Qwen2 ----------------------------------------------------------
    "qwen2-0.5B": dict(_QWEN2, num_layers=24, hidden_size=512, num_attention_heads=16, ffn_hidden_size=4864,
                       vocab_size=151936),
    "qwen2-0.5Boriginal": dict(_QWEN2, num_layers=24, hidden_size=896, num_attention_heads=14, num_query_groups=2,
                               ffn_hidden_size=4864, vocab_size=151936),
    "qwen2-1.5B": dict(_QWEN2, num_layers=28, hidden_size=1536, num_attention_heads=12, num_query_groups=2,
                       ffn_hidden_size=8960, vocab_size=151936),
    "qwen2-7B": dict(_QWEN2, num_layers=28, hidden_size=3584, num_attention_heads=28, num_query_groups=4,
                     ffn_hidden_size=18944, vocab_size=152064),
    "qwen2-72B": dict(_QWEN2, num_layers=80, hidden_size=8192, num_attention_heads=64, num_query_groups=8,
                      ffn_hidden_size=29568, vocab_size=152064),
    "qwen2-A0.3B": dict(_QWEN2, num_layers=12, hidden_size=1024, num_attention_heads=8, ffn_hidden_size=896,
                        num_experts=64, moe_topk=8, moe_ffn_hidden_size=896, rotary_base=1e4, vocab_size=151936),
    "qwen2-A1B": dict(_QWEN2, num_layers=16, hidden_size=2048, num_attention_heads=16, ffn_hidden_size=1024,
                      num_experts=64, moe_topk=8, moe_ffn_hidden_size=1024, vocab_size=151936),
    "qwen2-A14B": dict(_QWEN2, num_layers=28, hidden_size=3584, num_attention_heads=28, num_query_groups=4,
                       ffn_hidden_size=18944, num_experts=64, moe_topk=8, moe_ffn_hidden_size=2560,
                       shared_moe_ffn_hidden_size=20480, enable_shared_expert=True, vocab_size=152064),
    # ---- Llama3 ---------------------------------------------------------
    "llama3-0.3B": dict(_LLAMA3, num_layers=12, hidden_size=1024, num_attention_heads=32, num_query_groups=8,
                        ffn_hidden_size=4096, vocab_size=128256),
    "llama3-1B": dict(_LLAMA3, num_layers=16, hidden_size=2048, num_attention_heads=32, num_query_groups=8,
                      ffn_hidden_size=8192, vocab_size=128256),
    "llama3-8B": dict(_LLAMA3, num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8,
                      ffn_hidden_size=14336, vocab_size=128256),
    # ---- Mixtral --------------------------------------------------------
    "mixtral-Small": dict(_MIXTRAL, num_layers=8, hidden_size=1024, num_attention_heads=8, num_query_groups=8,
                          ffn_hidden_size=14336, num_experts=8, moe_topk=2, moe_aux_loss_coeff=1e-2,
                          vocab_size=32000),
    "mixtral-8x7B": dict(_MIXTRAL, num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8,
                         ffn_hidden_size=14336, num_experts=8, moe_topk=2, moe_aux_loss_coeff=1e-2,
                         vocab_size=32000),
    # ---- DeepSeek-V2 ----------------------------------------------------
    "deepseek_v2-A2.4B": dict(_DSV2, num_layers=27, hidden_size=2048, num_attention_heads=16,
                              ffn_hidden_size=10944, num_experts=64, moe_topk=6, moe_ffn_hidden_size=1408,
                              enable_shared_expert=True, num_shared_experts=2, shared_moe_ffn_hidden_size=2816,
                              moe_layer_freq=1, vocab_size=102400),
    "deepseek_v2-A21B": dict(_DSV2, num_layers=60, hidden_size=5120, num_attention_heads=128,
                             ffn_hidden_size=12288, num_experts=160, moe_topk=6, moe_ffn_hidden_size=1536,
                             enable_shared_expert=True, num_shared_experts=2, shared_moe_ffn_hidden_size=3072,
                             q_lora_rank=1536, moe_layer_freq=1, vocab_size=102400),
    # ---- benchmark configurations --------------------------------------
    # 1: CPU plumbing (gloo, world 2, fp32)
    "bench-cpu-plumbing": dict(base_model="qwen2", num_layers=2, hidden_size=256, num_attention_heads=4,
                               kv_channels=64, ffn_hidden_size=512, num_experts=4, moe_topk=2,
                               moe_ffn_hidden_size=512, vocab_size=32000, use_la_module=True,
                               la_module="linear_attention", la_feature_map="elu", layer_type_list="LL",
                               init_method_std=0.02, position_embedding_type="none"),
    # 2: A0.3B-2B, 16 x GLA, EP=8
    "bench-a0.3b-2b-gla": dict(_QWEN2, num_layers=16, hidden_size=1024, num_attention_heads=8, kv_channels=128,
                               ffn_hidden_size=896, num_experts=64, moe_topk=8, moe_ffn_hidden_size=896,
                               enable_shared_expert=True, shared_moe_ffn_hidden_size=3584, vocab_size=151936,
                               use_la_module=True, la_module="gla", layer_type_list="L" * 16,
                               init_method_std=0.02, params_dtype=torch.bfloat16),
    # 3: A1B-7B hybrid LLLN x 6 (Gated DeltaNet + GQA flash attention), TP=2 EP=4
    "bench-a1b-7b-hybrid": dict(_QWEN2, num_layers=24, hidden_size=2048, num_attention_heads=16,
                                num_query_groups=4, kv_channels=128, ffn_hidden_size=1408, num_experts=64,
                                moe_topk=8, moe_ffn_hidden_size=1408, vocab_size=151936, use_la_module=True,
                                la_module="gated_deltanet", layer_type_list="LLLN" * 6, use_short_conv=True,
                                conv_size=4, init_method_std=0.02, params_dtype=torch.bfloat16),
    # 4: LASP-2 Linear-Llama3-1B dense, lightning attention, SP=8, seq 131072
    "bench-lasp2-llama3-1b": dict(_LLAMA3, num_layers=16, hidden_size=2048, num_attention_heads=16,
                                  kv_channels=128, ffn_hidden_size=8192, vocab_size=128256, use_la_module=True,
                                  la_module="lightning_attention", layer_type_list="L" * 16,
                                  init_method_std=0.02, max_position_embeddings=131072,
                                  params_dtype=torch.bfloat16),
    # 5: Mixtral-style Mamba2 hybrid, e4m3 GEMMs (one scale per operand row, not 1x128 / 128x128 blocks), TP=2 EP=4 + ZeRO-1
    "bench-mixtral-mamba2-fp8": dict(_MIXTRAL, num_layers=32, hidden_size=4096, num_attention_heads=32,
                                     num_query_groups=8, ffn_hidden_size=14336, num_experts=8, moe_topk=2,
                                     vocab_size=32000, use_la_module=True, la_module="mamba2",
                                     hybrid_override_pattern=("M" * 7 + "*") * 4, mamba_d_state=128,
                                     mamba_head_dim=64, mamba_chunk_size=256, fp8="rowwise",
                                     init_method_std=0.02, params_dtype=torch.bfloat16, sliding_window=None),
}


def get_preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return ModelConfig(**kw)

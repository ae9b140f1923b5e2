"""Convertor parity against real HuggingFace models: a tiny random-init ``transformers`` model is converted with
``hf_to_mcore``, loaded into this framework's ``CausalLM`` and must produce the same logits (what the reference checks
with check_hf_mg_forward, hf2mcore_qwen2_dense_and_moe_gqa.py:765-877).  Catches the GQA packing order, rope layout,
router order / normalisation and shared-expert wiring."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from linear_moe_b200.ckpt import hf_convert
from linear_moe_b200.config.model_config import ModelConfig
from linear_moe_b200.models.transformer import CausalLM


def _load(cfg, hf_model):
    mc = hf_convert.hf_to_mcore({k: v.detach().clone() for k, v in hf_model.state_dict().items()}, cfg)
    ours = CausalLM(cfg)
    own = ours.state_dict()
    missing = [k for k in own if k not in mc and not k.endswith("_extra_state")]
    extra = [k for k in mc if k not in own]
    assert not missing and not extra, (missing[:5], extra[:5])
    ours.load_state_dict(mc, strict=False)
    return ours.eval()


def _per_expert_keys(sd, cfg):
    """The on-disk HF layout (one key per expert matrix, Mixtral under ``block_sparse_moe``) from the stacked in-memory
    layout of transformers >= 5."""
    out = {}
    mixtral = cfg.base_model == "mixtral"
    for k, v in sd.items():
        if k.endswith(".experts.gate_up_proj"):
            base = k[: -len("gate_up_proj")]
            base = base.replace(".mlp.", ".block_sparse_moe.") if mixtral else base
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, 0)
                out[f"{base}{e}.{'w1' if mixtral else 'gate_proj'}.weight"] = g
                out[f"{base}{e}.{'w3' if mixtral else 'up_proj'}.weight"] = u
        elif k.endswith(".experts.down_proj"):
            base = k[: -len("down_proj")]
            base = base.replace(".mlp.", ".block_sparse_moe.") if mixtral else base
            for e in range(v.shape[0]):
                out[f"{base}{e}.{'w2' if mixtral else 'down_proj'}.weight"] = v[e]
        elif mixtral and k.endswith(".mlp.gate.weight"):
            out[k.replace(".mlp.", ".block_sparse_moe.")] = v
        else:
            out[k] = v
    return out


def _check(cfg, hf_model, vocab):
    torch.manual_seed(1)
    ids = torch.randint(0, vocab, (2, 24))
    ours = _load(cfg, hf_model.eval())
    diff = hf_convert.check_hf_mg_forward(hf_model, ours, ids)
    assert diff < 1e-4, diff
    # and back: MCore -> HF reproduces the HF state dict
    back = hf_convert.mcore_to_hf(ours.state_dict(), cfg)
    ref = _per_expert_keys(hf_model.state_dict(), cfg)
    assert set(back) == set(ref), sorted(set(back) ^ set(ref))[:6]
    for k, v in back.items():
        assert torch.equal(v, ref[k]), k


def test_llama_parity():
    hc = transformers.LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                  rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(hc)
    cfg = ModelConfig(base_model="llama3", num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                      ffn_hidden_size=112, vocab_size=320, norm_eps=1e-5, rotary_base=10000.0, max_position_embeddings=128)
    _check(cfg, hf, 320)


def test_qwen2_moe_parity():
    hc = transformers.Qwen2MoeConfig(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                     num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                     rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False,
                                     decoder_sparse_step=1, moe_intermediate_size=48, shared_expert_intermediate_size=96,
                                     num_experts_per_tok=2, num_experts=4, norm_topk_prob=False, mlp_only_layers=[],
                                     use_sliding_window=False)
    torch.manual_seed(0)
    hf = transformers.Qwen2MoeForCausalLM(hc)
    cfg = ModelConfig(base_model="qwen2", num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                      ffn_hidden_size=112, vocab_size=320, norm_eps=1e-6, rotary_base=10000.0, add_qkv_bias=True,
                      num_experts=4, moe_topk=2, moe_ffn_hidden_size=48, enable_shared_expert=True,
                      shared_moe_ffn_hidden_size=96, max_position_embeddings=128)
    _check(cfg, hf, 320)


def test_mixtral_parity():
    hc = transformers.MixtralConfig(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                    rms_norm_eps=1e-5, rope_theta=10000.0, num_local_experts=4, num_experts_per_tok=2,
                                    sliding_window=None, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.MixtralForCausalLM(hc)
    cfg = ModelConfig(base_model="mixtral", num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                      ffn_hidden_size=96, vocab_size=320, norm_eps=1e-5, rotary_base=10000.0, num_experts=4, moe_topk=2,
                      moe_ffn_hidden_size=96, max_position_embeddings=128)
    _check(cfg, hf, 320)


def test_deepseek_v2_parity():
    if not hasattr(transformers, "DeepseekV2ForCausalLM"):
        pytest.skip("transformers build without DeepseekV2")
    hc = transformers.DeepseekV2Config(vocab_size=320, hidden_size=64, intermediate_size=112, moe_intermediate_size=48,
                                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                                       n_shared_experts=2, n_routed_experts=4, num_experts_per_tok=2, first_k_dense_replace=1,
                                       kv_lora_rank=32, q_lora_rank=None, qk_rope_head_dim=8, qk_nope_head_dim=16,
                                       v_head_dim=16, head_dim=8, max_position_embeddings=128, rms_norm_eps=1e-6,
                                       rope_theta=10000.0, routed_scaling_factor=1.0, topk_method="greedy",
                                       norm_topk_prob=False, n_group=1, topk_group=1, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.DeepseekV2ForCausalLM(hc)
    cfg = ModelConfig(base_model="deepseek_v2", num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=112,
                      vocab_size=320, norm_eps=1e-6, rotary_base=10000.0, num_experts=4, moe_topk=2, moe_ffn_hidden_size=48,
                      enable_shared_expert=True, num_shared_experts=2, shared_moe_ffn_hidden_size=96, moe_layer_freq=1,
                      kv_lora_rank=32, q_lora_rank=None, qk_rope_head_dim=8, qk_nope_head_dim=16, v_head_dim=16,
                      max_position_embeddings=128)
    _check(cfg, hf, 320)


def test_qwen2_dense_parity():
    """Dense Qwen2 / Qwen1.5 (QKV bias, GQA): the dense branch of the Qwen convertor."""
    hc = transformers.Qwen2Config(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                  rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False, use_sliding_window=False)
    torch.manual_seed(0)
    hf = transformers.Qwen2ForCausalLM(hc)
    with torch.no_grad():                                   # biases are zero at init: make them count
        for n, p in hf.named_parameters():
            if n.endswith("_proj.bias"):
                p.normal_(0, 0.05)
    cfg = ModelConfig(base_model="qwen2", num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                      ffn_hidden_size=112, vocab_size=320, norm_eps=1e-6, rotary_base=10000.0, add_qkv_bias=True,
                      max_position_embeddings=128)
    _check(cfg, hf, 320)


def test_mistral_dense_parity_with_sliding_window():
    """Dense Mistral (the reference's mistral convertor): Llama layout plus a sliding attention window shorter than the
    test sequence."""
    hc = transformers.MistralConfig(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                    rms_norm_eps=1e-5, rope_theta=10000.0, sliding_window=8, tie_word_embeddings=False)
    hc._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = transformers.MistralForCausalLM(hc)
    cfg = ModelConfig(base_model="mixtral", num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                      ffn_hidden_size=112, vocab_size=320, norm_eps=1e-5, rotary_base=10000.0, sliding_window=8,
                      max_position_embeddings=128)
    _check(cfg, hf, 320)

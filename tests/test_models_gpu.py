"""Whole models on the GPU (bf16, CUDA kernels) against the same model on the CPU (fp32, eager definitions)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from linear_moe_b200.config.model_config import ModelConfig
from linear_moe_b200.models.transformer import CausalLM
from linear_moe_b200.ops import cuda as K

BASE = dict(num_layers=2, hidden_size=256, num_attention_heads=2, kv_channels=128, ffn_hidden_size=512, vocab_size=1024,
            init_method_std=0.02)
CASES = {
    "lightning": dict(use_la_module=True, la_module="lightning_attention", layer_type_list="LL"),
    "gla_moe_shared": dict(use_la_module=True, la_module="gla", layer_type_list="LL", num_experts=8, moe_topk=2,
                           moe_ffn_hidden_size=128, enable_shared_expert=True, shared_moe_ffn_hidden_size=256),
    "gdn_conv_hybrid_gqa": dict(use_la_module=True, la_module="gated_deltanet", layer_type_list="LN", use_short_conv=True,
                                num_attention_heads=4, num_query_groups=2, kv_channels=64, num_experts=4, moe_ffn_hidden_size=128),
    "mamba2_mixtral": dict(base_model="mixtral", use_la_module=True, la_module="mamba2", hybrid_override_pattern="M*",
                           mamba_head_dim=64, mamba_d_state=128, mamba_ngroups=2, num_experts=4, moe_ffn_hidden_size=128),
    "retention_basic": dict(use_la_module=True, la_module="retention", layer_type_list="LN"),
    "deepseek_mla": dict(base_model="deepseek_v2", num_experts=4, moe_topk=2, moe_ffn_hidden_size=128, kv_lora_rank=64,
                         qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, moe_layer_freq=1),
}


@pytest.mark.parametrize("name", list(CASES))
def test_gpu_model_matches_cpu_model(name):
    kw = dict(BASE)
    kw.update(CASES[name])
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    ids = torch.randint(0, 1024, (2, 192))
    labels = torch.roll(ids, -1, 1)
    cpu = CausalLM(ModelConfig(**kw))
    gpu = CausalLM(ModelConfig(params_dtype=torch.bfloat16, **kw)).to(dev)      # same seeded CPU init, rounded to bf16
    with torch.no_grad():
        ref = cpu(ids, labels).mean().item()
    K.reset_launch_count()
    loss = gpu(ids.to(dev), labels.to(dev)).mean()
    loss.backward()
    torch.cuda.synchronize()
    assert K.reset_launch_count() > 0, "the CUDA kernel library was not used"
    assert abs(loss.item() - ref) < 5e-2, (loss.item(), ref)
    for n, p in gpu.named_parameters():
        if p.grad is not None:
            assert torch.isfinite(p.grad).all(), n
    from linear_moe_b200.ops import gemm
    gemm.check_error()

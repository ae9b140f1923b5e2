"""HuggingFace <-> Megatron-Core state-dict conversion for the four backbones, plus TP/PP/EP split and merge.

Reference: toolkits/model_checkpoints_convertor/qwen/hf2mcore_qwen2_dense_and_moe_gqa.py:307-441 (name mapping,
QKV interleave by query group ``[ng, q_per_g + 2, hd, h]``, fc1 = cat(gate, up), router / experts / shared expert /
shared-expert gate), :444-739 (split by TP: qkv by group, proj/fc2 by column, fc1 per GLU half, embedding / lm_head
by row; by EP: experts renumbered to local ids; by PP: layers renumbered), :765-877 (``check_hf_mg_forward``);
deepseek/hf2mcore_deepseek_v2_moe.py:219-260 (MLA names); mistral/hf2mcore_mixtral.py (Mixtral
``block_sparse_moe``); llama/hf2mcore.py (Llama).

Everything here works on plain ``dict[str, Tensor]`` objects, so it runs on CPU without the model classes; the
functions are pure and are round-trip tested (HF -> MCore -> HF is the identity).
The MCore side uses this framework's parameter names, which follow the Megatron-Core schema (``ckpt.legacy``
translates grouped expert tensors to ``local_experts.{e}`` keys on disk).
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional

import torch

from ..config.model_config import ModelConfig

SD = Dict[str, torch.Tensor]


# ---- attention packing -------------------------------------------------------
def pack_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_groups: int, head_dim: int) -> torch.Tensor:
    """HF q ``[H*hd, h]``, k/v ``[G*hd, h]`` (or biases ``[H*hd]``) -> Megatron rows grouped per query group:
    for each group its q heads, then its k head, then its v head."""
    tail = q.shape[1:]
    qg = q.reshape(num_groups, -1, *tail)
    kg = k.reshape(num_groups, head_dim, *tail)
    vg = v.reshape(num_groups, head_dim, *tail)
    return torch.cat([qg, kg, vg], dim=1).reshape(-1, *tail).contiguous()


def unpack_qkv(qkv: torch.Tensor, num_heads: int, num_groups: int, head_dim: int):
    tail = qkv.shape[1:]
    qpg = num_heads // num_groups
    g = qkv.reshape(num_groups, (qpg + 2) * head_dim, *tail)
    q = g[:, : qpg * head_dim].reshape(-1, *tail)
    k = g[:, qpg * head_dim:(qpg + 1) * head_dim].reshape(-1, *tail)
    v = g[:, (qpg + 1) * head_dim:].reshape(-1, *tail)
    return q.contiguous(), k.contiguous(), v.contiguous()


# ---- name tables ----------------------------------------------------------------
def _hf_layer_prefix(i: int) -> str:
    return f"model.layers.{i}."


def hf_to_mcore(hf: SD, cfg: ModelConfig) -> SD:
    """Full (unsharded) HF state dict -> full MCore state dict of a softmax-attention backbone."""
    out: SD = {}
    H, G, hd = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
    fam = cfg.base_model
    out["embedding.word_embeddings.weight"] = hf["model.embed_tokens.weight"]
    for i in range(cfg.num_layers):
        p, m = _hf_layer_prefix(i), f"decoder.layers.{i}."
        out[m + "input_layernorm.weight"] = hf[p + "input_layernorm.weight"]
        out[m + "pre_mlp_layernorm.weight"] = hf[p + "post_attention_layernorm.weight"]
        a = p + "self_attn."
        if fam == "deepseek_v2":
            if cfg.q_lora_rank is None:
                out[m + "self_attention.linear_q_proj.weight"] = hf[a + "q_proj.weight"]
            else:
                out[m + "self_attention.linear_q_a_proj.weight"] = hf[a + "q_a_proj.weight"]
                out[m + "self_attention.q_a_layernorm.weight"] = hf[a + "q_a_layernorm.weight"]
                out[m + "self_attention.linear_q_b_proj.weight"] = hf[a + "q_b_proj.weight"]
            out[m + "self_attention.linear_kv_a_proj_with_mqa.weight"] = hf[a + "kv_a_proj_with_mqa.weight"]
            out[m + "self_attention.kv_a_layernorm.weight"] = hf[a + "kv_a_layernorm.weight"]
            out[m + "self_attention.linear_kv_b_proj.weight"] = hf[a + "kv_b_proj.weight"]
        else:
            out[m + "self_attention.linear_qkv.weight"] = pack_qkv(hf[a + "q_proj.weight"], hf[a + "k_proj.weight"],
                                                                   hf[a + "v_proj.weight"], G, hd)
            if a + "q_proj.bias" in hf:
                out[m + "self_attention.linear_qkv.bias"] = pack_qkv(hf[a + "q_proj.bias"], hf[a + "k_proj.bias"],
                                                                     hf[a + "v_proj.bias"], G, hd)
        out[m + "self_attention.linear_proj.weight"] = hf[a + "o_proj.weight"]
        moe_here = cfg.is_moe and (fam != "deepseek_v2" or i >= cfg.moe_layer_freq)
        if not moe_here:
            x = p + "mlp."
            out[m + "mlp.linear_fc1.weight"] = torch.cat([hf[x + "gate_proj.weight"], hf[x + "up_proj.weight"]], 0)
            out[m + "mlp.linear_fc2.weight"] = hf[x + "down_proj.weight"]
            continue
        x = p + ("block_sparse_moe." if (fam == "mixtral" and p + "block_sparse_moe.gate.weight" in hf) else "mlp.")
        out[m + "mlp.router.weight"] = hf[x + "gate.weight"]
        if x + "experts.gate_up_proj" in hf:
            # in-memory layout of transformers >= 5: experts stacked as gate_up_proj [E, 2f, h], down_proj [E, h, f]
            w1 = list(hf[x + "experts.gate_up_proj"].transpose(1, 2))
            w2 = list(hf[x + "experts.down_proj"].transpose(1, 2))
        elif fam == "mixtral":
            w1 = [torch.cat([hf[f"{x}experts.{e}.w1.weight"], hf[f"{x}experts.{e}.w3.weight"]], 0).t() for e in range(cfg.num_experts)]
            w2 = [hf[f"{x}experts.{e}.w2.weight"].t() for e in range(cfg.num_experts)]
        else:
            w1 = [torch.cat([hf[f"{x}experts.{e}.gate_proj.weight"], hf[f"{x}experts.{e}.up_proj.weight"]], 0).t()
                  for e in range(cfg.num_experts)]
            w2 = [hf[f"{x}experts.{e}.down_proj.weight"].t() for e in range(cfg.num_experts)]
        if fam != "mixtral":
            sh = "shared_expert." if fam == "qwen2" else "shared_experts."
            if x + sh + "gate_proj.weight" in hf:
                out[m + "mlp.shared_expert.linear_fc1.weight"] = torch.cat([hf[x + sh + "gate_proj.weight"],
                                                                            hf[x + sh + "up_proj.weight"]], 0)
                out[m + "mlp.shared_expert.linear_fc2.weight"] = hf[x + sh + "down_proj.weight"]
            if x + "shared_expert_gate.weight" in hf:
                out[m + "mlp.shared_expert_gate.weight"] = hf[x + "shared_expert_gate.weight"]
        out[m + "mlp.experts.weight1"] = torch.stack(w1).contiguous()       # [E, h, 2f]
        out[m + "mlp.experts.weight2"] = torch.stack(w2).contiguous()       # [E, f, h]
    out["decoder.final_layernorm.weight"] = hf["model.norm.weight"]
    if not cfg.tie_embeddings:
        out["output_layer.weight"] = hf.get("lm_head.weight", hf["model.embed_tokens.weight"])
    return out


def mcore_to_hf(mc: SD, cfg: ModelConfig) -> SD:
    out: SD = {}
    H, G, hd = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
    fam = cfg.base_model
    out["model.embed_tokens.weight"] = mc["embedding.word_embeddings.weight"]
    for i in range(cfg.num_layers):
        p, m = _hf_layer_prefix(i), f"decoder.layers.{i}."
        out[p + "input_layernorm.weight"] = mc[m + "input_layernorm.weight"]
        out[p + "post_attention_layernorm.weight"] = mc[m + "pre_mlp_layernorm.weight"]
        a = p + "self_attn."
        if fam == "deepseek_v2":
            if cfg.q_lora_rank is None:
                out[a + "q_proj.weight"] = mc[m + "self_attention.linear_q_proj.weight"]
            else:
                out[a + "q_a_proj.weight"] = mc[m + "self_attention.linear_q_a_proj.weight"]
                out[a + "q_a_layernorm.weight"] = mc[m + "self_attention.q_a_layernorm.weight"]
                out[a + "q_b_proj.weight"] = mc[m + "self_attention.linear_q_b_proj.weight"]
            out[a + "kv_a_proj_with_mqa.weight"] = mc[m + "self_attention.linear_kv_a_proj_with_mqa.weight"]
            out[a + "kv_a_layernorm.weight"] = mc[m + "self_attention.kv_a_layernorm.weight"]
            out[a + "kv_b_proj.weight"] = mc[m + "self_attention.linear_kv_b_proj.weight"]
        else:
            q, k, v = unpack_qkv(mc[m + "self_attention.linear_qkv.weight"], H, G, hd)
            out[a + "q_proj.weight"], out[a + "k_proj.weight"], out[a + "v_proj.weight"] = q, k, v
            if m + "self_attention.linear_qkv.bias" in mc:
                qb, kb, vb = unpack_qkv(mc[m + "self_attention.linear_qkv.bias"], H, G, hd)
                out[a + "q_proj.bias"], out[a + "k_proj.bias"], out[a + "v_proj.bias"] = qb, kb, vb
        out[a + "o_proj.weight"] = mc[m + "self_attention.linear_proj.weight"]
        if m + "mlp.linear_fc1.weight" in mc:
            x = p + "mlp."
            g, u = mc[m + "mlp.linear_fc1.weight"].chunk(2, 0)
            out[x + "gate_proj.weight"], out[x + "up_proj.weight"] = g.contiguous(), u.contiguous()
            out[x + "down_proj.weight"] = mc[m + "mlp.linear_fc2.weight"]
            continue
        w1, w2 = mc[m + "mlp.experts.weight1"], mc[m + "mlp.experts.weight2"]
        if fam == "mixtral":
            x = p + "block_sparse_moe."
            out[x + "gate.weight"] = mc[m + "mlp.router.weight"]
            for e in range(w1.shape[0]):
                g, u = w1[e].t().chunk(2, 0)
                out[f"{x}experts.{e}.w1.weight"], out[f"{x}experts.{e}.w3.weight"] = g.contiguous(), u.contiguous()
                out[f"{x}experts.{e}.w2.weight"] = w2[e].t().contiguous()
        else:
            x = p + "mlp."
            out[x + "gate.weight"] = mc[m + "mlp.router.weight"]
            for e in range(w1.shape[0]):
                g, u = w1[e].t().chunk(2, 0)
                out[f"{x}experts.{e}.gate_proj.weight"], out[f"{x}experts.{e}.up_proj.weight"] = g.contiguous(), u.contiguous()
                out[f"{x}experts.{e}.down_proj.weight"] = w2[e].t().contiguous()
            sh = "shared_expert." if fam == "qwen2" else "shared_experts."
            if m + "mlp.shared_expert.linear_fc1.weight" in mc:
                g, u = mc[m + "mlp.shared_expert.linear_fc1.weight"].chunk(2, 0)
                out[x + sh + "gate_proj.weight"], out[x + sh + "up_proj.weight"] = g.contiguous(), u.contiguous()
                out[x + sh + "down_proj.weight"] = mc[m + "mlp.shared_expert.linear_fc2.weight"]
            if m + "mlp.shared_expert_gate.weight" in mc:
                out[x + "shared_expert_gate.weight"] = mc[m + "mlp.shared_expert_gate.weight"]
    out["model.norm.weight"] = mc["decoder.final_layernorm.weight"]
    if "output_layer.weight" in mc:
        out["lm_head.weight"] = mc["output_layer.weight"]
    return out


@torch.no_grad()
def check_hf_mg_forward(hf_model, our_model, input_ids: torch.Tensor, eps: float = 1e-5) -> float:
    """Max abs difference of the logits of a HuggingFace model and the converted model on the same ids
    (hf2mcore_qwen2_dense_and_moe_gqa.py:765-877)."""
    a = hf_model(input_ids=input_ids).logits.float()
    b = our_model(input_ids).float()[..., : a.shape[-1]]
    diff = (a - b).abs().max().item()
    print(f"check_hf_mg_forward: max |logits diff| = {diff:.3e} ({'ok' if diff < max(eps, 1e-3) else 'MISMATCH'})")
    return diff

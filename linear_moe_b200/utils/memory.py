"""Analytic parameter / memory / FLOP estimators.

``compute_weight_and_optimizer_memory`` follows the reference's accounting
(linear_moe/utils.py:22-131): attention + (MoE or dense) FFN + norms per layer, embeddings, total
versus *activated* parameters (top-k experts only), the most-loaded (TP, PP) shard, and
18 bytes/parameter for mixed-precision Adam or ``6 + 12/DP`` with the distributed optimizer.
Expert parallelism, which the reference's estimate ignores, divides the expert share here.
"""
from __future__ import annotations

from typing import Dict, Iterable

from ..config.model_config import ModelConfig, ParallelConfig


def analytic_parameter_counts(cfg: ModelConfig) -> Dict[str, float]:
    h, L = cfg.hidden_size, cfg.num_layers
    qproj = cfg.kv_channels * cfg.num_attention_heads
    ratio = qproj / h
    E = cfg.num_experts or 1
    glu = 1.5 if cfg.swiglu else 1.0
    inter = cfg.moe_ffn_hidden_size if cfg.moe_ffn_hidden_size is not None else cfg.ffn_hidden_size
    shared = cfg.shared_moe_ffn_hidden_size or 0
    attn = (1 + cfg.num_query_groups / cfg.num_attention_heads) * ratio
    common = 2 / h + 1 / (L * h)
    expert_total = (inter / h) * E * glu
    expert_act = (inter / h) * (cfg.moe_topk if cfg.is_moe else 1) * glu
    shared_t = (shared / h) * glu
    layers_total = 2 * L * h * h * (attn + expert_total + shared_t + common)
    layers_act = 2 * L * h * h * (attn + expert_act + shared_t + common)
    experts_only = 2 * L * h * h * expert_total if cfg.is_moe else 0.0
    emb = h * cfg.vocab_size
    emb_total = emb if cfg.tie_embeddings else 2 * emb
    return {"transformer": layers_total, "transformer_activated": layers_act, "experts": experts_only,
            "embedding": emb_total, "embedding_one": emb, "total": layers_total + emb_total,
            "activated": layers_act + emb_total}


def compute_weight_and_optimizer_memory(cfg: ModelConfig, par: ParallelConfig, world_size: int = None,
                                        verbose: bool = False) -> float:
    c = analytic_parameter_counts(cfg)
    tp, pp, ep = par.tp, par.pp, par.ep
    dense_layers = c["transformer"] - c["experts"]
    dense_shard = (dense_layers / pp + c["embedding_one"]) / tp
    if not cfg.tie_embeddings and pp == 1:
        dense_shard += c["embedding_one"] / tp
    expert_shard = c["experts"] / ep / pp / tp
    shard = dense_shard + expert_shard
    dp = 1
    if world_size:
        dp = max(world_size // (tp * pp), 1)              # data x context parallel ranks: dense gradients are reduced over them
    edp = max(dp // ep, 1)                                # expert-data-parallel ranks: the only ones that share an expert shard
    # 2 (bf16 weight) + 4 (fp32 gradient) + 12 (fp32 master, two Adam moments); the distributed optimizer shards the 12
    # bytes over the ranks that hold the same parameters: dp for dense parameters, edp for experts
    if par.use_distributed_optimizer:
        mem = dense_shard * (6.0 + 12.0 / dp) + expert_shard * (6.0 + 12.0 / edp)
    else:
        mem = shard * 18.0
    if verbose:
        print(f"Number of parameters in transformer layers in billions: {c['transformer'] / 1e9:.2f}")
        print(f"Number of parameters in embedding layers in billions: {c['embedding'] / 1e9:.2f}")
        print(f"Total number of parameters in billions: {c['total'] / 1e9:.2f}")
        print(f"Act number of parameters in billions: {c['activated'] / 1e9:.2f}")
        print(f"Number of parameters in most loaded shard in billions: {shard / 1e9:.4f}")
        print(f"Theoretical memory footprints: weight and optimizer={mem / 2**20:.2f} MB")
    return mem


def count_parameters(models: Iterable) -> int:
    seen, n = set(), 0
    for m in models:
        for p in m.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                n += p.numel()
    return n


def model_flops_per_token(cfg: ModelConfig, seq_length: int) -> float:
    """Training FLOPs per token: 6 x activated matmul parameters (embedding table excluded, LM head
    included) + the sequence-mixing term (softmax layers: 12*s*h per layer causal-halved; linear layers:
    chunked scan ~ 6*(2*C*d + 2*d*d) per head)."""
    c = analytic_parameter_counts(cfg)
    matmul_params = c["transformer_activated"] + c["embedding_one"]
    flops = 6.0 * matmul_params
    try:
        specs = cfg.layer_types()
    except Exception:
        specs = []
    H, d = cfg.num_attention_heads, cfg.kv_channels
    for s in specs:
        if s.mixer in ("attn", "mla"):
            flops += 6.0 * seq_length * H * d          # fwd 2*2*s*H*d/2 (causal) x3 for fwd+bwd
        elif s.mixer in ("lsm", "mamba"):
            C = cfg.la_chunk_size
            flops += 3.0 * H * 2.0 * (2 * C * d + 2 * d * d)
    return flops

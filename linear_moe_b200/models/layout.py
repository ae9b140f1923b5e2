"""Layer-pattern strings → an explicit per-layer list.

Two pattern languages exist in the reference:

* ``--layer-type-list`` over {L, N}: 'L' builds a linear-sequence-modeling layer,
  'N' a softmax-attention layer, each followed by the MLP/MoE of the same
  transformer layer (hybrid_transformer_block.py:144-165).
* ``--hybrid-override-pattern`` over {M, *, -} for Mamba2 stacks: 'M' Mamba2 mixer,
  '*' softmax attention, '-' MLP/MoE, each a residual block of its own.  By default
  the reference appends an MLP/MoE block after every M or * (ssm.py:138-157);
  ``--megatron-hybrid-mamba-method`` uses the pattern literally (ssm.py:117-137).
  Without an override the pattern comes from target ratios
  (mamba_hybrid_layer_allocation.py:26-62).

Both are expanded here into ``LayerSpec`` entries so that pipeline stages can slice a
heterogeneous list (the reference's hybrid block builds every layer on every stage,
hybrid_transformer_block.py:144-165, which this design does not reproduce).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple


@dataclass(frozen=True)
class LayerSpec:
    mixer: Optional[str]      # 'lsm' | 'attn' | 'mla' | 'mamba' | None
    ffn: Optional[str]        # 'mlp' | 'moe' | None
    symbol: str               # source symbol, for logs and checkpoints
    index: int                # global index in the expanded list


def allocate_mamba_pattern(total: int, attn_ratio: float, mlp_ratio: float,
                           override: Optional[str] = None) -> List[str]:
    """Spread attention ('*') and MLP ('-') blocks evenly among Mamba ('M') blocks."""
    assert total > 0 and 0.0 <= attn_ratio <= 1.0 and 0.0 <= mlp_ratio <= 1.0
    assert attn_ratio + mlp_ratio <= 1.0
    n_attn = round(total * attn_ratio)
    n_mamba = total - n_attn
    section = n_mamba / (n_attn + 1)
    out = ["M"] * total
    x = section
    for i in range(total):
        if x < 0.5:
            out[i] = "*"
            x += section
        else:
            x -= 1
    n_mlp = round(total * mlp_ratio)
    if n_mlp > 0:
        n_mamba -= n_mlp
        ratio = n_mamba / n_mlp
        x = ratio
        for i in range(total):
            if out[i] == "M":
                if x < 0.5:
                    out[i] = "-"
                    x += ratio
                else:
                    x -= 1
    if override is not None:
        ov = list(override)
        if len(ov) != total:
            raise ValueError(f"hybrid override pattern has length {len(ov)}, expected {total}")
        bad = set(ov) - set("M*-")
        if bad:
            raise ValueError(f"invalid symbols in hybrid override pattern: {sorted(bad)}")
        if (attn_ratio > 0.0 or mlp_ratio > 0.0) and any(ov.count(s) != out.count(s) for s in "M*-"):
            raise ValueError("override pattern layer counts do not match the target ratios")
        out = ov
    return out


def _ffn_kind(cfg, layer_idx: int) -> str:
    """MoE or dense MLP for transformer layer ``layer_idx`` (0-based).

    DeepSeek-V2 keeps the first ``moe_layer_freq`` layers dense
    (deepseek_v2/transformer_layer.py:142-145); other families place an MoE every
    ``expert_interval`` layers."""
    if not cfg.is_moe:
        return "mlp"
    if cfg.base_model == "deepseek_v2":
        return "moe" if layer_idx >= cfg.moe_layer_freq else "mlp"
    return "moe" if (layer_idx + 1) % max(cfg.expert_interval, 1) == 0 else "mlp"


def expand_layer_pattern(cfg) -> List[LayerSpec]:
    attn_kind = "mla" if cfg.base_model == "deepseek_v2" else "attn"
    specs: List[Tuple[Optional[str], Optional[str], str]] = []
    if cfg.use_la_module and cfg.la_module == "mamba2":
        pat = allocate_mamba_pattern(cfg.num_layers, cfg.hybrid_attention_ratio, cfg.hybrid_mlp_ratio,
                                     cfg.hybrid_override_pattern)
        tl = 0
        for sym in pat:
            if sym == "M":
                specs.append(("mamba", None, sym))
            elif sym == "*":
                specs.append((attn_kind, None, sym))
            else:
                specs.append((None, _ffn_kind(cfg, tl), sym))
                tl += 1
            if not cfg.megatron_hybrid_mamba_method and sym != "-":
                specs.append((None, _ffn_kind(cfg, tl), "-"))
                tl += 1
    else:
        if cfg.use_la_module and cfg.la_module is not None:
            pat = cfg.layer_type_list or "L" * cfg.num_layers
        else:
            pat = "N" * cfg.num_layers
        if len(pat) != cfg.num_layers:
            raise ValueError(f"--layer-type-list has length {len(pat)}, expected {cfg.num_layers}")
        for i, sym in enumerate(pat):
            if sym == "L":
                specs.append(("lsm", _ffn_kind(cfg, i), sym))
            elif sym == "N":
                specs.append((attn_kind, _ffn_kind(cfg, i), sym))
            else:
                raise ValueError(f"invalid symbol {sym!r} in --layer-type-list")
    return [LayerSpec(m, f, s, i) for i, (m, f, s) in enumerate(specs)]


def split_for_pipeline(specs: List[LayerSpec], pp: int, pp_rank: int, vpp: Optional[int] = None,
                       vpp_rank: int = 0) -> List[LayerSpec]:
    """Contiguous slice of the layer list owned by (pp_rank, vpp_rank).

    Interleaved schedule: the list is cut into ``pp*vpp`` chunks and chunk ``c`` goes to
    stage ``c % pp``, model chunk ``c // pp`` (transformer_block.py:42-74 semantics)."""
    n = len(specs)
    v = vpp or 1
    if n % (pp * v) != 0:
        raise ValueError(f"{n} layers do not divide into pp={pp} x vpp={v} chunks")
    per = n // (pp * v)
    chunk = vpp_rank * pp + pp_rank
    return specs[chunk * per:(chunk + 1) * per]

"""Split a full state dict into (TP, PP, EP) shards and merge shards back: checkpoint resharding.

Rules (reference: hf2mcore_qwen2_dense_and_moe_gqa.py:119-135,564-600 and the ``sharded_state_dict``
implementations in mlp.py:157-230, experts.py:230-273, hybrid_transformer_block.py:434-474):

* norms, router, shared-expert gate, low-rank "a" projections: replicated;
* embedding / LM head / column-parallel weights and biases: split along dim 0 (fused QKV by query group and LSM
  q|k|v by head are contiguous row blocks, so a plain chunk is right);
* SwiGLU fc1: each GLU half split separately; Mamba2 ``in_proj`` / ``conv1d``: each of its parts split separately;
* row-parallel weights (``linear_proj``, ``o_proj``, ``linear_fc2``, ``out_proj``): split along dim 1;
* experts: EP takes contiguous blocks of experts (renumbered locally); within an expert fc1 per GLU half, fc2 by row;
* per-head vectors (``A_log``, ``D``, ``dt_bias``, ``bonus``, Mamba ``norm.weight``): dim 0;
* PP: a stage takes a contiguous block of ``decoder.layers`` renumbered from 0; embedding on the first stage, final
  norm and LM head on the last.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Tuple

import torch

from ..config.model_config import ModelConfig

SD = Dict[str, torch.Tensor]
_LAYER = re.compile(r"^decoder\.layers\.(\d+)\.(.*)$")

_COL = ("linear_qkv.", "qkv_proj.", "o_gate_proj.", "beta_proj.", "a_proj.", "linear_q_proj.", "linear_q_b_proj.",
        "linear_kv_b_proj.", "f_proj.", "shared_qkv_proj.", "shared_beta_proj.", "shared_a_proj.")
_ROW = ("linear_proj.weight", "o_proj.weight", "linear_fc2.weight", "out_proj.weight")
_HEADVEC = ("A_log", "D", "dt_bias", "bonus", "booster", "removal")
_GLA_GATE = re.compile(r"gk_proj\.([01])\.(?:weight|bias)$")
_RNN_ANY = re.compile(r"\.[a-z]_proj\.")
_RNN_ROWS = re.compile(r"\.(?:[qfirkv]_proj\.(?:weight|bias)|[rwkvg]_proj\.linear\.(?:weight|bias)"
                       r"|[rwkvag]_proj\.(?:linear\.)?lora\.2\.(?:weight|bias))$")


def _mamba_parts(cfg: ModelConfig):
    d_inner = cfg.mamba_expand * cfg.hidden_size
    gs = cfg.mamba_ngroups * cfg.mamba_d_state
    return d_inner, gs, d_inner // cfg.mamba_head_dim


def _rule(name: str, cfg: ModelConfig):
    """-> (kind, arg): 'rep' | 'dim0' | 'dim1' | 'parts0' (list of sizes) | 'w1' | 'w2'."""
    if name.endswith("experts.weight1"):
        return "w1", None
    if name.endswith("experts.weight2"):
        return "w2", None
    if name.startswith("embedding.word_embeddings") or name.startswith("output_layer"):
        return "dim0", None
    if "linear_fc1." in name:
        return "glu0", None
    if ".mixer.in_proj." in name:
        d, gs, nh = _mamba_parts(cfg)
        return "parts0", [d, d, gs, gs, nh]
    if ".mixer.conv1d." in name:
        d, gs, _ = _mamba_parts(cfg)
        return "parts0", [d, gs, gs]
    if name.endswith(".mixer.norm.weight") or ".self_attention.conv1d." in name:
        return "dim0", None
    if any(name.endswith(r) for r in _ROW):
        return "dim1", None
    if cfg.la_module in ("hgrn2", "rwkv6", "rwkv7") and ".self_attention." in name and _RNN_ANY.search(name):
        # HGRN2 / RWKV6 / RWKV7 mixers: projections into key / value space keep the rank's heads (rows); of a low-rank
        # pair only the up-projection does; token-shift mixers (x_proj, mu, x) stay whole
        return ("dim0", None) if _RNN_ROWS.search(name) else ("rep", None)
    m = _GLA_GATE.search(name)
    if m:                                   # low-rank GLA gate (also one per MoM memory): only the up-projection is sharded
        return ("dim0", None) if m.group(1) == "1" else ("rep", None)
    if any(c in name for c in _COL) and "linear_q_a_proj" not in name and "kv_a_proj" not in name:
        return "dim0", None
    last = name.rsplit(".", 1)[-1]
    if last in _HEADVEC and (".self_attention." in name or ".mixer." in name) and "core_linear_attention" not in name:
        return "dim0", None
    return "rep", None


def _take(t: torch.Tensor, kind: str, arg, tp: int, r: int) -> torch.Tensor:
    if tp == 1 or kind == "rep":
        return t
    if kind == "dim0":
        return t.chunk(tp, 0)[r].contiguous()
    if kind == "dim1":
        return t.chunk(tp, 1)[r].contiguous()
    if kind == "glu0":
        return torch.cat([h.chunk(tp, 0)[r] for h in t.chunk(2, 0)], 0).contiguous()
    if kind == "parts0":
        return torch.cat([p.chunk(tp, 0)[r] for p in t.split(arg, 0)], 0).contiguous()
    if kind == "w1":                                      # [E, h, 2f]
        return torch.cat([h.chunk(tp, -1)[r] for h in t.chunk(2, -1)], -1).contiguous()
    if kind == "w2":                                      # [E, f, h]
        return t.chunk(tp, 1)[r].contiguous()
    raise ValueError(kind)


def _join(ts: List[torch.Tensor], kind: str, arg, tp: int) -> torch.Tensor:
    if tp == 1 or kind == "rep":
        return ts[0]
    if kind == "dim0":
        return torch.cat(ts, 0)
    if kind == "dim1":
        return torch.cat(ts, 1)
    if kind == "glu0":
        halves = [t.chunk(2, 0) for t in ts]
        return torch.cat([torch.cat([h[0] for h in halves], 0), torch.cat([h[1] for h in halves], 0)], 0)
    if kind == "parts0":
        sizes = [a // tp for a in arg]
        parts = [t.split(sizes, 0) for t in ts]
        return torch.cat([torch.cat([p[i] for p in parts], 0) for i in range(len(arg))], 0)
    if kind == "w1":
        halves = [t.chunk(2, -1) for t in ts]
        return torch.cat([torch.cat([h[0] for h in halves], -1), torch.cat([h[1] for h in halves], -1)], -1)
    if kind == "w2":
        return torch.cat(ts, 1)
    raise ValueError(kind)


def num_layer_entries(full: SD) -> int:
    idx = [int(m.group(1)) for m in (_LAYER.match(k) for k in full) if m]
    return max(idx) + 1 if idx else 0


def shard_state_dict(full: SD, cfg: ModelConfig, tp: int = 1, pp: int = 1, ep: int = 1, tp_rank: int = 0, pp_rank: int = 0,
                     ep_rank: int = 0) -> SD:
    n = num_layer_entries(full)
    assert n % pp == 0, f"{n} layer entries do not divide into {pp} stages"
    per = n // pp
    lo, hi = pp_rank * per, (pp_rank + 1) * per
    out: SD = {}
    for name, t in full.items():
        m = _LAYER.match(name)
        if m:
            i = int(m.group(1))
            if not lo <= i < hi:
                continue
            new = f"decoder.layers.{i - lo}.{m.group(2)}"
        else:
            if name.startswith("embedding.") and pp_rank != 0:
                continue
            if (name.startswith("decoder.final_layernorm") or name.startswith("output_layer")) and pp_rank != pp - 1:
                continue
            new = name
        kind, arg = _rule(name, cfg)
        if kind in ("w1", "w2") and ep > 1:
            E = t.shape[0]
            t = t[ep_rank * (E // ep):(ep_rank + 1) * (E // ep)]
        out[new] = _take(t, kind, arg, tp, tp_rank).clone()
    return out


def merge_state_dicts(shards: Dict[Tuple[int, int, int], SD], cfg: ModelConfig, tp: int = 1, pp: int = 1, ep: int = 1) -> SD:
    """``shards[(tp_rank, pp_rank, ep_rank)]`` -> full state dict."""
    full: SD = {}
    per = num_layer_entries(shards[(0, 0, 0)])
    for p in range(pp):
        names = list(shards[(0, p, 0)].keys())
        for name in names:
            m = _LAYER.match(name)
            gname = f"decoder.layers.{int(m.group(1)) + p * per}.{m.group(2)}" if m else name
            kind, arg = _rule(gname, cfg)
            if kind in ("w1", "w2"):
                per_ep = [_join([shards[(t, p, e)][name] for t in range(tp)], kind, arg, tp) for e in range(ep)]
                full[gname] = torch.cat(per_ep, 0)
            else:
                full[gname] = _join([shards[(t, p, 0)][name] for t in range(tp)], kind, arg, tp)
    return full


def reshard(shards: Dict[Tuple[int, int, int], SD], cfg: ModelConfig, src: Tuple[int, int, int], dst: Tuple[int, int, int]
            ) -> Dict[Tuple[int, int, int], SD]:
    """Convert a checkpoint from a ``(tp, pp, ep)`` layout to another one."""
    full = merge_state_dicts(shards, cfg, *src)
    tp, pp, ep = dst
    return {(t, p, e): shard_state_dict(full, cfg, tp, pp, ep, t, p, e)
            for t in range(tp) for p in range(pp) for e in range(ep)}


def reshard_optimizer_shards(states: List[dict], new_dp: int) -> List[dict]:
    """ZeRO-1 optimizer shards saved for one data-parallel size -> shards for another (elastic restart).  The flat
    buffers are concatenated in rank order and re-cut; padding at the end of a buffer is re-derived."""
    out = [dict(step=states[0]["step"], loss_scale=states[0].get("loss_scale"), zero1=True, buffers=[]) for _ in range(new_dp)]
    for b in range(len(states[0]["buffers"])):
        ref = states[0]["buffers"][b]
        cat = {k: torch.cat([s["buffers"][b][k] for s in states]) for k in ("exp_avg", "exp_avg_sq")}
        master = None if ref["master"] is None else torch.cat([s["buffers"][b]["master"] for s in states])
        used = ref["numel"]
        mult = 128 * new_dp
        numel = (used + mult - 1) // mult * mult
        def fit(t):
            return t[:numel] if t.numel() >= numel else torch.cat([t, t.new_zeros(numel - t.numel())])
        cat = {k: fit(v) for k, v in cat.items()}
        master = None if master is None else fit(master)
        n = numel // new_dp
        for r in range(new_dp):
            out[r]["buffers"].append({"expert": ref["expert"], "weight_decay": ref["weight_decay"],
                                      "shard": (r * n, (r + 1) * n), "numel": numel, "names": ref["names"],
                                      "master": None if master is None else master[r * n:(r + 1) * n].clone(),
                                      "exp_avg": cat["exp_avg"][r * n:(r + 1) * n].clone(),
                                      "exp_avg_sq": cat["exp_avg_sq"][r * n:(r + 1) * n].clone()})
    return out

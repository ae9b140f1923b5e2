"""Softmax attention layers: GQA self-attention with RoPE, and DeepSeek-V2 multi-head latent
attention (MLA) with YaRN.

Reference: model/qwen2/transformer/attention.py:54-342,345-517 (fused QKV with GQA packing,
optional q/k layernorm, RoPE, KV cache, row-parallel projection) and
model/deepseek_v2/transformer/attention.py:42-406 (low-rank q / kv projections, decoupled rope
dims, eager softmax).  The core is ``ops.softmax_attention`` (flash attention on CUDA) instead
of baddbmm + softmax + bmm (sequence_modeling/attention/dot_product_attention.py:139-183).

Under a context-parallel mesh axis the 'N' layers all-gather K and V along the sequence
(cheap under GQA) and run causal attention with the rank's query offset, which the reference
cannot do (dot_product_attention.py:46-48 asserts CP == 1).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..config.model_config import ModelConfig
from ..dist import collectives as C
from ..dist.mesh import Mesh, single_process_mesh
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from ..ref import ops as R


class RotaryCache:
    """cos/sin tables built on demand per (length, offset, device)."""

    def __init__(self, cfg: ModelConfig, dim: int, yarn: bool = False):
        self.cfg, self.dim, self.yarn = cfg, dim, yarn
        self.mscale = 1.0
        self._key, self._val = None, None

    def get(self, T: int, offset: int, device):
        key = (T, offset, str(device))
        if self._key != key:
            cfg = self.cfg
            rot = int(self.dim * cfg.rotary_percent)
            if self.yarn and cfg.rotary_scaling_factor > 1:
                cos, sin, m = R.yarn_freqs(T, rot, cfg.rotary_base, cfg.rotary_scaling_factor, offset=offset,
                                           device=device, mscale=0.707, mscale_all_dim=0.707)
                self.mscale = m
            else:
                cos, sin = R.rope_freqs(T, rot, cfg.rotary_base, offset, device,
                                        cfg.rotary_seq_len_interpolation_factor)
            self._key, self._val = key, (cos, sin)
        return self._val


def _kv_cache_update(cache: Optional[dict], k, v):
    """Append to the KV cache of a softmax layer; returns the full K, V and the query offset."""
    if cache is None:
        return k, v, 0
    if "k" in cache:
        off = cache["k"].shape[1]
        k = torch.cat([cache["k"], k], dim=1)
        v = torch.cat([cache["v"], v], dim=1)
    else:
        off = 0
    cache["k"], cache["v"] = k.detach(), v.detach()
    return k, v, off


class SelfAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        mesh = self.mesh
        H, G, D = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
        assert H % G == 0 and G % mesh.tp == 0, (H, G, mesh.tp)
        self.H, self.G, self.D = H, G, D
        self.Gl, self.qpg = G // mesh.tp, H // G
        dt, std = cfg.params_dtype, cfg.init_method_std
        # rows grouped by query group: [G, (qpg q heads | k | v), D]  (hf2mcore_qwen2_dense_and_moe_gqa.py:380-441)
        self.linear_qkv = ColumnParallelLinear(cfg.hidden_size, G * (self.qpg + 2) * D, mesh=mesh,
                                               bias=cfg.add_bias_linear or cfg.add_qkv_bias, std=std,
                                               key=key + ".linear_qkv", sequence_parallel=sequence_parallel,
                                               dtype=dt, device=device)
        self.linear_proj = RowParallelLinear(H * D, cfg.hidden_size, mesh=mesh, bias=cfg.add_bias_linear,
                                             std=std / math.sqrt(2.0 * cfg.num_layers), key=key + ".linear_proj",
                                             sequence_parallel=sequence_parallel, dtype=dt, device=device)
        if cfg.qk_layernorm:
            self.q_layernorm = nn.Module()
            self.q_layernorm.weight = nn.Parameter(torch.ones(D, dtype=dt, device=device))
            self.k_layernorm = nn.Module()
            self.k_layernorm.weight = nn.Parameter(torch.ones(D, dtype=dt, device=device))
            # shared by all heads, applied to this rank's heads: the optimizer sums the partial gradients over TP
            self.q_layernorm.weight.tp_partial_grad = self.k_layernorm.weight.tp_partial_grad = True
        self.rope = RotaryCache(cfg, D) if cfg.position_embedding_type == "rope" else None

    def forward(self, x, cache: Optional[dict] = None, position_offset: int = 0, **_):
        cfg = self.cfg
        qkv = self.linear_qkv(x)
        B, T = qkv.shape[:2]
        qkv = qkv.reshape(B, T, self.Gl, self.qpg + 2, self.D)
        q = qkv[:, :, :, : self.qpg].reshape(B, T, self.Gl * self.qpg, self.D)
        k, v = qkv[:, :, :, self.qpg], qkv[:, :, :, self.qpg + 1]
        if cfg.qk_layernorm:
            q = ops.rms_norm(q.contiguous(), self.q_layernorm.weight, cfg.norm_eps)
            k = ops.rms_norm(k.contiguous(), self.k_layernorm.weight, cfg.norm_eps)
        cp = self.mesh["cp"]
        past = cache["k"].shape[1] if (cache is not None and "k" in cache) else 0
        # position_offset is the absolute position of this call's first token (the cache length when decoding)
        pos0 = position_offset + (cp.rank * T if not cp.is_trivial else 0)
        if self.rope is not None:
            cos, sin = self.rope.get(T, pos0, x.device)
            q = ops.apply_rope(q.contiguous(), cos, sin, cfg.rotary_interleaved)
            k = ops.apply_rope(k.contiguous(), cos, sin, cfg.rotary_interleaved)
        k, v, q_off = _kv_cache_update(cache, k, v)
        if not cp.is_trivial:
            k = C.all_gather(k.contiguous(), cp, dim=1)
            v = C.all_gather(v.contiguous(), cp, dim=1)
            q_off = cp.rank * T
        o = ops.softmax_attention(q.contiguous(), k.contiguous(), v.contiguous(), None, True, q_off, cfg.sliding_window)
        return self.linear_proj(o.reshape(B, T, -1))

    @torch.no_grad()
    def run_realtime_tests(self):
        """Check that the q/k layernorm weights agree across the DP and TP groups
        (attention.py:400-467 ``run_realtime_tests``, enabled by ``test_mode``)."""
        if not self.cfg.qk_layernorm:
            return True
        ok = True
        for gname in ("dp", "tp"):
            g = self.mesh[gname]
            for w in (self.q_layernorm.weight, self.k_layernorm.weight):
                allw = C.all_gather_raw(w.detach()[None].float(), g, dim=0)
                ok = ok and bool((allw - allw[0:1]).abs().max() == 0)
        return ok


class MLASelfAttention(nn.Module):
    """Multi-head latent attention.  The low-rank down-projections are replicated over TP and the
    up-projections are sharded by head (the reference instead scales the low-rank widths with the TP
    size, deepseek_v2/transformer/attention.py:280,293,318)."""

    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        mesh = self.mesh
        H = cfg.num_attention_heads
        assert H % mesh.tp == 0
        self.H, self.Hl = H, H // mesh.tp
        self.dn, self.dr, self.dvh = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.dq = self.dn + self.dr
        dt, std = cfg.params_dtype, cfg.init_method_std
        self.sp = sequence_parallel and mesh.tp > 1
        kw = dict(dtype=dt, device=device)
        from ..parallel.tensor_parallel import init_normal
        if cfg.q_lora_rank is None:
            self.linear_q_proj = ColumnParallelLinear(cfg.hidden_size, H * self.dq, mesh=mesh, std=std,
                                                      key=key + ".linear_q_proj", **kw)
        else:
            self.linear_q_a_proj = nn.Linear(cfg.hidden_size, cfg.q_lora_rank, bias=False, **kw)
            self.q_a_layernorm = nn.Module()
            self.q_a_layernorm.weight = nn.Parameter(torch.ones(cfg.q_lora_rank, **kw))
            self.linear_q_b_proj = ColumnParallelLinear(cfg.q_lora_rank, H * self.dq, mesh=mesh, std=std,
                                                        key=key + ".linear_q_b_proj", **kw)
            with torch.no_grad():
                self.linear_q_a_proj.weight.copy_(init_normal((cfg.q_lora_rank, cfg.hidden_size), std,
                                                              key + ".linear_q_a_proj.weight", device))
        self.linear_kv_a_proj_with_mqa = nn.Linear(cfg.hidden_size, cfg.kv_lora_rank + self.dr, bias=False, **kw)
        with torch.no_grad():
            self.linear_kv_a_proj_with_mqa.weight.copy_(init_normal((cfg.kv_lora_rank + self.dr, cfg.hidden_size), std,
                                                                    key + ".linear_kv_a_proj_with_mqa.weight", device))
        self.kv_a_layernorm = nn.Module()
        self.kv_a_layernorm.weight = nn.Parameter(torch.ones(cfg.kv_lora_rank, **kw))
        self.linear_kv_b_proj = ColumnParallelLinear(cfg.kv_lora_rank, H * (self.dn + self.dvh), mesh=mesh, std=std,
                                                     key=key + ".linear_kv_b_proj", **kw)
        self.linear_proj = RowParallelLinear(H * self.dvh, cfg.hidden_size, mesh=mesh,
                                             std=std / math.sqrt(2.0 * cfg.num_layers), key=key + ".linear_proj",
                                             sequence_parallel=sequence_parallel, **kw)
        self.rope = RotaryCache(cfg, self.dr, yarn=True)
        self.scale = self.dq ** -0.5

    def forward(self, x, cache: Optional[dict] = None, position_offset: int = 0, **_):
        cfg = self.cfg
        tp = self.mesh["tp"]
        if self.sp:
            # every path from x into head-sharded work passes a point that all-reduces its gradient (the column-parallel
            # up-projections, the shared rope key below), so each rank ends up with the complete gradient of the
            # gathered input and the backward of the gather is a slice
            x = C.gather_no_reduce(x, tp, dim=1)
        B, T, _ = x.shape
        if cfg.q_lora_rank is None:
            q = self.linear_q_proj(x)
        else:
            q = self.linear_q_b_proj(ops.rms_norm(self.linear_q_a_proj(x), self.q_a_layernorm.weight, cfg.norm_eps))
        q = q.reshape(B, T, self.Hl, self.dq)
        q_nope, q_pe = q.split([self.dn, self.dr], dim=-1)
        ckv = self.linear_kv_a_proj_with_mqa(x)
        ckv, k_pe = ckv.split([cfg.kv_lora_rank, self.dr], dim=-1)
        kv = self.linear_kv_b_proj(ops.rms_norm(ckv.contiguous(), self.kv_a_layernorm.weight, cfg.norm_eps))
        kv = kv.reshape(B, T, self.Hl, self.dn + self.dvh)
        k_nope, v = kv.split([self.dn, self.dvh], dim=-1)
        cp = self.mesh["cp"]
        past = cache["k"].shape[1] if (cache is not None and "k" in cache) else 0
        # position_offset is the absolute position of this call's first token (the cache length when decoding)
        pos0 = position_offset + (cp.rank * T if not cp.is_trivial else 0)
        cos, sin = self.rope.get(T, pos0, x.device)
        # HF DeepSeek stores the rope dims interleaved; the reference permutes them to half layout
        # before rotating (yarn_rotary_pos_embedding.py:198-202): same as rotating interleaved pairs.
        q_pe = ops.apply_rope(q_pe.contiguous(), cos, sin, True)
        k_pe = ops.apply_rope(k_pe.reshape(B, T, 1, self.dr).contiguous(), cos, sin, True)
        if not tp.is_trivial:
            k_pe = C.copy_to_region(k_pe, tp)       # one rope key for all heads: its gradient is the sum over every rank's heads
        qf = torch.cat([q_nope, q_pe], dim=-1)
        kf = torch.cat([k_nope, k_pe.expand(B, T, self.Hl, self.dr)], dim=-1)
        kf, v, q_off = _kv_cache_update(cache, kf, v)
        if not cp.is_trivial:
            kf = C.all_gather(kf.contiguous(), cp, dim=1)
            v = C.all_gather(v.contiguous(), cp, dim=1)
            q_off = cp.rank * T
        scale = self.scale * self.rope.mscale * self.rope.mscale
        o = ops.softmax_attention(qf.contiguous(), kf.contiguous(), v.contiguous(), scale, True, q_off, None)
        return self.linear_proj(o.reshape(B, T, -1))

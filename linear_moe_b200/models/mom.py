"""Mixture-of-Memories (MoM) token mixer.

Reference: sequence_modeling/mom_linear_attention.py:15-120 (``transform``/``reconstruct``),
:132-270 (parameters), :272-421 (forward), :507-609 (shared memory).  A router sends every token
to ``topk`` of ``num_memories`` independent recurrent memories.  For each (batch, memory) the
routed tokens form a subsequence that is left-padded to a fixed capacity (the oldest tokens are
dropped beyond it); each memory has its own q/k/v (and gate) projections; the LSM core runs on
all subsequences at once (batched over memories, not a Python loop over memories as in the
reference :369-410); outputs are scattered back, weighted by the renormalised routing weights and
summed.  An optional shared memory sees every token.  Cores: GLA, Gated DeltaNet, basic LA.

The routing plan is built with vectorised index arithmetic (no sort): a token routed to memory m
lands in slot ``L - count(b,m) + rank(b,t,m)`` of that memory's padded row.

Parallel layouts: heads split over the tensor-parallel ranks (the routing weights' gradient is summed over them);
under sequence parallelism the input is gathered along T at the entry and ``o_proj`` reduce-scatters; under context
parallelism every memory's subsequence continues across the ranks through the LASP-2 state exchange of the core
(padding slots neither decay nor write the state), with the capacity applied per rank slice.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config.model_config import ModelConfig
from ..dist import collectives as C
from ..dist.mesh import Mesh, single_process_mesh
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, init_normal, init_uniform
from .lsm_layers import GLAGate, LSMCore, _tp_slice


def mom_plan(selected: torch.Tensor, num_memories: int, capacity_len: int):
    """selected ``[B,T,k]`` memory ids -> slot ``[B,T,k]`` (-1 = dropped) and gather index
    ``[B,M,L]`` (token position, -1 = padding)."""
    B, T, k = selected.shape
    M, L = num_memories, capacity_len
    onehot = F.one_hot(selected, M).sum(2)                             # [B,T,M] 0/1
    rank = onehot.cumsum(1) - onehot                                   # tokens of this memory before t
    count = onehot.sum(1)                                              # [B,M]
    slot_m = L - count[:, None, :] + rank                              # [B,T,M]
    slot = torch.gather(slot_m, 2, selected)                           # [B,T,k]
    slot = torch.where(slot >= 0, slot, torch.full_like(slot, -1))
    gidx = torch.full((B, M, L), -1, dtype=torch.long, device=selected.device)
    b_ix = torch.arange(B, device=selected.device)[:, None, None].expand(B, T, k)
    t_ix = torch.arange(T, device=selected.device)[None, :, None].expand(B, T, k)
    ok = slot >= 0
    gidx[b_ix[ok], selected[ok], slot[ok]] = t_ix[ok]
    return slot, gidx


def mom_transform(x: torch.Tensor, gidx: torch.Tensor) -> torch.Tensor:
    """x ``[B,T,d]`` -> ``[M,B,L,d]`` with zeros at padding."""
    B, M, L = gidx.shape
    pad = gidx < 0
    g = gidx.clamp(min=0).reshape(B, M * L)
    out = torch.gather(x, 1, g[..., None].expand(B, M * L, x.shape[-1])).reshape(B, M, L, -1)
    out = out.masked_fill(pad[..., None], 0.0)
    return out.permute(1, 0, 2, 3).contiguous()


def mom_reconstruct(o: torch.Tensor, selected: torch.Tensor, slot: torch.Tensor, weights: torch.Tensor):
    """o ``[M,B,L,H,d]`` -> ``[B,T,H,d]``: ``sum_j w[b,t,j] * o[selected[b,t,j], b, slot[b,t,j]]``."""
    M, B, L, H, d = o.shape
    T, k = selected.shape[1:]
    flat = o.permute(1, 0, 2, 3, 4).reshape(B, M * L, H * d)
    pos = (selected * L + slot.clamp(min=0)).reshape(B, T * k)
    got = torch.gather(flat, 1, pos[..., None].expand(B, T * k, H * d)).reshape(B, T, k, H * d)
    w = (weights * (slot >= 0).to(weights.dtype))[..., None]
    return (got * w.to(got.dtype)).sum(2).reshape(B, T, H, d)


class MomLinearAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        mesh = self.mesh
        self.core_kind = {"mom_gla": "gla", "mom_gated_deltanet": "gated_deltanet",
                          "mom_linear_attention": "linear_attention"}[cfg.la_module]
        core_cfg = cfg.replace(la_module=self.core_kind)
        H = cfg.num_attention_heads
        self.H, self.Hl = H, H // mesh.tp
        self.dk, self.dv = cfg.key_dim // H, cfg.value_dim // H
        self.M, self.topk, self.capacity, self.shared_mem = cfg.mom_num_memories, cfg.mom_topk, cfg.mom_capacity, cfg.mom_shared_mem
        dt, std = cfg.params_dtype, cfg.init_method_std
        # sequence parallelism: gather the input along T at the entry (every path below completes its input gradient over
        # the TP ranks, so the backward of the gather is a slice), reduce-scatter at o_proj
        self.sp = sequence_parallel and mesh.tp > 1
        qkv_bias = (cfg.add_bias_linear or cfg.add_qkv_bias) if cfg.base_model == "qwen2" else cfg.add_bias_linear
        self.gate = nn.Linear(cfg.hidden_size, self.M, bias=False, dtype=dt, device=device)
        with torch.no_grad():
            self.gate.weight.copy_(init_normal((self.M, cfg.hidden_size), std, key + ".gate.weight", device))
        out = H * (2 * self.dk + self.dv)

        def col(name, o, bias=False):
            return ColumnParallelLinear(cfg.hidden_size, o, mesh=mesh, bias=bias, std=std, key=f"{key}.{name}",
                                        dtype=dt, device=device)
        self.qkv_proj = nn.ModuleList([col(f"qkv_proj.{m}", out, qkv_bias) for m in range(self.M)])
        if self.shared_mem:
            self.shared_qkv_proj = col("shared_qkv_proj", out, qkv_bias)
        self.o_gate_proj = col("o_gate_proj", cfg.value_dim, qkv_bias)
        if self.core_kind == "gla":
            self.gk_proj = nn.ModuleList([GLAGate(cfg, mesh, f"{key}.gk_proj.{m}", dt, device) for m in range(self.M)])
            if self.shared_mem:
                self.shared_gk_proj = GLAGate(cfg, mesh, key + ".shared_gk_proj", dt, device)
        if self.core_kind == "gated_deltanet":
            self.beta_proj = nn.ModuleList([col(f"beta_proj.{m}", H) for m in range(self.M)])
            self.a_proj = nn.ModuleList([col(f"a_proj.{m}", H) for m in range(self.M)])
            if self.shared_mem:
                self.shared_beta_proj = col("shared_beta_proj", H)
                self.shared_a_proj = col("shared_a_proj", H)
            A = init_uniform((H,), 1e-3, 16.0, key + ".A_log", device)
            self.A_log = nn.Parameter(_tp_slice(torch.log(A), mesh))
            self.D = nn.Parameter(_tp_slice(torch.ones(H, device=device), mesh))
            u = init_uniform((H,), 0.0, 1.0, key + ".dt_bias", device)
            dtv = torch.exp(u * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
            self.dt_bias = nn.Parameter(_tp_slice(dtv + torch.log(-torch.expm1(-dtv)), mesh))
            for p in (self.A_log, self.D, self.dt_bias):
                p._no_weight_decay = True
                p.tensor_parallel, p.partition_dim, p.partition_stride = mesh.tp > 1, 0, 1
        self.core_linear_attention = LSMCore(core_cfg, mesh, self.Hl, self.dk, self.dv,
                                             key + ".core_linear_attention", device)
        self.o_proj = RowParallelLinear(cfg.value_dim, cfg.hidden_size, mesh=mesh, bias=cfg.add_bias_linear,
                                        std=std / math.sqrt(2.0 * cfg.num_layers), key=key + ".o_proj",
                                        sequence_parallel=self.sp, dtype=dt, device=device)

    def _extras(self, x, gk_proj, beta_proj, a_proj):
        B, T = x.shape[:2]
        extra = {}
        if self.core_kind == "gla":
            extra["gk"] = gk_proj(x).reshape(B, T, self.Hl, self.dk)
        if self.core_kind == "gated_deltanet":
            extra["beta"] = torch.sigmoid(beta_proj(x).float())
            extra["g"] = -self.A_log.float().exp() * F.softplus(a_proj(x).float() + self.dt_bias.float())
        return extra

    def _split(self, qkv):
        B, T = qkv.shape[:2]
        return qkv.reshape(B, T, self.Hl, 2 * self.dk + self.dv).split([self.dk, self.dk, self.dv], dim=-1)

    def forward(self, x, cache: Optional[dict] = None, **_):
        assert cache is None or x.shape[1] >= 1
        tp = self.mesh["tp"]
        if self.sp:
            x = C.gather_no_reduce(x, tp, dim=1)
        B, T, _ = x.shape
        M, k = self.M, self.topk
        gate = self.o_gate_proj(x)
        scores = F.softmax(self.gate(x).float(), dim=-1)
        w, sel = torch.topk(scores, k, dim=-1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        if not tp.is_trivial:
            w = C.copy_to_region(w, tp)     # the routing weights scale this rank's heads only: sum their gradient over TP
        L = math.ceil(T / k * self.capacity)
        slot, gidx = mom_plan(sel, M, L)
        xm = mom_transform(x, gidx)                                           # [M,B,L,h]
        pad = (gidx < 0).permute(1, 0, 2)                                     # [M,B,L]
        qs, ks, vs, ex = [], [], [], {}
        for m in range(M):
            q, kk, v = self._split(self.qkv_proj[m](xm[m]))
            keep = (~pad[m])[..., None, None].to(q.dtype)
            qs.append(q * keep), ks.append(kk * keep), vs.append(v * keep)
            e = self._extras(xm[m], self.gk_proj[m] if self.core_kind == "gla" else None,
                             self.beta_proj[m] if self.core_kind == "gated_deltanet" else None,
                             self.a_proj[m] if self.core_kind == "gated_deltanet" else None)
            for name, t in e.items():
                if name == "beta":
                    t = t * (~pad[m])[..., None].to(t.dtype)
                ex.setdefault(name, []).append(t)
        cat = lambda ts: torch.cat(ts, dim=0)                                 # batch (M*B)
        mem_cache = None if cache is None else cache.setdefault("mom", {})
        o = self.core_linear_attention(cat(qs), cat(ks), cat(vs), cache=mem_cache,
                                       token_mask=(~pad).reshape(M * B, L),
                                       **{n: cat(t) for n, t in ex.items()})
        o = o.reshape(M, B, L, self.Hl, self.dv)
        out = mom_reconstruct(o, sel, slot, w)
        if self.shared_mem:
            q, kk, v = self._split(self.shared_qkv_proj(x))
            e = self._extras(x, getattr(self, "shared_gk_proj", None), getattr(self, "shared_beta_proj", None),
                             getattr(self, "shared_a_proj", None))
            sh_cache = None if cache is None else cache.setdefault("shared", {})
            out = out + self.core_linear_attention(q, kk, v, cache=sh_cache, **e).to(out.dtype)
        out = self.core_linear_attention.finish(out, gate)
        return self.o_proj(out)

"""Mamba2 mixer (SSD).

Reference: sequence_modeling/mamba2/mamba_mixer.py:54-518 — ``in_proj`` to
``[z | x | B | C | dt]``, depthwise causal conv (k=4) + SiLU over ``(x, B, C)``, the SSD chunk
scan, gated RMSNorm grouped over ``d_inner/ngroups`` channels, ``out_proj``; tensor
parallelism shards d_inner / ngroups / nheads (:101-112); ``step()`` is the single-token decode.

Here the scan is ``ops.ssd`` (the scalar-gated linear-attention kernel with q=C, k=B, v=dt*x,
g=dt*A), the conv and the recurrent state both support the sequence-parallel (LASP-2) split and
the decode cache, so ``forward`` with ``cache`` replaces ``step()``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config.model_config import ModelConfig
from ..dist.mesh import Mesh, single_process_mesh
from ..parallel.lasp2 import lasp2
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, init_uniform
from .lsm_layers import ShortConv, _tp_slice


class MambaMixer(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        mesh = self.mesh
        tp = mesh.tp
        self.d_model = cfg.hidden_size
        self.d_inner = cfg.mamba_expand * cfg.hidden_size
        self.headdim, self.d_state, self.ngroups = cfg.mamba_head_dim, cfg.mamba_d_state, cfg.mamba_ngroups
        self.nheads = self.d_inner // self.headdim
        assert self.d_inner % tp == 0 and self.ngroups % tp == 0 and self.nheads % tp == 0
        self.d_inner_l, self.ngroups_l, self.nheads_l = self.d_inner // tp, self.ngroups // tp, self.nheads // tp
        dt, std = cfg.params_dtype, cfg.init_method_std
        gs = self.ngroups * self.d_state
        self.in_proj = ColumnParallelLinear(self.d_model, 2 * self.d_inner + 2 * gs + self.nheads, mesh=mesh, std=std,
                                            key=key + ".in_proj", sequence_parallel=sequence_parallel, dtype=dt,
                                            device=device, part_sizes=[self.d_inner, self.d_inner, gs, gs, self.nheads])
        conv_dim_l = self.d_inner_l + 2 * self.ngroups_l * self.d_state
        self.conv1d = _MambaConv(self, cfg.mamba_d_conv, key + ".conv1d", dt, device)
        u = init_uniform((self.nheads,), 0.0, 1.0, key + ".dt_bias", device)
        dtv = torch.exp(u * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
        self.dt_bias = nn.Parameter(_tp_slice(dtv + torch.log(-torch.expm1(-dtv)), mesh))
        A = init_uniform((self.nheads,), 1.0, 16.0, key + ".A_log", device)
        self.A_log = nn.Parameter(_tp_slice(torch.log(A), mesh))
        self.D = nn.Parameter(torch.ones(self.nheads_l, device=device))
        for p in (self.dt_bias, self.A_log, self.D):
            p._no_weight_decay = True
            p.tensor_parallel = tp > 1
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.d_inner_l, dtype=dt, device=device))
        self.norm.weight.tensor_parallel = tp > 1
        self.out_proj = RowParallelLinear(self.d_inner, self.d_model, mesh=mesh,
                                          std=std / math.sqrt(2.0 * cfg.num_layers), key=key + ".out_proj",
                                          sequence_parallel=sequence_parallel, dtype=dt, device=device)

    def forward(self, x, cache: Optional[dict] = None, **_):
        cfg = self.cfg
        zxbcdt = self.in_proj(x)
        B, T = zxbcdt.shape[:2]
        gs_l = self.ngroups_l * self.d_state
        z, xBC, dt = zxbcdt.split([self.d_inner_l, self.d_inner_l + 2 * gs_l, self.nheads_l], dim=-1)
        xBC = self.conv1d(xBC.contiguous(), cache)
        xs, Bm, Cm = xBC.split([self.d_inner_l, gs_l, gs_l], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -self.A_log.float().exp()
        xh = xs.reshape(B, T, self.nheads_l, self.headdim)
        Bm = Bm.reshape(B, T, self.ngroups_l, self.d_state)
        Cm = Cm.reshape(B, T, self.ngroups_l, self.d_state)
        rep = self.nheads_l // self.ngroups_l
        kk = Bm.repeat_interleave(rep, dim=2) if rep > 1 else Bm
        qq = Cm.repeat_interleave(rep, dim=2) if rep > 1 else Cm
        g = dt * A[None, None, :]
        vv = (xh.float() * dt[..., None]).to(xh.dtype)
        init = cache.get("ssm") if cache is not None else None
        # --mamba-chunk-size is the tile length of the chunked scan.  It does not change the result (the scan is exact
        # for any tiling); the eager form tiles by it, the CUDA kernel always tiles by 64 tokens (its register /
        # shared-memory budget), so the value is passed through unchanged and only the eager form reads it.
        y, S = lasp2("scalar", qq, kk, vv, group=self.mesh["cp"], g=g, scale=1.0, chunk_size=cfg.mamba_chunk_size,
                     initial_state=init)
        if cache is not None:
            cache["ssm"] = S.detach()
        y = y.to(xh.dtype) + (xh.float() * self.D.float()[None, None, :, None]).to(xh.dtype)
        y = ops.gated_rms_norm(y.reshape(B, T, self.d_inner_l), z, self.norm.weight, 1e-5,
                               self.d_inner_l // self.ngroups_l)
        return self.out_proj(y)


class _MambaConv(ShortConv):
    """Depthwise conv over the TP-local ``(x, B, C)`` channels; the full weight is generated per part
    and sliced so that TP shards match the single-process model."""

    def __init__(self, mixer: MambaMixer, kernel: int, key: str, dtype, device):
        nn.Module.__init__(self)
        self.mesh, self.kernel, self.activation = mixer.mesh, kernel, "silu"
        gs = mixer.ngroups * mixer.d_state
        bound = 1.0 / math.sqrt(kernel)
        full = init_uniform((mixer.d_inner + 2 * gs, kernel), -bound, bound, key + ".weight", device)
        parts = full.split([mixer.d_inner, gs, gs], dim=0)
        w = torch.cat([_tp_slice(p, mixer.mesh) for p in parts], dim=0)
        self.weight = nn.Parameter(w.to(dtype))
        self.weight.tensor_parallel = mixer.mesh.tp > 1
        self.bias = nn.Parameter(torch.zeros(w.shape[0], dtype=dtype, device=device))
        self.bias.tensor_parallel = mixer.mesh.tp > 1

"""Linear-sequence-modeling token mixers.

``LinearAttention`` covers basic linear attention, lightning attention, retention, GLA,
DeltaNet, Gated DeltaNet, Based, Rebased, GSA and the LASP-2 variant of basic linear
attention (reference wrapper: sequence_modeling/linear_attention.py:24-258 and the cores under
sequence_modeling/{basic_linear_attention,lightning_attention,retention,gla,deltanet,
gated_deltanet,based,rebased,lasp2}/).  ``LinearRNN`` covers HGRN2, RWKV6 and RWKV7
(sequence_modeling/linear_rnn.py:32-347).

Differences from the reference, on purpose:

* every per-head projection (GLA gate, beta, a, A_log, dt_bias, bonus ...) is sharded by head
  under tensor parallelism; the reference leaves them unsharded while q/k/v are sharded
  (gla_gate.py:22-23, linear_attention.py:88-113).
* every mixer runs under LASP-2 sequence parallelism when the mesh has a context-parallel
  axis (the reference has it for undecayed linear attention only).
* every mixer keeps an O(1) recurrent state cache for decoding (the reference allocates a
  softmax-style KV buffer, linear_attention.py:260-342).
* ``LinearRNN.forward`` returns a tensor like the other mixers (the reference returns a bare
  tensor where the caller unpacks a tuple, linear_rnn.py:346-347).

Activations are ``[B, T, h]``; heads are ``[B, T, H, d]``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config.model_config import ModelConfig
from ..dist import collectives as C
from ..dist.mesh import Mesh, single_process_mesh
from ..parallel.lasp2 import lasp2
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, init_normal, init_uniform
from ..ref import lsm as RL
from ..ref import ops as R
from .feature_maps import build_feature_map, elu_p1, RebasedMap, Taylor


def _tp_slice(full: torch.Tensor, mesh: Mesh, dim: int = 0) -> torch.Tensor:
    return full.chunk(mesh.tp, dim=dim)[mesh.tp_rank].contiguous() if mesh.tp > 1 else full


class ShortConv(nn.Module):
    """Depthwise causal convolution + SiLU over time with sequence-parallel halo exchange and a decode
    cache (counterpart of ``causal_conv1d_fn`` / ``causal_conv1d_update``, mamba_mixer.py:291-296,383-389)."""

    def __init__(self, dim: int, kernel: int, *, mesh: Mesh, key: str, bias: bool = False, dtype=torch.float32,
                 device=None, full_dim: Optional[int] = None, activation: Optional[str] = "silu"):
        super().__init__()
        self.mesh, self.kernel, self.activation = mesh, kernel, activation
        bound = 1.0 / math.sqrt(kernel)
        full = init_uniform((full_dim or dim, kernel), -bound, bound, key + ".weight", device)
        if full_dim is not None and full_dim != dim:
            full = _tp_slice(full, mesh)
        self.weight = nn.Parameter(full.to(dtype))
        self.weight.tensor_parallel = mesh.tp > 1
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if bias else None

    def forward(self, x, cache: Optional[dict] = None, cache_key: str = "conv"):
        init = None
        g = self.mesh["cp"]
        if cache is not None and cache_key in cache:
            init = cache[cache_key]
        elif not g.is_trivial:
            tail = x[:, -(self.kernel - 1):].contiguous()
            tails = C.all_gather(tail[None], g, dim=0)
            init = tails[g.rank - 1] if g.rank > 0 else torch.zeros_like(tail) + 0.0 * tails.sum(0)
        y, final = ops.causal_conv1d(x, self.weight, self.bias, self.activation, init)
        if cache is not None:
            cache[cache_key] = final.detach()
        return y


class GLAGate(nn.Module):
    """Low-rank gate ``W2 (W1 x) + b`` (gla_gate.py:9-31); the second factor is split by head."""

    def __init__(self, cfg: ModelConfig, mesh: Mesh, key: str, dtype, device):
        super().__init__()
        r = cfg.gla_la_gate_low_rank_dim
        w0 = init_normal((r, cfg.hidden_size), cfg.init_method_std, key + ".gk_proj.0.weight", device)
        self.gk_proj = nn.ModuleList([nn.Linear(cfg.hidden_size, r, bias=False, dtype=dtype, device=device),
                                      ColumnParallelLinear(r, cfg.key_dim, mesh=mesh, bias=True,
                                                           std=cfg.init_method_std, key=key + ".gk_proj.1",
                                                           dtype=dtype, device=device)])
        with torch.no_grad():
            self.gk_proj[0].weight.copy_(w0)
        self.mesh = mesh

    def forward(self, x):
        return self.gk_proj[1](F.linear(x, self.gk_proj[0].weight))


class LinearAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        mesh = self.mesh
        self.kind = cfg.la_module
        if self.kind == "lasp2":
            self.kind = "linear_attention"
        H = cfg.num_attention_heads
        assert H % mesh.tp == 0
        self.H, self.Hl = H, H // mesh.tp
        self.dk, self.dv = cfg.key_dim // H, cfg.value_dim // H
        dt, std = cfg.params_dtype, cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        qkv_bias = (cfg.add_bias_linear or cfg.add_qkv_bias) if cfg.base_model == "qwen2" else cfg.add_bias_linear
        sp = sequence_parallel
        # fused projection laid out per head as [q(dk) | k(dk) | v(dv)] so that TP splits whole heads
        self.qkv_proj = ColumnParallelLinear(cfg.hidden_size, H * (2 * self.dk + self.dv), mesh=mesh, bias=qkv_bias,
                                             std=std, key=key + ".qkv_proj", sequence_parallel=sp, dtype=dt,
                                             device=device)
        self.o_gate_proj = ColumnParallelLinear(cfg.hidden_size, cfg.value_dim, mesh=mesh, bias=qkv_bias, std=std,
                                                key=key + ".o_gate_proj", sequence_parallel=sp, dtype=dt,
                                                device=device)
        self.o_proj = RowParallelLinear(cfg.value_dim, cfg.hidden_size, mesh=mesh, bias=cfg.add_bias_linear,
                                        std=out_std, key=key + ".o_proj", sequence_parallel=sp, dtype=dt,
                                        device=device)
        kind = self.kind
        if kind == "gla":
            self.gk_proj = GLAGate(cfg, mesh, key + ".gk_proj", dt, device)
        if kind in ("deltanet", "gated_deltanet"):
            self.beta_proj = ColumnParallelLinear(cfg.hidden_size, H, mesh=mesh, std=std, key=key + ".beta_proj",
                                                  sequence_parallel=sp, dtype=dt, device=device)
        if kind == "gated_deltanet":
            self.a_proj = ColumnParallelLinear(cfg.hidden_size, H, mesh=mesh, std=std, key=key + ".a_proj",
                                               sequence_parallel=sp, dtype=dt, device=device)
            A = init_uniform((H,), 1e-3, 16.0, key + ".A_log", device)
            self.A_log = nn.Parameter(_tp_slice(torch.log(A), mesh))
            self.D = nn.Parameter(_tp_slice(torch.ones(H, device=device), mesh))
            u = init_uniform((H,), 0.0, 1.0, key + ".dt_bias", device)
            dtv = torch.exp(u * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
            self.dt_bias = nn.Parameter(_tp_slice(dtv + torch.log(-torch.expm1(-dtv)), mesh))
            for p in (self.A_log, self.D, self.dt_bias):
                p._no_weight_decay = True
                p.tensor_parallel = mesh.tp > 1
        if kind == "gsa":
            self.num_slots = cfg.gsa_num_slots
            self.f_proj = ColumnParallelLinear(cfg.hidden_size, H * self.num_slots, mesh=mesh, std=std,
                                               key=key + ".f_proj", sequence_parallel=sp, dtype=dt, device=device)
        use_conv = cfg.use_short_conv and kind in ("gated_deltanet", "deltanet", "gla", "gsa")
        if use_conv:
            dim = self.Hl * (2 * self.dk + self.dv)
            self.conv1d = ShortConv(dim, cfg.conv_size, mesh=mesh, key=key + ".conv1d", dtype=dt, device=device,
                                    full_dim=H * (2 * self.dk + self.dv))
        else:
            self.conv1d = None
        self.core_linear_attention = LSMCore(cfg, mesh, self.Hl, self.dk, self.dv, key + ".core_linear_attention",
                                             device)

    # ------------------------------------------------------------------
    def forward(self, x: torch.Tensor, cache: Optional[dict] = None, **_) -> torch.Tensor:
        cfg, kind = self.cfg, self.kind
        qkv = self.qkv_proj(x)
        gate = self.o_gate_proj(x)
        B, T = qkv.shape[:2]
        extra: Dict[str, torch.Tensor] = {}
        if kind == "gla":
            extra["gk"] = self.gk_proj(x if not self.qkv_proj.sequence_parallel else
                                       C.all_gather(x, self.mesh["tp"], dim=1)).reshape(B, T, self.Hl, self.dk)
        if kind in ("deltanet", "gated_deltanet"):
            extra["beta"] = torch.sigmoid(self.beta_proj(x).float())
        if kind == "gated_deltanet":
            extra["g"] = -self.A_log.float().exp() * F.softplus(self.a_proj(x).float() + self.dt_bias.float())
        if kind == "gsa":
            extra["f"] = self.f_proj(x).reshape(B, T, self.Hl, self.num_slots)
        if self.conv1d is not None:
            qkv = self.conv1d(qkv, cache)
        qkv = qkv.reshape(B, T, self.Hl, 2 * self.dk + self.dv)
        q, k, v = qkv.split([self.dk, self.dk, self.dv], dim=-1)
        o = self.core_linear_attention(q, k, v, cache=cache, conv_applied=self.conv1d is not None, **extra)
        o = self.core_linear_attention.finish(o, gate)
        return self.o_proj(o)


class LSMCore(nn.Module):
    """The per-family math between the projections: activations / feature maps, the recurrence
    (through ``ops.lsm_*`` or LASP-2), and the per-head output norm + gate."""

    def __init__(self, cfg: ModelConfig, mesh: Mesh, heads_local: int, dk: int, dv: int, key: str, device=None):
        super().__init__()
        self.cfg, self.mesh, self.Hl, self.dk, self.dv = cfg, mesh, heads_local, dk, dv
        self.kind = "linear_attention" if cfg.la_module == "lasp2" else cfg.la_module
        kind = self.kind
        H = cfg.num_attention_heads
        dt = cfg.params_dtype
        fm = cfg.la_feature_map
        if kind == "linear_attention" and fm is None:
            fm = "elu"
        if kind == "based":
            self.feature_map_q = self.feature_map_k = Taylor(dk)
        elif kind == "rebased":
            self.feature_map_q = self.feature_map_k = RebasedMap(dk)
        elif kind in ("linear_attention", "lightning_attention", "retention", "gla", "gsa"):
            self.feature_map_q = build_feature_map(fm, dk, key + ".feature_map_q")
            self.feature_map_k = self.feature_map_q if (cfg.la_tie_feature_map_qk or fm is None) else \
                build_feature_map(fm, dk, key + ".feature_map_k")
        else:
            self.feature_map_q = self.feature_map_k = None
        if kind == "lightning_attention":
            slopes = RL.lightning_slopes(H)
            self.register_buffer("log_decay", -_tp_slice(slopes, mesh).to(device), persistent=False)
        elif kind == "retention":
            self.register_buffer("log_decay", _tp_slice(RL.retention_log_decay(H), mesh).to(device), persistent=False)
        self.output_norm = cfg.la_output_norm
        if self.output_norm in ("rmsnorm", "groupnorm") and cfg.la_elementwise_affine:
            self.la_output_norm = nn.Module()
            self.la_output_norm.weight = nn.Parameter(torch.ones(dv, dtype=dt, device=device))
            if self.output_norm == "groupnorm":
                self.la_output_norm.bias = nn.Parameter(torch.zeros(dv, dtype=dt, device=device))
        else:
            self.la_output_norm = None
        # replicated over the tensor-parallel ranks but applied to the rank's own heads only: every rank holds a partial
        # gradient, which the optimizer sums over the TP group
        shared = [self.la_output_norm, self.feature_map_q, self.feature_map_k]
        for mod in shared:
            for p in (mod.parameters() if mod is not None else ()):
                p.tp_partial_grad = True

    # -- helpers --------------------------------------------------------
    def _run(self, op: str, q, k, v, cache, name="state", **kw):
        """Dispatch to LASP-2 when the sequence is split over the cp group, keep the decode cache."""
        g = self.mesh["cp"]
        init = cache.get(name) if cache is not None else None
        o, S = lasp2(op, q, k, v, group=g, chunk_size=self.cfg.la_chunk_size, initial_state=init,
                     mode=self.cfg.la_mode if (init is None or self.cfg.la_mode != "parallel") else "chunk", **kw)
        if cache is not None:
            cache[name] = S.detach()
        return o

    def _normalized(self, q, k, v, cache, scale):
        """Linear attention divided by ``q . sum k``: the denominator is obtained from the same kernel
        by appending a column of ones to v."""
        ones = torch.ones_like(v[..., :1])
        o = self._run("scalar", q, k, torch.cat([v, ones], dim=-1), cache, scale=scale)
        return o[..., :-1] / (o[..., -1:] + 1e-10)

    # -- forward ----------------------------------------------------------
    def forward(self, q, k, v, cache=None, gk=None, beta=None, g=None, f=None, conv_applied=False,
                token_mask=None):
        """``token_mask`` ``[B,T]`` (1 = real token) switches the decay off at padding tokens, so that a
        padded position leaves the state untouched (MoM rows)."""
        cfg, kind = self.cfg, self.kind
        if kind == "linear_attention":
            q, k = self.feature_map_q(q), self.feature_map_k(k)
            if cfg.la_norm_q:
                q = q / (q.sum(-1, keepdim=True) + 1e-4)
            if cfg.la_norm_k:
                k = k / (k.sum(-1, keepdim=True) + 1e-4)
            if cfg.la_do_feature_map_norm:
                return self._normalized(q, k, v, cache, None)
            return self._run("scalar", q, k, v, cache, scale=None)
        if kind in ("lightning_attention", "retention"):
            if self.feature_map_q is not None:
                q, k = self.feature_map_q(q), self.feature_map_k(k)
            scale = 1.0 if kind == "lightning_attention" else None
            return self._run("scalar", q, k, v, cache, g=self.log_decay, scale=scale)
        if kind == "gla":
            if self.feature_map_q is not None:
                q, k = self.feature_map_q(q), self.feature_map_k(k)
            gk = F.logsigmoid(gk.float()) / cfg.gla_la_gate_logit_normalizer
            if cfg.gla_la_clamp_min is not None:
                gk = gk.clamp_min(cfg.gla_la_clamp_min)
            if token_mask is not None:
                gk = gk * token_mask[..., None, None].to(gk.dtype)
            return self._run("vector", q, k, v, cache, gk=gk, scale=None)
        if kind in ("deltanet", "gated_deltanet"):
            act = cfg.deltanet_qk_activation if kind == "deltanet" else "silu"
            if not conv_applied:            # the short conv already applies SiLU
                if act == "silu":
                    q, k = F.silu(q), F.silu(k)
                    if kind == "gated_deltanet":
                        v = F.silu(v)       # gated_deltanet.py:99-101
                elif act == "relu":
                    q, k = q.relu(), k.relu()
                elif act == "elu":
                    q, k = elu_p1(q), elu_p1(k)
            if cfg.deltanet_qk_norm == "l2":
                q, k = ops.l2_norm(q), ops.l2_norm(k)
            elif cfg.deltanet_qk_norm == "sum":
                q, k = q / q.sum(-1, keepdim=True), k / k.sum(-1, keepdim=True)
            if token_mask is not None and g is not None:
                g = g * token_mask[..., None].to(g.dtype)
            return self._run("delta", q, k, v, cache, beta=beta, g=g if kind == "gated_deltanet" else None,
                             scale=None)
        if kind in ("based", "rebased"):
            q, k = self.feature_map_q(q), self.feature_map_k(k)
            return self._normalized(q, k, v, cache, 1.0)
        if kind == "gsa":
            return self._gsa(q, k, v, f, cache)
        raise NotImplementedError(kind)

    def _gsa(self, q, k, v, f, cache):
        """Gated slot attention = two gated linear-attention passes through ``m`` slots:
        scores over slots from a slot-wise decayed key memory, softmax, read of a slot-wise decayed
        value memory.  (Advertised by the reference's README.md:29 without code; built from the paper.)"""
        cfg = self.cfg
        if self.feature_map_q is not None:
            q, k = self.feature_map_q(q), self.feature_map_k(k)
        else:
            q, k = F.silu(q), F.silu(k)
        v = F.silu(v)
        logf = F.logsigmoid(f.float()) / cfg.gla_la_gate_logit_normalizer            # [B,T,H,m]
        s = 1.0 - logf.exp()
        init1 = cache.get("gsa_k") if cache is not None else None
        ok, S1 = lasp2("value", q, k, s, group=self.mesh["cp"], gk=logf, scale=None, initial_state=init1)
        p = torch.softmax(ok, dim=-1).to(v.dtype)
        o = self._run("vector", p, s.to(v.dtype), v, cache, name="gsa_v", gk=logf, scale=1.0)
        if cache is not None:
            cache["gsa_k"] = S1.detach()
        return o

    def finish(self, o, gate):
        """Per-head output norm then ``* gate_fn(gate)``; returns ``[B,T,H*dv]``."""
        cfg = self.cfg
        B, T = o.shape[:2]
        if self.kind == "gated_deltanet":
            # the reference's Gated DeltaNet core has no output norm (gated_deltanet.py:112-116)
            norm, w = "identity", None
        else:
            norm = self.output_norm
            w = self.la_output_norm.weight if self.la_output_norm is not None else None
        o = o.to(gate.dtype)
        if norm == "groupnorm":
            y = ops.group_norm_heads(o, w, self.la_output_norm.bias if self.la_output_norm is not None else None,
                                     cfg.la_norm_eps).reshape(B, T, -1)
            return (y.float() * R.ACT2FN[cfg.la_gate_fn](gate.float())).to(gate.dtype)
        return ops.head_norm_gate(o.contiguous(), w, gate, cfg.la_norm_eps, cfg.la_gate_fn, norm)


# ---------------------------------------------------------------------------
class LerpLinear(nn.Module):
    """``W (x + delta * mu)`` with optional low-rank factorisation (rwkv6/dd_lerp_linear.py:10-60)."""

    def __init__(self, inp, out, low_rank: Optional[int] = None, dtype=torch.float32, device=None):
        super().__init__()
        self.mu = nn.Parameter(torch.zeros(inp, dtype=dtype, device=device))
        if low_rank is None:
            self.linear = nn.Linear(inp, out, bias=False, dtype=dtype, device=device)
        else:
            self.linear = LoRA(inp, out, low_rank, dtype=dtype, device=device)

    def forward(self, x, delta=None):
        if delta is None:
            delta = F.pad(x, (0, 0, 1, -1)) - x
        inp = x + delta * self.mu
        tp_in = getattr(self, "tp_in", None)
        return self.linear(inp if tp_in is None else tp_in(inp))


class DDLerpLinear(nn.Module):
    """Data-dependent lerp ``W (x + delta * mu_t)`` (rwkv6/dd_lerp_linear.py:63-115)."""

    def __init__(self, inp, out, low_rank: Optional[int] = None, dtype=torch.float32, device=None):
        super().__init__()
        if low_rank is None:
            self.linear = nn.Linear(inp, out, bias=False, dtype=dtype, device=device)
        else:
            self.linear = LoRA(inp, out, low_rank, dtype=dtype, device=device)

    def forward(self, x, mu, delta=None):
        if delta is None:
            delta = F.pad(x, (0, 0, 1, -1)) - x
        inp = x + delta * mu
        tp_in = getattr(self, "tp_in", None)
        return self.linear(inp if tp_in is None else tp_in(inp))


class LoRA(nn.Module):
    """``W2 act(W1 x) + b`` (rwkv6/dd_lerp_linear.py LoRA, rwkv7/lora_mlp.py:10-54)."""

    def __init__(self, inp, out, low_rank, bias: bool = True, activation: Optional[str] = "tanh",
                 dtype=torch.float32, device=None):
        super().__init__()
        act = {"tanh": nn.Tanh(), "sigmoid": nn.Sigmoid(), "relu": nn.ReLU(), None: nn.Identity()}[activation]
        self.lora = nn.Sequential(nn.Linear(inp, low_rank, bias=False, dtype=dtype, device=device), act,
                                  nn.Linear(low_rank, out, bias=bias, dtype=dtype, device=device))

    def forward(self, x):
        tp_in = getattr(self, "tp_in", None)
        if tp_in is None:
            return self.lora(x)
        return self.lora[2](tp_in(self.lora[1](self.lora[0](x))))      # head-sharded up-projection under TP


class _HeadShardedInput(nn.Module):
    """Marks the input of a head-sharded projection under tensor parallelism: identity in the forward pass, all-reduce of
    the gradient over the TP group in the backward pass, so that everything upstream (the block input, the token-shift
    mixing coefficients, the replicated low-rank factors) receives the complete gradient on every rank."""

    def __init__(self, mesh: Mesh, enabled: bool):
        super().__init__()
        self.mesh, self.enabled = mesh, enabled

    def forward(self, x):
        return C.copy_to_region(x, self.mesh["tp"]) if self.enabled else x


def _shard_rows(linear: nn.Linear, mesh: Mesh):
    """Keep this TP rank's block of output rows (= its heads) of a projection that was initialised at full size."""
    linear.weight = nn.Parameter(_tp_slice(linear.weight.data, mesh, 0))
    linear.weight.tensor_parallel, linear.weight.partition_dim, linear.weight.partition_stride = True, 0, 1
    if linear.bias is not None:
        linear.bias = nn.Parameter(_tp_slice(linear.bias.data, mesh, 0))
        linear.bias.tensor_parallel, linear.bias.partition_dim, linear.bias.partition_stride = True, 0, 1
    linear.out_features = linear.weight.shape[0]


class LinearRNN(nn.Module):
    """HGRN2 / RWKV6 / RWKV7 token mixers.  Under tensor parallelism the heads are split over the TP ranks: every
    projection into key / value space keeps its ranks' rows, the per-head vectors are sliced, the low-rank mixers in
    front of them stay replicated (their gradients are completed by an all-reduce at the sharded projections' inputs)
    and ``o_proj`` is row-parallel (reduce-scattering along T under sequence parallelism).  (The reference builds these
    mixers without TP support.)"""

    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        tp = self.mesh.tp
        # sequence parallelism: the block's input arrives split along T over the TP ranks; it is gathered at the entry
        # (every rank then holds the complete input gradient, so the backward is a slice) and o_proj reduce-scatters
        self.sp = sequence_parallel and tp > 1
        assert cfg.num_attention_heads % tp == 0, "heads must divide over the tensor-parallel ranks"
        self.kind = cfg.la_module
        H, hid = cfg.num_attention_heads, cfg.hidden_size
        self.H = H
        self.key_dim, self.value_dim = cfg.key_dim, cfg.value_dim
        self.dk, self.dv = self.key_dim // H, self.value_dim // H
        dt = cfg.params_dtype
        kw = dict(dtype=dt, device=device)
        self.layer_number = layer_number
        if self.kind == "rwkv6":
            r = cfg.rwkv6_la_proj_low_rank_dim
            self.x_proj = nn.Sequential(LerpLinear(hid, r * 5, **kw), nn.Tanh(), nn.Linear(r * 5, hid, bias=False, **kw))
            self.x_bias = nn.Parameter(torch.zeros(5, hid, **kw))
            self.r_proj = DDLerpLinear(hid, self.key_dim, **kw)
            self.w_proj = DDLerpLinear(hid, self.key_dim, low_rank=cfg.rwkv6_la_gate_low_rank_dim, **kw)
            self.k_proj = DDLerpLinear(hid, self.key_dim, **kw)
            self.v_proj = DDLerpLinear(hid, self.value_dim, **kw)
            self.g_proj = DDLerpLinear(hid, self.value_dim, **kw)
            self.bonus = nn.Parameter(torch.zeros(H, self.dk, **kw))
        elif self.kind == "rwkv7":
            self.x = nn.Parameter(torch.zeros(6, hid, **kw))
            self.r_proj = nn.Linear(hid, self.key_dim, bias=False, **kw)
            self.k_proj = nn.Linear(hid, self.key_dim, bias=False, **kw)
            self.v_proj = nn.Linear(hid, self.value_dim, bias=False, **kw)
            self.w_proj = LoRA(hid, self.key_dim, cfg.rwkv7_la_decay_low_rank_dim, activation="tanh", **kw)
            self.a_proj = LoRA(hid, self.key_dim, cfg.rwkv7_la_a_low_rank_dim, activation=None, **kw)
            self.g_proj = LoRA(hid, self.value_dim, cfg.rwkv7_la_gate_low_rank_dim, activation="sigmoid", bias=False, **kw)
            self.bonus = nn.Parameter(torch.zeros(H, self.dk, **kw))
            self.booster = nn.Parameter(torch.zeros(self.key_dim, **kw))
            self.removal = nn.Parameter(torch.zeros(self.key_dim, **kw))
        elif self.kind == "hgrn2":
            self.q_proj = nn.Linear(hid, self.key_dim, bias=False, **kw)
            self.f_proj = nn.Linear(hid, self.key_dim, bias=False, **kw)
            self.i_proj = nn.Linear(hid, self.value_dim, bias=False, **kw)
        else:
            raise NotImplementedError(self.kind)
        for name, m in self.named_modules():
            if isinstance(m, nn.Linear):
                with torch.no_grad():
                    m.weight.copy_(init_normal(tuple(m.weight.shape), cfg.init_method_std, f"{key}.{name}.weight", device))
                    if m.bias is not None:
                        m.bias.zero_()       # nn.Linear drew it from the process-global generator: not the same on every rank
        out_std = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        self.o_proj = RowParallelLinear(self.value_dim, hid, mesh=self.mesh, std=out_std, key=key + ".o_proj",
                                        sequence_parallel=self.sp, dtype=dt, device=device)
        self.norm_weight = nn.Parameter(torch.ones(self.dv, **kw)) if cfg.la_output_norm != "identity" else None
        self.tp_in = _HeadShardedInput(self.mesh, tp > 1)
        if tp > 1:
            self._shard_for_tp()

    def _shard_for_tp(self):
        """Cut the full-size, seed-initialised parameters down to this rank's heads (same values as the tp = 1 model)."""
        mesh = self.mesh
        self.H = self.H // mesh.tp
        projs = {"rwkv6": ["r_proj", "w_proj", "k_proj", "v_proj", "g_proj"],
                 "rwkv7": ["r_proj", "k_proj", "v_proj", "w_proj", "a_proj", "g_proj"],
                 "hgrn2": ["q_proj", "f_proj", "i_proj"]}[self.kind]
        for name in projs:
            m = getattr(self, name)
            if isinstance(m, nn.Linear):
                _shard_rows(m, mesh)
                continue
            inner = m.linear if hasattr(m, "linear") else m          # DDLerpLinear -> Linear | LoRA; or a bare LoRA
            if isinstance(inner, nn.Linear):
                _shard_rows(inner, mesh)
                m.tp_in = _HeadShardedInput(mesh, True)
            else:
                _shard_rows(inner.lora[2], mesh)                      # LoRA: the up-projection carries the heads
                inner.tp_in = _HeadShardedInput(mesh, True)
        for name in ("bonus", "booster", "removal"):
            if hasattr(self, name):
                p = nn.Parameter(_tp_slice(getattr(self, name).data, mesh, 0))
                p.tensor_parallel, p.partition_dim, p.partition_stride = True, 0, 1
                setattr(self, name, p)

    def _shift(self, x, cache, name="shift"):
        """Token shift ``x_{t-1}`` with sequence-parallel halo and decode cache."""
        g = self.mesh["cp"]
        prev = None
        if cache is not None and name in cache:
            prev = cache[name]
        elif not g.is_trivial:
            tails = C.all_gather(x[:, -1:][None].contiguous(), g, dim=0)
            prev = tails[g.rank - 1] if g.rank > 0 else torch.zeros_like(x[:, :1]) + 0.0 * tails.sum(0)
        shifted = F.pad(x, (0, 0, 1, -1))
        if prev is not None:
            shifted = torch.cat([prev.to(x.dtype), x[:, :-1]], dim=1)
        if cache is not None:
            cache[name] = x[:, -1:].detach()
        return shifted

    def _run(self, op, q, k, v, cache, **kw):
        init = cache.get("state") if cache is not None else None
        o, S = lasp2(op, q, k, v, group=self.mesh["cp"], chunk_size=self.cfg.la_chunk_size, initial_state=init,
                     mode=self.cfg.la_mode, **kw)
        if cache is not None:
            cache["state"] = S.detach()
        return o

    def forward(self, x, cache: Optional[dict] = None, lower_bound: Optional[torch.Tensor] = None, **_):
        if self.sp:
            x = C.gather_no_reduce(x, self.mesh["tp"], dim=1)
        B, T, hid = x.shape
        H, act = self.H, R.ACT2FN[self.cfg.la_gate_fn]
        hv = lambda t, d: t.reshape(B, T, H, d)
        if self.kind == "rwkv6":
            delta = self._shift(x, cache) - x
            r5 = self.cfg.rwkv6_la_proj_low_rank_dim
            xx = self.x_proj[0](x, delta).view(B, T, 5, r5)
            xx = torch.einsum("blnr,hnr->blnh", self.x_proj[1](xx), self.x_proj[2].weight.view(hid, 5, r5))
            r, w, k, v, g = (xx + self.x_bias).unbind(-2)
            r, w, k = self.r_proj(x, r, delta), self.w_proj(x, w, delta), self.k_proj(x, k, delta)
            v, g = self.v_proj(x, v, delta), self.g_proj(x, g, delta)
            w = -torch.exp(w.float())
            o = self._run("vector", hv(r, self.dk), hv(k, self.dk), hv(v, self.dv), cache, gk=hv(w, self.dk),
                          scale=1.0, bonus=self.bonus)
            o = self._out_norm(o).reshape(B, T, -1) * act(g)
        elif self.kind == "rwkv7":
            delta = self._shift(x, cache) - x
            xr, xw, xk, xv, xa, xg = torch.addcmul(x[None], delta[None], self.x.view(6, 1, 1, -1)).unbind(0)
            r = self.r_proj(self.tp_in(xr))
            w = -math.exp(-0.5) * self.w_proj(xw).float().sigmoid()
            k, v = self.k_proj(self.tp_in(xk)), self.v_proj(self.tp_in(xv))
            a = self.a_proj(xa).sigmoid()
            g = self.g_proj(xg)
            kk = ops.l2_norm(hv(k * self.removal, self.dk)).reshape(B, T, -1)
            k = torch.addcmul(k, k * (a - 1), self.booster)
            o = self._run("dplr", hv(r, self.dk), hv(k, self.dk), hv(v, self.dv), cache, gk=hv(w, self.dk), scale=1.0,
                          dplr=(hv(-kk, self.dk), hv(kk * a, self.dk)))
            o = self._out_norm(o.to(x.dtype))
            o = o + ((hv(r, self.dk) * hv(k, self.dk) * self.bonus).sum(-1, keepdim=True) * hv(v, self.dv))
            o = o.reshape(B, T, -1) * act(g)
        else:  # hgrn2
            xs = self.tp_in(x)
            q, f, i = F.silu(self.q_proj(xs)), self.f_proj(xs).float(), self.i_proj(xs)
            if lower_bound is not None and self.mesh.tp > 1:
                # the bounds are a replicated parameter indexed by key channel: take this rank's heads, complete its
                # gradient over the TP ranks
                lower_bound = _tp_slice(C.copy_to_region(lower_bound, self.mesh["tp"]), self.mesh, -1)
            if lower_bound is None or not self.cfg.hgrn2_lower_bound:
                k, g = 1 - f.sigmoid(), F.logsigmoid(f)
            else:
                gg = lower_bound + (1 - lower_bound) * f.sigmoid()
                k, g = 1 - gg, gg.log()
            o = self._run("vector", hv(q, self.dk), hv(k.to(i.dtype), self.dk), hv(i, self.dv), cache,
                          gk=hv(g, self.dk), scale=1.0)
            o = self._out_norm(o).reshape(B, T, -1)
        return self.o_proj(o.to(x.dtype))

    def _out_norm(self, o):
        if self.norm_weight is None:
            return o
        # the per-head norm weight is shared by all heads: under TP its gradient is summed over the ranks' heads
        w = C.copy_to_region(self.norm_weight, self.mesh["tp"])
        return ops.rms_norm(o.to(self.norm_weight.dtype).contiguous(), w, self.cfg.la_norm_eps)

"""Dense MLP and Mixture-of-Experts layers: router, token dispatcher, experts, shared expert.

Reference: model/qwen2/transformer/mlp.py:40-230, model/qwen2/moe/{moe_layer,router,
token_dispatcher,experts}.py, model/mixtral/moe/*, model/deepseek_v2/moe/*.

Design notes

* One router class covers both orders (softmax->top-k for Qwen2/DeepSeek, top-k->softmax for
  Mixtral/Llama3), aux load-balancing loss, z-loss, sinkhorn, input jitter and capacity-based
  token dropping.
* Experts are always stored grouped: ``weight1 [E_local, h, 2f/TP]`` (gate|up) and
  ``weight2 [E_local, f/TP, h]``; the checkpoint writer renames them to the reference's
  ``local_experts.{e}.linear_fc1/linear_fc2`` keys.
* Dispatch: tokens are sorted by global expert id; with expert parallelism they are exchanged
  with one all-to-all-v each way.  The per-rank counts that an NCCL all-to-all needs on the host
  cost one device->host copy per layer (the reference pays the same, token_dispatcher.py:363,
  369-386); the fused P2P dispatcher of ``ops.cuda`` keeps the counts on the device.
* With TP > 1 the MoE region is sequence parallel (as moe_layer.py:146-154 demands): each TP rank
  routes its own T/TP tokens; tokens arriving at an expert rank are all-gathered over TP before
  the expert GEMMs (which are TP-sharded along ffn) and reduce-scattered after.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config.model_config import ModelConfig
from ..dist import collectives as C
from ..dist.mesh import Mesh, single_process_mesh
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, init_normal
from ..ref import ops as R


class MLP(nn.Module):
    """``fc2(swiglu(fc1(x)))``; fc1 = [gate; up] column-parallel (split per GLU half), fc2 row-parallel."""

    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, key: str = "", ffn: Optional[int] = None,
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        ffn = ffn or cfg.ffn_hidden_size
        dt, std = cfg.params_dtype, cfg.init_method_std
        self.glu = cfg.swiglu
        self.linear_fc1 = ColumnParallelLinear(cfg.hidden_size, ffn * (2 if self.glu else 1), mesh=self.mesh,
                                               bias=cfg.add_bias_linear, std=std, key=key + ".linear_fc1",
                                               sequence_parallel=sequence_parallel, stride=2 if self.glu else 1,
                                               dtype=dt, device=device)
        self.linear_fc2 = RowParallelLinear(ffn, cfg.hidden_size, mesh=self.mesh, bias=cfg.add_bias_linear,
                                            std=std / math.sqrt(2.0 * cfg.num_layers), key=key + ".linear_fc2",
                                            sequence_parallel=sequence_parallel, dtype=dt, device=device)

    def forward(self, x):
        fc1, fc2 = self.linear_fc1, self.linear_fc2
        if (self.glu and fc1.bias is None and fc2.bias is None and not fc1.sequence_parallel and not fc1.gather_output
                and not fc2.sequence_parallel and fc2.input_is_parallel and x.is_cuda):
            # both linears and the activation in one autograd node: SwiGLU forward and backward live in GEMM epilogues;
            # the row-parallel reduction of fc2 follows outside
            g = self.mesh["tp"]
            return C.all_reduce(ops.mlp_swiglu(C.copy_to_region(x, g), fc1.weight, fc2.weight), g)
        if self.glu and fc1.bias is None and not fc1.sequence_parallel and not fc1.gather_output:
            h = ops.linear_swiglu(C.copy_to_region(x, self.mesh["tp"]), fc1.weight)
        else:
            h = fc1(x)
            h = ops.swiglu(h) if self.glu else F.gelu(h)
        return self.linear_fc2(h)


class MoEAuxLossAutoScaler(torch.autograd.Function):
    """Attach an auxiliary loss to an activation: forward returns the activation, backward adds a
    gradient of ``scale`` to the aux loss (mixtral/moe/moe_utils.py:75-118)."""
    main_loss_backward_scale: float = 1.0

    @staticmethod
    def forward(ctx, output, aux_loss):
        ctx.save_for_backward(aux_loss)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (aux_loss,) = ctx.saved_tensors
        return grad_output, torch.ones_like(aux_loss) * MoEAuxLossAutoScaler.main_loss_backward_scale

    @staticmethod
    def set_loss_scale(scale: float):
        MoEAuxLossAutoScaler.main_loss_backward_scale = float(scale)


class AuxLossTracker:
    """Per-layer record of auxiliary losses for logging (``save_to_aux_losses_tracker``,
    router.py:270-275,295-300)."""
    values = {}

    @classmethod
    def save(cls, name: str, loss: torch.Tensor, layer_number: int, num_layers: int):
        if torch._C._current_graph_task_id() != -1:
            return      # a forward pass replayed inside backward (activation recompute): already recorded once
        if name not in cls.values:
            cls.values[name] = torch.zeros(num_layers, device=loss.device)
        if cls.values[name].device != loss.device or cls.values[name].numel() != num_layers:
            cls.values[name] = torch.zeros(num_layers, device=loss.device)
        cls.values[name][layer_number - 1] += loss.detach().float()

    @classmethod
    def pop(cls):
        out = {k: v.clone() for k, v in cls.values.items()}
        for v in cls.values.values():
            v.zero_()
        return out


def get_capacity(num_tokens: int, num_experts: int, capacity_factor: float, min_capacity: Optional[int] = None) -> int:
    cap = math.ceil(num_tokens / num_experts * capacity_factor)
    if min_capacity is not None and cap < min_capacity:
        cap = min_capacity
    return cap


class TopKRouter(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 device=None):
        super().__init__()
        self.cfg, self.mesh, self.layer_number = cfg, mesh or single_process_mesh(), layer_number
        self.E, self.k = cfg.num_experts, cfg.moe_topk
        # replicated on every rank; its gradient is summed over TP by the data-parallel reducer because
        # each TP rank routes a different slice of the sequence (router.py:134-139 'sequence_parallel' tag)
        self.weight = nn.Parameter(init_normal((self.E, cfg.hidden_size), cfg.init_method_std, key + ".weight",
                                               device).to(cfg.params_dtype))
        self.weight.sequence_parallel_grad = True

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x ``[T, h]`` -> (probs ``[T, k]`` fp32, indices ``[T, k]`` int64)."""
        cfg = self.cfg
        if self.training and cfg.moe_input_jitter_eps:
            eps = cfg.moe_input_jitter_eps
            x = x * torch.empty_like(x).uniform_(1.0 - eps, 1.0 + eps)
        logits = ops.linear(x, self.weight.to(x.dtype)).float()
        if self.training and cfg.moe_z_loss_coeff:
            zl = R.z_loss(logits, cfg.moe_z_loss_coeff / self.mesh.tp)
            logits = MoEAuxLossAutoScaler.apply(logits, zl)
            AuxLossTracker.save("z_loss", zl / cfg.moe_z_loss_coeff, self.layer_number, cfg.num_layers)
        if cfg.moe_router_load_balancing_type == "sinkhorn":
            return self._sinkhorn(logits)
        probs, idx, full = ops.router_topk(logits, self.k, cfg.moe_router_order)
        if self.training and cfg.moe_router_load_balancing_type == "aux_loss" and cfg.moe_aux_loss_coeff:
            coeff = cfg.moe_aux_loss_coeff / self.mesh.tp            # router.py:264-269
            aux = R.switch_load_balancing_loss(full, idx, self.E, coeff)
            probs = MoEAuxLossAutoScaler.apply(probs, aux)
            AuxLossTracker.save("load_balancing_loss", aux / coeff, self.layer_number, cfg.num_layers)
        cf = cfg.moe_train_capacity_factor if self.training else (cfg.moe_eval_capacity_factor or
                                                                  cfg.moe_train_capacity_factor)
        if cfg.moe_token_dropping and cf is not None:
            probs, idx = self._apply_capacity(probs, idx, cf)
        return probs, idx

    def _sinkhorn(self, logits):
        assert self.cfg.moe_aux_loss_coeff == 0, "sinkhorn routing does not support an aux loss"
        if self.training:
            with torch.no_grad():
                norm = R.sinkhorn(logits.float())
                _, idx = torch.topk(norm, self.k, dim=1)
            act = torch.sigmoid(logits) if self.k == 1 else torch.softmax(logits, dim=-1)
            return torch.gather(act, 1, idx), idx
        act = torch.sigmoid(logits) if self.k == 1 else torch.softmax(logits, dim=-1)
        p, idx = torch.topk(act, self.k, dim=1)
        return p, idx

    def _apply_capacity(self, probs, idx, capacity_factor):
        """Drop assignments beyond each expert's capacity.  ``probs`` policy keeps the highest-probability
        tokens of an expert, ``position`` the earliest (router.py:77-115).  Dropped slots get probability 0
        and index -1."""
        cfg = self.cfg
        T, k = idx.shape
        cap = get_capacity(T * k, self.E, capacity_factor, cfg.moe_min_capacity)
        flat_e = idx.reshape(-1)
        score = probs.reshape(-1) if cfg.moe_token_drop_policy == "probs" else \
            -torch.arange(T * k, device=idx.device, dtype=torch.float32)
        order = torch.argsort(score, descending=True, stable=True)
        e_sorted = flat_e[order]
        order2 = torch.argsort(e_sorted, stable=True)
        e2 = e_sorted[order2]
        counts = torch.bincount(e2, minlength=self.E)
        starts = torch.cumsum(counts, 0) - counts
        rank_in_e = torch.arange(T * k, device=idx.device) - starts[e2]
        keep2 = rank_in_e < cap
        keep = torch.zeros(T * k, dtype=torch.bool, device=idx.device)
        keep[order[order2]] = keep2
        keep = keep.reshape(T, k)
        return probs * keep.to(probs.dtype), torch.where(keep, idx, torch.full_like(idx, -1))


class GroupedExperts(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Mesh, key: str, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh
        E, ep, tp = cfg.num_experts, mesh.ep, mesh.tp
        assert E % ep == 0
        self.El = E // ep
        f = cfg.moe_ffn_hidden_size
        assert f % tp == 0
        fl = f // tp
        h, std, dt = cfg.hidden_size, cfg.init_method_std, cfg.params_dtype
        std2 = std / math.sqrt(2.0 * cfg.num_layers)
        w1, w2 = [], []
        for le in range(self.El):
            ge = mesh.ep_rank * self.El + le                      # global expert id
            fc1 = init_normal((2 * f, h), std, f"{key}.local_experts.{ge}.linear_fc1.weight", device)
            fc2 = init_normal((h, f), std2, f"{key}.local_experts.{ge}.linear_fc2.weight", device)
            if tp > 1:
                r = mesh.tp_rank
                gate, up = fc1[:f], fc1[f:]
                fc1 = torch.cat([gate[r * fl:(r + 1) * fl], up[r * fl:(r + 1) * fl]], 0)
                fc2 = fc2[:, r * fl:(r + 1) * fl]
            w1.append(fc1.t().contiguous())                       # [h, 2fl]
            w2.append(fc2.t().contiguous())                       # [fl, h]
        self.weight1 = nn.Parameter(torch.stack(w1).to(dt))       # [El, h, 2fl]
        self.weight2 = nn.Parameter(torch.stack(w2).to(dt))       # [El, fl, h]
        for p in (self.weight1, self.weight2):
            p.expert_parallel = True                              # reduced over the edp group only
            p.tensor_parallel = tp > 1

    def forward(self, x_sorted: torch.Tensor, tokens_per_expert) -> torch.Tensor:
        if x_sorted.shape[0] == 0:
            # keep the weights in the graph so that their (zero) gradients exist (experts.py:169-180)
            return x_sorted @ self.weight1[0, :, : self.weight2.shape[1]].to(x_sorted.dtype) @ \
                self.weight2[0].to(x_sorted.dtype)
        return ops.grouped_mlp(x_sorted, tokens_per_expert, self.weight1, self.weight2)


def permute(tokens: torch.Tensor, idx: torch.Tensor, num_experts: int):
    """Replicate each token to its k experts and sort by expert id (dropped slots, id -1, are removed).
    Returns (permuted ``[N, h]``, sort order into the flattened (token, slot) list, tokens per expert)."""
    T, k = idx.shape
    flat = idx.reshape(-1)
    valid = flat >= 0
    key = torch.where(valid, flat, torch.full_like(flat, num_experts))
    order = torch.argsort(key, stable=True)
    n_valid = int(valid.sum()) if not bool(valid.all()) else T * k
    order = order[:n_valid]
    permuted = tokens.index_select(0, order // k)
    counts = torch.bincount(flat[order], minlength=num_experts)
    return permuted, order, counts


def unpermute(expert_out: torch.Tensor, order: torch.Tensor, probs: torch.Tensor, T: int, k: int) -> torch.Tensor:
    """Scale expert outputs by their routing probability and sum the k copies of each token
    (token_dispatcher.py:533-539)."""
    w = probs.reshape(-1).index_select(0, order).to(torch.float32)
    out = torch.zeros(T, expert_out.shape[-1], dtype=torch.float32, device=expert_out.device)
    out.index_add_(0, order // k, expert_out.float() * w[:, None])
    return out.to(expert_out.dtype)


class MoELayer(nn.Module):
    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, layer_number: int = 1, key: str = "",
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg, self.mesh = cfg, mesh or single_process_mesh()
        mesh = self.mesh
        self.sp = sequence_parallel and mesh.tp > 1
        assert mesh.tp == 1 or self.sp, "MoE with tensor parallelism requires sequence parallelism"
        self.router = TopKRouter(cfg, mesh, layer_number, key + ".router", device)
        self.experts = GroupedExperts(cfg, mesh, key + ".experts", device)
        self.E, self.El, self.k = cfg.num_experts, self.experts.El, cfg.moe_topk
        if cfg.enable_shared_expert and cfg.shared_moe_ffn_hidden_size:
            self.shared_expert = MLP(cfg, mesh, key + ".shared_expert", ffn=cfg.shared_moe_ffn_hidden_size,
                                     sequence_parallel=sequence_parallel, device=device)
            if cfg.shared_expert_gate:
                self.shared_expert_gate = nn.Module()
                self.shared_expert_gate.weight = nn.Parameter(
                    init_normal((1, cfg.hidden_size), cfg.init_method_std, key + ".shared_expert_gate.weight",
                                device).to(cfg.params_dtype))
                self.shared_expert_gate.weight.sequence_parallel_grad = True
            else:
                self.shared_expert_gate = None
        else:
            self.shared_expert = None

    # ------------------------------------------------------------------
    def _fused_workspace(self, h: torch.Tensor):
        """The peer-memory exchange applies to bf16 CUDA tokens on an expert-parallel group without expert TP."""
        mesh = self.mesh
        if not (h.is_cuda and h.dtype == torch.bfloat16) or self.k * mesh.tp > 16:
            return None
        from ..ops import gemm
        from ..parallel import fused_comm
        if not gemm.supports_grouped(h, self.experts.weight1, self.experts.weight2) or h.shape[-1] % 8:
            return None
        if not mesh["tp"].is_trivial:
            # experts are ffn-sharded over TP: every (expert, TP shard) pair is a virtual expert of the TP x EP group
            ws = fused_comm.moe_workspace(mesh["tp_ep"])
            if ws is None or ws.h != h.shape[-1] or ws.E != self.E * mesh.tp:
                return None
            return ws
        if mesh["ep"].is_trivial:
            if os.environ.get("LMOE_FUSED_MOE", "1") == "0":
                return None
            rows = h.shape[0] * self.k + gemm.ROW_ALIGN * self.E
            return fused_comm.local_moe_workspace(self.E, h.shape[-1], rows, h.device)
        ws = fused_comm.moe_workspace(mesh["ep"])
        if ws is None or ws.h != h.shape[-1] or ws.E != self.E:
            return None
        return ws

    def _experts_with_ep(self, permuted: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """Expert computation on expert-sorted tokens, exchanging them over the EP group."""
        mesh = self.mesh
        ep, tpg = mesh["ep"], mesh["tp"]
        if ep.is_trivial and tpg.is_trivial:
            return self.experts(permuted, counts)
        W, El = ep.size, self.El
        if not ep.is_trivial:
            # counts[e] tokens for global expert e; rank r owns experts [r*El, (r+1)*El)
            all_counts = C.all_gather_raw(counts[None], ep, dim=0)                     # [W, E]
            recv = all_counts[:, ep.rank * El:(ep.rank + 1) * El]                      # [W(src), El]
            in_splits = counts.reshape(W, El).sum(1).tolist()                          # host sync
            out_splits = recv.sum(1).tolist()
            got = C.all_to_all(permuted, ep, out_splits, in_splits)                    # ordered (src, local expert)
            # regroup to (local expert, src)
            seg = recv.reshape(-1)                                                     # [W*El] segment lengths
            seg_id = torch.repeat_interleave(torch.arange(W * El, device=got.device), seg)
            local_e = seg_id % El
            order2 = torch.argsort(local_e, stable=True)
            got = got.index_select(0, order2)
            local_counts = recv.sum(0)
        else:
            got, local_counts, order2 = permuted, counts, None
        if not tpg.is_trivial:
            # every TP rank needs all tokens of the local experts: gather along tokens, experts are
            # ffn-sharded, partial outputs are reduce-scattered back
            n_loc = torch.tensor([got.shape[0]], device=got.device)
            n_all = C.all_gather_raw(n_loc, tpg, dim=0).tolist()
            cnt_all = C.all_gather_raw(local_counts[None], tpg, dim=0)                 # [tp, El]
            pad = max(n_all)
            gp = F.pad(got, (0, 0, 0, pad - got.shape[0]))
            allg = C.all_gather(gp, tpg, dim=0).reshape(tpg.size, pad, -1)
            parts = [allg[r, : n_all[r]] for r in range(tpg.size)]
            cat = torch.cat(parts, 0)
            eid = torch.cat([torch.repeat_interleave(torch.arange(El, device=got.device), cnt_all[r])
                             for r in range(tpg.size)])
            o3 = torch.argsort(eid, stable=True)
            y = self.experts(cat.index_select(0, o3), cnt_all.sum(0))
            inv3 = torch.empty_like(o3)
            inv3[o3] = torch.arange(o3.numel(), device=o3.device)
            y = y.index_select(0, inv3)
            ys = list(y.split(n_all, 0))
            ypad = torch.stack([F.pad(t, (0, 0, 0, pad - t.shape[0])) for t in ys], 0).reshape(tpg.size * pad, -1)
            out = C.reduce_scatter(ypad, tpg, dim=0)[: got.shape[0]]
        else:
            out = self.experts(got, local_counts)
        if not ep.is_trivial:
            inv2 = torch.empty_like(order2)
            inv2[order2] = torch.arange(order2.numel(), device=order2.device)
            out = out.index_select(0, inv2)
            out = C.all_to_all(out, ep, in_splits, out_splits)
        return out

    def _experts_allgather(self, h: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """All-gather token dispatcher (``--moe-token-dispatcher-type allgather``, token_dispatcher.py:69-291): every
        rank of the TP x EP group gathers all tokens and their routing, keeps the copies routed to its local experts,
        runs them, and the weighted outputs are reduce-scattered back to the token owners (which also sums the partial
        outputs of tensor-parallel expert shards)."""
        mesh = self.mesh
        g = mesh["tp_ep"] if not mesh["tp"].is_trivial else mesh["ep"]
        T = h.shape[0]
        if g.is_trivial:
            permuted, order, counts = permute(h, idx, self.E)
            return unpermute(self.experts(permuted, counts), order, probs, T, self.k)
        h_all = C.all_gather(h, g, dim=0)                                     # backward: reduce-scatter of the gradients
        probs_all = C.all_gather(probs, g, dim=0)
        idx_all = C.all_gather_raw(idx.contiguous(), g, dim=0)
        lo = mesh.ep_rank * self.El
        local = (idx_all >= lo) & (idx_all < lo + self.El)
        idx_loc = torch.where(local, idx_all - lo, torch.full_like(idx_all, -1))
        permuted, order, counts = permute(h_all, idx_loc, self.El)
        y = self.experts(permuted, counts)
        out_all = unpermute(y, order, probs_all, h_all.shape[0], self.k)
        return C.reduce_scatter(out_all, g, dim=0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        h = x.reshape(-1, shape[-1])
        T = h.shape[0]
        probs, idx = self.router(h)
        if self.cfg.moe_token_dispatcher_type == "allgather":
            out = self._experts_allgather(h, probs, idx).reshape(shape)
            ws = False
        else:
            ws = self._fused_workspace(h)
        if ws is False:
            pass
        elif ws is not None:
            from ..ops.moe_fused import fused_moe
            tp = self.mesh.tp
            if tp > 1:
                # token -> all TP shards of its experts; the partial outputs of the shards are summed by the combine.
                # Rank g = ep_rank * tp + tp_rank of the TP x EP group owns virtual experts [g * El, (g + 1) * El).
                El = self.El
                base = torch.div(idx, El, rounding_mode="floor") * (tp * El) + idx % El
                idx_v = torch.stack([base + r * El for r in range(tp)], dim=-1)
                idx_v = torch.where(idx[..., None] >= 0, idx_v, torch.full_like(idx_v, -1)).reshape(T, self.k * tp)
                probs_v = probs.repeat_interleave(tp, dim=1)
                out = fused_moe(h, probs_v, idx_v, self.experts.weight1, self.experts.weight2, ws).reshape(shape)
            else:
                out = fused_moe(h, probs, idx, self.experts.weight1, self.experts.weight2, ws).reshape(shape)
        else:
            permuted, order, counts = permute(h, idx, self.E)
            y = self._experts_with_ep(permuted, counts)
            out = unpermute(y, order, probs, T, self.k).reshape(shape)
        if self.shared_expert is not None:
            s = self.shared_expert(x)
            if self.shared_expert_gate is not None:
                out = ops.gated_add(out, s, F.linear(x, self.shared_expert_gate.weight.to(x.dtype)))
            else:
                out = out + s
        return out

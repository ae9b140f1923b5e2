"""CPU oracle tests of the MoE building blocks: router orders, auxiliary losses, sinkhorn, capacity, permute / unpermute,
the MoE layer against a per-token loop over its experts, and expert parallelism over gloo ranks against one rank."""
import math

import pytest
import torch

from linear_moe_b200.config.model_config import ModelConfig, ParallelConfig
from linear_moe_b200.models import moe as M
from linear_moe_b200.ref import ops as R

from dist_utils import run_distributed


def test_router_orders():
    torch.manual_seed(0)
    logits = torch.randn(50, 8)
    p, idx, full = R.router_topk(logits, 2, "softmax_topk")
    assert torch.allclose(full.sum(-1), torch.ones(50), atol=1e-6)
    assert torch.equal(idx, logits.topk(2, -1).indices)
    assert torch.allclose(p, full.gather(1, idx)) and bool((p.sum(-1) < 1).all())      # no renormalisation over the k
    p2, idx2, _ = R.router_topk(logits, 2, "topk_softmax")
    assert torch.equal(idx2, idx) and torch.allclose(p2.sum(-1), torch.ones(50), atol=1e-6)


def test_aux_and_z_loss_values():
    T, E, k = 64, 4, 2
    # perfectly balanced routing with uniform probabilities: loss = coeff (E * sum_e (1/E)(1/E) = 1)
    full = torch.full((T, E), 1.0 / E)
    idx = torch.stack([torch.arange(T) % E, (torch.arange(T) + 1) % E], 1)
    assert math.isclose(R.switch_load_balancing_loss(full, idx, E, 0.01).item(), 0.01, rel_tol=1e-6)
    # probability 1 on expert 0, slots on experts 0 and 1: mean prob = (1,0,0,0), token share = (1/2,1/2,0,0) -> E * 1/2
    full = torch.zeros(T, E)
    full[:, 0] = 1.0
    idx = torch.stack([torch.zeros(T, dtype=torch.long), torch.ones(T, dtype=torch.long)], 1)
    assert math.isclose(R.switch_load_balancing_loss(full, idx, E, 1.0).item(), E * 0.5, rel_tol=1e-6)
    logits = torch.zeros(T, E)
    assert math.isclose(R.z_loss(logits, 2.0).item(), 2.0 * math.log(E) ** 2, rel_tol=1e-6)


def test_sinkhorn_balances_columns():
    torch.manual_seed(1)
    cost = torch.randn(128, 8)
    out = R.sinkhorn(cost, tol=1e-6, max_iter=500)
    assert torch.allclose(out.sum(0), torch.full((8,), 1.0 / 8), atol=1e-3)
    assert torch.allclose(out.sum(1), torch.full((128,), 1.0 / 128), atol=1e-3)


def test_capacity():
    assert M.get_capacity(100, 8, 1.0) == 13
    assert M.get_capacity(100, 8, 1.25) == 16
    assert M.get_capacity(8, 8, 1.0, min_capacity=4) == 4


def test_permute_unpermute_roundtrip_and_drops():
    torch.manual_seed(2)
    T, k, E, h = 37, 2, 5, 6
    x = torch.randn(T, h)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    perm, order, counts = M.permute(x, idx, E)
    assert perm.shape == (T * k, h) and int(counts.sum()) == T * k
    assert torch.equal(counts, torch.bincount(idx.reshape(-1), minlength=E))
    experts_of_rows = idx.reshape(-1)[order]
    assert bool((experts_of_rows[1:] >= experts_of_rows[:-1]).all())                  # sorted by expert, stable
    probs = torch.rand(T, k)
    y = M.unpermute(perm, order, probs, T, k)                                          # identity experts
    assert torch.allclose(y, x * probs.sum(-1, keepdim=True), atol=1e-6)
    idx2 = idx.clone()
    idx2[::3, 1] = -1                                                                 # dropped slots
    perm2, order2, counts2 = M.permute(x, idx2, E)
    n = int((idx2 >= 0).sum())
    assert perm2.shape[0] == n and int(counts2.sum()) == n
    y2 = M.unpermute(perm2, order2, probs, T, k)
    w = torch.where(idx2 >= 0, probs, torch.zeros_like(probs)).sum(-1, keepdim=True)
    assert torch.allclose(y2, x * w, atol=1e-6)


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=32, num_attention_heads=2, ffn_hidden_size=64, vocab_size=128, num_experts=4,
                moe_topk=2, moe_ffn_hidden_size=48, params_dtype=torch.float32, moe_aux_loss_coeff=0.0)
    base.update(kw)
    return ModelConfig(**base)


@pytest.mark.parametrize("shared", [False, True])
def test_moe_layer_matches_per_token_loop(shared):
    """MoE layer output = sum over the token's k experts of prob * SwiGLU-MLP_e(x), plus the (gated) shared expert."""
    torch.manual_seed(3)
    kw = dict(enable_shared_expert=True, shared_moe_ffn_hidden_size=40, shared_expert_gate=True) if shared else {}
    cfg = _cfg(**kw)
    layer = M.MoELayer(cfg, None, 1, "layers.0.mlp").eval()
    assert (layer.shared_expert is not None) == shared
    x = torch.randn(2, 9, 32)
    with torch.no_grad():
        y = layer(x).reshape(-1, 32)
        flat = x.reshape(-1, 32)
        probs, idx = layer.router(flat)
        w1, w2 = layer.experts.weight1, layer.experts.weight2                         # [E, h, 2f], [E, f, h]
        ref = torch.zeros_like(flat)
        for t in range(flat.shape[0]):
            for s in range(cfg.moe_topk):
                e = int(idx[t, s])
                ref[t] += probs[t, s] * (R.swiglu(flat[t] @ w1[e]) @ w2[e])
        if shared:
            sh = layer.shared_expert(x).reshape(-1, 32)
            gate = torch.sigmoid(flat @ layer.shared_expert_gate.weight.t())
            ref = ref + gate * sh
    assert torch.allclose(y, ref, atol=1e-5), (y - ref).abs().max()


def _ep_worker(rank, world, seed):
    from linear_moe_b200.dist.mesh import Mesh
    mesh = Mesh(ParallelConfig(expert_model_parallel_size=world))
    cfg = _cfg(num_experts=4)
    layer = M.MoELayer(cfg, mesh, 1, "layers.0.mlp").train()
    g = torch.Generator().manual_seed(seed + rank)                                     # each data-parallel rank has its own tokens
    x = torch.randn(1, 11, 32, generator=g, requires_grad=True)
    y = layer(x)
    y.square().sum().backward()
    return x.detach(), y.detach(), x.grad


def test_expert_parallel_matches_one_rank():
    """EP=2: every rank routes its own tokens to experts on both ranks; outputs and input gradients equal a single
    rank that holds all four experts (parameters are seeded by name, so both layouts hold the same weights)."""
    outs = run_distributed(_ep_worker, 2, seed=5)
    cfg = _cfg(num_experts=4)
    layer = M.MoELayer(cfg, None, 1, "layers.0.mlp").train()
    for x, y, gx in outs:
        x1 = x.clone().requires_grad_(True)
        y1 = layer(x1)
        y1.square().sum().backward()
        assert torch.allclose(y1, y, atol=1e-5), (y1 - y).abs().max()
        assert torch.allclose(x1.grad, gx, atol=1e-5)

"""Blocked composition of the square-state scan (ops/lsm_blocked.py) against the unblocked definition, on CPU."""
import pytest
import torch

from linear_moe_b200.ops import lsm_torch as LT
from linear_moe_b200.ops.lsm_blocked import blocked_scalar, narrow_columns
from linear_moe_b200.ref import lsm as RL


def _inner(calls):
    def run(q, k, v, g, scale, init, chunk):
        assert q.shape[-1] == k.shape[-1] == v.shape[-1] and q.shape[-1] in (64, 128)
        if init is not None:
            assert init.shape[-2:] == (q.shape[-1], v.shape[-1])
        calls.append(q.shape[-1])
        return LT.chunk_scalar_gated(q, k, v, g, scale, init, chunk)
    return run


@pytest.mark.parametrize("Fd,Dv,gkind,init,ncalls", [
    (153, 129, None, True, 2),        # Based features + the normaliser's ones column: 2 key blocks, column by cumsum
    (153, 64, "head", False, 2),      # decay: everything through the blocks
    (40, 33, None, True, 1),          # 64-wide instantiation, remainder wider than the cumsum form -> padded
    (136, 130, "token", True, 4),     # data-dependent decay: the remainder is padded, 2 x 2 blocks
    (128, 260, None, False, 2),       # wide values, 4-column remainder by cumsum
])
def test_blocked_matches_definition(Fd, Dv, gkind, init, ncalls):
    torch.manual_seed(0)
    B, T, H = 2, 70, 3
    dt = torch.float64
    q = torch.randn(B, T, H, Fd, dtype=dt, requires_grad=True)
    k = (torch.randn(B, T, H, Fd, dtype=dt) * 0.3).requires_grad_(True)
    v = torch.randn(B, T, H, Dv, dtype=dt, requires_grad=True)
    g = None
    if gkind == "head":
        g = -torch.rand(H, dtype=dt) * 0.1
    elif gkind == "token":
        g = (-torch.rand(B, T, H, dtype=dt) * 0.2).requires_grad_(True)
    s0 = torch.randn(B, H, Fd, Dv, dtype=dt, requires_grad=True) if init else None
    calls = []
    o, S = blocked_scalar(_inner(calls), q, k, v, g, None, s0, 16)
    assert len(calls) == ncalls and o.shape == v.shape and S.shape == (B, H, Fd, Dv)
    gg = g if (g is None or g.dim() == 3) else g[None, None, :].expand(B, T, H)
    o_ref, S_ref = RL.recurrent_lsm(q, k, v, g=gg, scale=Fd ** -0.5, initial_state=s0)
    # the composition runs in fp32 internally (as the kernels do)
    assert torch.allclose(o, o_ref.to(o.dtype), rtol=2e-4, atol=2e-4)
    assert torch.allclose(S.double(), S_ref.double(), rtol=2e-4, atol=2e-4)
    go, gS = torch.randn_like(o), torch.randn_like(S)
    leaves = [t for t in (q, k, v, g if gkind == "token" else None, s0) if t is not None]
    got = torch.autograd.grad((o * go).sum() + (S * gS).sum(), leaves)
    want = torch.autograd.grad((o_ref * go).sum() + (S_ref * gS.to(S_ref.dtype)).sum(), leaves)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, rtol=5e-4, atol=5e-4), (a - b).abs().max()


def test_narrow_columns_is_the_cumulative_sum_form():
    torch.manual_seed(1)
    B, T, H, Fd = 2, 33, 2, 20
    q, k = torch.randn(B, T, H, Fd), torch.randn(B, T, H, Fd)
    v = torch.randn(B, T, H, 2)
    s0 = torch.randn(B, H, Fd, 2)
    o, S = narrow_columns(q, k, v, 0.5, s0)
    o_ref, S_ref = RL.recurrent_lsm(q, k, v, scale=0.5, initial_state=s0)
    assert torch.allclose(o, o_ref.float(), rtol=1e-4, atol=1e-4) and torch.allclose(S, S_ref.float(), rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("Fd,Dv,gkind", [(153, 129, None), (153, 128, "head"), (40, 33, None)])
def test_blocked_kernels_on_gpu(Fd, Dv, gkind):
    """Based / normalised shapes through the scan kernels: outputs, state and gradients against the fp32 recurrence."""
    from linear_moe_b200 import ops
    torch.manual_seed(2)
    dev = torch.device("cuda", 0)
    B, T, H = 2, 300, 4
    q = torch.rand(B, T, H, Fd, device=dev).bfloat16().requires_grad_(True)          # positive features (Taylor map)
    k = (torch.rand(B, T, H, Fd, device=dev) * 0.2).bfloat16().requires_grad_(True)
    v = torch.randn(B, T, H, Dv, device=dev).bfloat16().requires_grad_(True)
    g = None if gkind is None else -torch.rand(H, device=dev) * 0.05
    s0 = torch.randn(B, H, Fd, Dv, device=dev) * 0.1
    o, S = ops.lsm_scalar(q, k, v, g, 1.0, s0, 64)
    go = torch.randn_like(o)
    (o.float() * go.float()).sum().backward()
    qf, kf, vf = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    gg = None if g is None else g[None, None, :].expand(B, T, H)
    o_ref, S_ref = RL.recurrent_lsm(qf, kf, vf, g=gg, scale=1.0, initial_state=s0)
    (o_ref * go.float()).sum().backward()
    rel = lambda a, r: ((a.float() - r.float()).norm() / r.float().norm().clamp_min(1e-9)).item()
    assert rel(o, o_ref) < 2e-2 and rel(S, S_ref) < 1e-2, (rel(o, o_ref), rel(S, S_ref))
    for a, r in zip((q, k, v), (qf, kf, vf)):
        assert rel(a.grad, r.grad) < 3e-2, rel(a.grad, r.grad)

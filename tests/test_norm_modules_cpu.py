"""Norm modules with the reference's call contract (``forward(x, residual, prenorm, residual_in_fp32)``) and their fused
norm + linear forms, against plain PyTorch definitions on CPU."""
import pytest
import torch
import torch.nn.functional as F

from linear_moe_b200.models.norms import (GroupNorm, GroupNormLinear, LayerNorm, LayerNormLinear, RMSNorm,
                                           RMSNormLinear)


def _ref_norm(kind, h, w, b, eps, groups=None):
    if kind == "rms":
        y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    elif kind == "layer":
        y = F.layer_norm(h, h.shape[-1:], None, None, eps)
    else:
        g = h.reshape(*h.shape[:-1], groups, -1)
        y = F.layer_norm(g, g.shape[-1:], None, None, eps).reshape(h.shape)
    if w is not None:
        y = y * w
    if b is not None:
        y = y + b
    return y


@pytest.mark.parametrize("kind", ["rms", "layer", "group"])
@pytest.mark.parametrize("with_residual,prenorm", [(False, False), (True, True), (True, False)])
@pytest.mark.parametrize("bias", [False, True])
def test_norm_modules_match_definitions(kind, with_residual, prenorm, bias):
    torch.manual_seed(0)
    N = 32
    cls = {"rms": RMSNorm, "layer": LayerNorm, "group": GroupNorm}[kind]
    m = cls(4, N, bias=bias, eps=1e-5) if kind == "group" else cls(N, bias=bias, eps=1e-5)
    with torch.no_grad():
        m.weight.copy_(1 + 0.1 * torch.randn(N))
        if m.bias is not None:
            m.bias.copy_(0.1 * torch.randn(N))
    x = torch.randn(3, 7, N, requires_grad=True)
    r = torch.randn(3, 7, N) if with_residual else None
    out = m(x, residual=r, prenorm=prenorm)
    y, stream = out if prenorm else (out, None)
    h = x if r is None else x + r
    want = _ref_norm(kind, h, m.weight, m.bias, 1e-5, 4)
    assert torch.allclose(y, want, atol=1e-5)
    if prenorm:
        assert torch.allclose(stream, h)
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()


@pytest.mark.parametrize("kind", ["rms", "layer", "group"])
def test_norm_linear_recomputes_and_matches(kind):
    """The fused norm + linear modules give the output and every gradient of norm followed by ``F.linear`` while saving
    only their inputs (the normalised activation is recomputed in backward)."""
    torch.manual_seed(1)
    N, O = 32, 24
    cls = {"rms": RMSNormLinear, "layer": LayerNormLinear, "group": GroupNormLinear}[kind]
    m = cls(4, N, bias=True) if kind == "group" else cls(N, bias=True)
    with torch.no_grad():
        m.weight.copy_(1 + 0.1 * torch.randn(N))
        m.bias.copy_(0.1 * torch.randn(N))
    x = torch.randn(5, 6, N, requires_grad=True)
    res = torch.randn(5, 6, N, requires_grad=True)
    w = (torch.randn(O, N) / N ** 0.5).requires_grad_(True)
    b = torch.randn(O).requires_grad_(True)
    out, stream = m(x, w, b, residual=res, prenorm=True)
    go = torch.randn_like(out)
    (out * go).sum().backward()
    got = [t.grad.clone() for t in (x, res, w, b, m.weight, m.bias)]
    for t in (x, res, w, b, m.weight, m.bias):
        t.grad = None
    h = x + res
    want = F.linear(_ref_norm(kind, h, m.weight, m.bias, m.eps, 4), w, b)
    assert torch.allclose(out, want, atol=1e-5) and torch.allclose(stream, h)
    (want * go).sum().backward()
    for a, t in zip(got, (x, res, w, b, m.weight, m.bias)):
        assert torch.allclose(a, t.grad, atol=1e-4), (kind, (a - t.grad).abs().max())
    # forward-only call takes the plain path
    with torch.no_grad():
        assert torch.allclose(m(x, w, b, residual=res), want, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["rms", "layer", "group"])
def test_norm_linear_modules_on_gpu(kind):
    """The same modules on the CUDA kernels (bf16): output and gradients against the fp32 definition."""
    torch.manual_seed(2)
    dev = torch.device("cuda", 0)
    N, O = 256, 128
    cls = {"rms": RMSNormLinear, "layer": LayerNormLinear, "group": GroupNormLinear}[kind]
    m = (cls(4, N, bias=True) if kind == "group" else cls(N, bias=True)).to(dev).to(torch.bfloat16)
    with torch.no_grad():
        m.weight.copy_(1 + 0.1 * torch.randn(N))
        m.bias.copy_(0.1 * torch.randn(N))
    x = torch.randn(4, 96, N, device=dev).bfloat16().requires_grad_(True)
    res = torch.randn(4, 96, N, device=dev).bfloat16().requires_grad_(True)
    w = (torch.randn(O, N, device=dev) / N ** 0.5).bfloat16().requires_grad_(True)
    b = torch.randn(O, device=dev).bfloat16().requires_grad_(True)
    out, stream = m(x, w, b, residual=res, prenorm=True)
    go = torch.randn_like(out)
    (out.float() * go.float()).sum().backward()
    xf, rf, wf, bf, mw, mb = [t.detach().float().requires_grad_(True) for t in (x, res, w, b, m.weight, m.bias)]
    want = F.linear(_ref_norm(kind, xf + rf, mw, mb, m.eps, 4), wf, bf)
    (want * go.float()).sum().backward()
    rel = lambda a, r: ((a.float() - r).norm() / r.norm().clamp_min(1e-9)).item()
    assert rel(out, want) < 2e-2 and rel(stream, (xf + rf).detach()) < 1e-2
    for a, r in zip((x, res, w, b, m.weight, m.bias), (xf, rf, wf, bf, mw, mb)):
        assert rel(a.grad, r.grad) < 3e-2, (kind, rel(a.grad, r.grad))

"""CUDA kernels against the plain fp32 PyTorch definition of the same operator."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from linear_moe_b200 import ops
from linear_moe_b200.ops import lsm_torch as LT
from linear_moe_b200.ref import lsm as RL
from linear_moe_b200.ref import ops as R
from linear_moe_b200.ops import cuda as K


def dev():
    return torch.device("cuda", 0)


def close(a, b, rtol, atol, name=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert torch.allclose(a, b, rtol=rtol, atol=atol), f"{name}: max abs err {err:.4e} (ref max {ref:.4e})"


def rel_close(a, b, tol, name=""):
    """Relative Frobenius error: a reduced gradient (a sum over rows) that lost one block of partial sums fails this
    even where an absolute tolerance sized for bf16 sums would let it through."""
    a, b = a.float(), b.float()
    rel = ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
    assert rel < tol, f"{name}: relative error {rel:.3e} (limit {tol:.1e})"


def grads(fn, inputs, gout):
    ins = [t.detach().clone().requires_grad_(True) for t in inputs]
    out = fn(*ins)
    outs = out if isinstance(out, (tuple, list)) else (out,)
    g = gout if isinstance(gout, (tuple, list)) else (gout,)
    torch.autograd.backward([o for o, gg in zip(outs, g) if gg is not None], [gg for gg in g if gg is not None])
    return outs, [t.grad for t in ins]


@pytest.mark.parametrize("N,rows", [(2048, 300), (128, 1000), (4096, 64), (1024, 33)])
@pytest.mark.parametrize("residual", [False, True])
def test_rms_norm(N, rows, residual):
    torch.manual_seed(0)
    x = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    r = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(N, device=dev())).to(torch.bfloat16)
    gy = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    gr = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    if residual:
        f_k = lambda x, r, w: ops.add_rms_norm(x, r, w, 1e-6)
        f_r = lambda x, r, w: (R.rms_norm(x + r, w, 1e-6), x + r)
        (y, ro), gk = grads(f_k, [x, r, w], (gy, gr))
        (y2, ro2), gr_ = grads(f_r, [x.float(), r.float(), w.float()], (gy.float(), gr.float()))
        close(ro, ro2, 1e-2, 1e-2, "residual out")
    else:
        f_k = lambda x, w: ops.rms_norm(x, w, 1e-6)
        f_r = lambda x, w: R.rms_norm(x, w, 1e-6)
        (y,), gk = grads(f_k, [x, w], gy)
        (y2,), gr_ = grads(f_r, [x.float(), w.float()], gy.float())
    close(y, y2, 2e-2, 2e-2, "y")
    close(gk[0], gr_[0], 3e-2, 3e-2, "dx")
    rel_close(gk[-1], gr_[-1], 1e-2, "dw")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("norm", [True, False])
def test_head_norm_gate(D, norm):
    torch.manual_seed(1)
    B, T, H = 2, 100, 4
    o = torch.randn(B, T, H, D, device=dev(), dtype=torch.bfloat16)
    g = torch.randn(B, T, H * D, device=dev(), dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(D, device=dev())).to(torch.bfloat16)
    gy = torch.randn(B, T, H * D, device=dev(), dtype=torch.bfloat16)

    def ref(o, w, g):
        y = R.rms_norm(o, w, 1e-5) if norm else o
        return y.reshape(B, T, -1) * F.silu(g)
    (y,), gk = grads(lambda o, w, g: ops.head_norm_gate(o, w, g, 1e-5, "swish", "rmsnorm" if norm else "identity"),
                     [o, w, g], gy)
    (y2,), gr = grads(ref, [o.float(), w.float(), g.float()], gy.float())
    close(y, y2, 2e-2, 2e-2, "y")
    close(gk[0], gr[0], 3e-2, 3e-2, "do")
    close(gk[2], gr[2], 3e-2, 3e-2, "dgate")
    if norm:
        rel_close(gk[1], gr[1], 1e-2, "dw")


def test_gated_rms_norm():
    torch.manual_seed(2)
    rows, N, G = 200, 512, 128
    x = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    z = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(N, device=dev())).to(torch.bfloat16)
    gy = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    (y,), gk = grads(lambda x, z, w: ops.gated_rms_norm(x, z, w, 1e-5, G), [x, z, w], gy)
    (y2,), gr = grads(lambda x, z, w: R.gated_rms_norm(x, z, w, 1e-5, G), [x.float(), z.float(), w.float()], gy.float())
    close(y, y2, 2e-2, 2e-2, "y")
    close(gk[0], gr[0], 3e-2, 3e-2, "dx")
    close(gk[1], gr[1], 3e-2, 3e-2, "dz")
    rel_close(gk[2], gr[2], 1e-2, "dw")


def test_swiglu_l2norm_rope():
    torch.manual_seed(3)
    x = torch.randn(300, 2 * 1408, device=dev(), dtype=torch.bfloat16)
    gy = torch.randn(300, 1408, device=dev(), dtype=torch.bfloat16)
    (y,), gk = grads(ops.swiglu, [x], gy)
    (y2,), gr = grads(R.swiglu, [x.float()], gy.float())
    close(y, y2, 2e-2, 2e-2, "swiglu")
    close(gk[0], gr[0], 3e-2, 3e-2, "dswiglu")
    x = torch.randn(2, 50, 4, 128, device=dev(), dtype=torch.bfloat16)
    gy = torch.randn_like(x)
    (y,), gk = grads(lambda t: ops.l2_norm(t), [x], gy)
    (y2,), gr = grads(lambda t: R.l2_norm(t), [x.float()], gy.float())
    close(y, y2, 2e-2, 2e-2, "l2norm")
    close(gk[0], gr[0], 3e-2, 3e-2, "dl2norm")
    for inter in (False, True):
        for rot in (128, 64):
            cos, sin = R.rope_freqs(50, rot, 10000.0, 7, dev())
            (y,), gk = grads(lambda t: ops.apply_rope(t, cos, sin, inter), [x], gy)
            (y2,), gr = grads(lambda t: R.apply_rope(t, cos, sin, inter), [x.float()], gy.float())
            close(y, y2, 2e-2, 2e-2, "rope")
            close(gk[0], gr[0], 3e-2, 3e-2, "drope")


@pytest.mark.parametrize("cached", [True, False])
def test_linear_cross_entropy(cached, monkeypatch):
    monkeypatch.setattr(ops, "_CE_CACHE_BYTES", (8 << 30) if cached else 0)
    torch.manual_seed(4)
    T, h, V = 700, 256, 32000
    x = (0.5 * torch.randn(T, h, device=dev())).to(torch.bfloat16)
    w = (0.05 * torch.randn(V, h, device=dev())).to(torch.bfloat16)
    lab = torch.randint(0, V, (T,), device=dev())
    lab[::7] = -100
    gl = torch.rand(T, device=dev())
    (l,), gk = grads(lambda x, w: ops.linear_cross_entropy(x, w, lab, -100, 256), [x, w], gl)
    (l2,), gr = grads(lambda x, w: R.linear_cross_entropy(x, w, lab), [x.float(), w.float()], gl)
    close(l, l2, 2e-2, 2e-2, "loss")
    close(gk[0], gr[0], 5e-2, 2e-3, "dh")
    close(gk[1], gr[1], 5e-2, 2e-3, "dw")


@pytest.mark.parametrize("init", [False, True])
def test_causal_conv1d(init):
    torch.manual_seed(5)
    B, T, D, K = 2, 300, 384, 4
    x = torch.randn(B, T, D, device=dev(), dtype=torch.bfloat16)
    w = (0.5 * torch.randn(D, K, device=dev())).to(torch.bfloat16)
    b = (0.1 * torch.randn(D, device=dev())).to(torch.bfloat16)
    s = torch.randn(B, K - 1, D, device=dev(), dtype=torch.bfloat16) if init else None
    gy = torch.randn(B, T, D, device=dev(), dtype=torch.bfloat16)
    ins = [x, w, b] + ([s] if init else [])
    f_k = lambda x, w, b, s=None: ops.causal_conv1d(x, w, b, "silu", s)[0]
    f_r = lambda x, w, b, s=None: R.causal_conv1d(x, w, b, "silu", s)[0]
    (y,), gk = grads(f_k, ins, gy)
    (y2,), gr = grads(f_r, [t.float() for t in ins], gy.float())
    close(y, y2, 2e-2, 2e-2, "y")
    close(gk[0], gr[0], 3e-2, 3e-2, "dx")
    rel_close(gk[1], gr[1], 1e-2, "dw")
    rel_close(gk[2], gr[2], 1e-2, "db")
    if init:
        close(gk[3], gr[3], 3e-2, 3e-2, "dinit")
        close(ops.causal_conv1d(x, w, b, "silu", s)[1], R.causal_conv1d(x, w, b, "silu", s)[1], 0, 0, "tail")


@pytest.mark.parametrize("order", ["softmax_topk", "topk_softmax"])
def test_router(order):
    torch.manual_seed(6)
    T, E, k = 500, 64, 8
    logits = torch.randn(T, E, device=dev())
    gp, gf = torch.randn(T, k, device=dev()), torch.randn(T, E, device=dev())
    (p, i, f), gk = grads(lambda l: ops.router_topk(l, k, order), [logits], (gp, None, gf))
    (p2, i2, f2), gr = grads(lambda l: R.router_topk(l, k, order), [logits], (gp, None, gf))
    assert torch.equal(i, i2)
    close(p, p2, 1e-4, 1e-5, "probs")
    close(f, f2, 1e-4, 1e-5, "full")
    close(gk[0], gr[0], 1e-3, 1e-5, "dlogits")


def test_fused_adam():
    torch.manual_seed(7)
    from linear_moe_b200.ops import cuda as K
    n = 4096 * 3
    p = torch.randn(n, device=dev()).to(torch.bfloat16)
    master = p.float().clone()
    g = torch.randn(n, device=dev())
    m, v = torch.zeros(n, device=dev()), torch.zeros(n, device=dev())
    w2, m2, v2 = master.clone(), m.clone(), v.clone()
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.95, 1e-8, 0.1
    for step in range(1, 4):
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        K.fused_adam(p, master, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, 0.5)
        gg = g * 0.5
        m2.mul_(b1).add_(gg, alpha=1 - b1)
        v2.mul_(b2).addcmul_(gg, gg, value=1 - b2)
        w2.mul_(1 - lr * wd).addcdiv_(m2 / bc1, (v2 / bc2).sqrt() + eps, value=-lr)
    close(master, w2, 1e-5, 1e-6, "master")
    close(p, w2.to(torch.bfloat16), 0, 0, "bf16 copy")


@pytest.mark.parametrize("N,rows", [(2048, 300), (128, 1000), (4096, 64), (1024, 33)])
@pytest.mark.parametrize("residual", [False, True])
def test_layer_norm(N, rows, residual):
    """LayerNorm (+ residual add) kernels against F.layer_norm in fp32: y, dx, dres, dw, db."""
    torch.manual_seed(0)
    x = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    r = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(N, device=dev())).to(torch.bfloat16)
    b = (0.1 * torch.randn(N, device=dev())).to(torch.bfloat16)
    gy = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    gr = torch.randn(rows, N, device=dev(), dtype=torch.bfloat16)
    K.reset_launch_count()
    if residual:
        f_k = lambda x, r, w, b: ops.add_layer_norm(x, r, w, b, 1e-5)
        f_r = lambda x, r, w, b: (R.layer_norm(x + r, w, b, 1e-5), x + r)
        (y, ro), gk = grads(f_k, [x, r, w, b], (gy, gr))
        (y2, ro2), gr_ = grads(f_r, [x.float(), r.float(), w.float(), b.float()], (gy.float(), gr.float()))
        close(ro, ro2, 2e-2, 2e-2, "residual out")
        names = ["dx", "dres", "dw", "db"]
    else:
        f_k = lambda x, w, b: ops.layer_norm(x, w, b, 1e-5)
        f_r = lambda x, w, b: R.layer_norm(x, w, b, 1e-5)
        (y,), gk = grads(f_k, [x, w, b], gy)
        (y2,), gr_ = grads(f_r, [x.float(), w.float(), b.float()], gy.float())
        names = ["dx", "dw", "db"]
    assert K.reset_launch_count() >= 2, "the LayerNorm kernels did not run"
    close(y, y2, 2e-2, 2e-2, "y")
    for name, a_, b_ in zip(names, gk, gr_):
        rel = ((a_.float() - b_).norm() / b_.norm().clamp_min(1e-6)).item()
        assert rel < 2e-2, (name, rel)


def test_group_norm_heads_uses_layer_norm_kernel():
    torch.manual_seed(1)
    o = torch.randn(2, 70, 3, 128, device=dev(), dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(128, device=dev())).to(torch.bfloat16)
    b = (0.1 * torch.randn(128, device=dev())).to(torch.bfloat16)
    K.reset_launch_count()
    y = ops.group_norm_heads(o, w, b, 1e-5)
    assert K.reset_launch_count() == 1
    close(y, R.group_norm_heads(o.float(), w.float(), b.float(), 1e-5), 2e-2, 2e-2, "y")


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("gmode", ["none", "const", "token"])
@pytest.mark.parametrize("T,with_state", [(1000, False), (256, True), (70, True)])
def test_lsm_scalar(D, gmode, T, with_state):
    torch.manual_seed(8)
    B, H = 2, 3
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev())).to(torch.bfloat16)
    q, k, v = qkv.split(D, dim=-1)                    # strided views, as in the model
    g = None
    if gmode == "const":
        g = -torch.tensor([0.02, 0.1, 0.5], device=dev())
    elif gmode == "token":
        g = -0.2 * torch.rand(B, T, H, device=dev())
    S0 = 0.3 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    go = torch.randn(B, T, H, D, device=dev(), dtype=torch.bfloat16)
    gS = 0.1 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    ins = [q, k, v] + ([g] if gmode == "token" else []) + ([S0] if with_state else [])

    def unpack(args):
        args = list(args)
        qq, kk, vv = args[:3]
        rest = args[3:]
        gg = rest.pop(0) if gmode == "token" else g
        ss = rest.pop(0) if with_state else None
        return qq, kk, vv, gg, ss
    f_k = lambda *a: ops.lsm_scalar(*unpack(a)[:4], None, unpack(a)[4], 64)
    f_r = lambda *a: LT.chunk_scalar_gated(*unpack(a)[:4], None, unpack(a)[4], 64)
    (o, S), gk = grads(f_k, ins, (go, gS))
    (o2, S2), gr = grads(f_r, [t.float() for t in ins], (go.float(), gS))
    scale_o = o2.abs().max().item()
    close(o, o2, 3e-2, 2e-2 * scale_o, "o")
    close(S, S2, 3e-2, 2e-2 * S2.abs().max().item(), "final state")
    for name, a, b in zip(["dq", "dk", "dv", "d3", "d4"], gk, gr):
        close(a, b, 5e-2, 3e-2 * b.abs().max().item(), name)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("T,with_state", [(1000, False), (200, True)])
def test_lsm_vector_gla(D, T, with_state):
    torch.manual_seed(9)
    B, H = 2, 3
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev())).to(torch.bfloat16)
    q, k, v = qkv.split(D, dim=-1)
    gk = torch.nn.functional.logsigmoid(2.0 * torch.randn(B, T, H, D, device=dev())) / 4.0      # strong decays
    S0 = 0.3 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    go = torch.randn(B, T, H, D, device=dev(), dtype=torch.bfloat16)
    gS = 0.1 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    ins = [q, k, v, gk] + ([S0] if with_state else [])
    f_k = lambda q, k, v, g, s=None: ops.lsm_vector(q, k, v, g, None, s, None, 64)
    f_r = lambda q, k, v, g, s=None: LT.chunk_vector_gated(q, k, v, g, None, s, 16)
    (o, S), gk_ = grads(f_k, ins, (go, gS))
    (o2, S2), gr = grads(f_r, [t.float() for t in ins], (go.float(), gS))
    close(o, o2, 3e-2, 2e-2 * o2.abs().max().item(), "o")
    close(S, S2, 3e-2, 2e-2 * S2.abs().max().item(), "final state")
    for name, a, b in zip(["dq", "dk", "dv", "dgk", "dS0"], gk_, gr):
        close(a, b, 5e-2, 3e-2 * b.abs().max().item(), name)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("Tq,Tk,q_offset,window,Hq,Hkv", [
    (300, 300, 0, None, 4, 2),           # ragged tiles, grouped-query heads
    (128, 384, 256, None, 2, 2),         # sequence-parallel rank: suffix of the positions against gathered keys
    (1, 200, 199, None, 4, 1),           # decoding against a cache
    (257, 257, 0, 100, 2, 1),            # sliding window
    (1024, 1024, 0, None, 2, 2),         # several key tiles per query tile
])
@pytest.mark.parametrize("tcgen05", [True, False])
def test_flash_attention(D, Tq, Tk, q_offset, window, Hq, Hkv, tcgen05, monkeypatch):
    from linear_moe_b200.ops import flash, gemm
    monkeypatch.setattr(flash, "_TCGEN05_FWD", tcgen05)
    monkeypatch.setattr(flash, "_TCGEN05_BWD", tcgen05)
    torch.manual_seed(11)
    B = 2
    q = torch.randn(B, Tq, Hq, D, device=dev()).to(torch.bfloat16)
    kv = torch.randn(B, Tk, Hkv, 2 * D, device=dev()).to(torch.bfloat16)
    k, v = kv.split(D, dim=-1)                                   # strided views, as out of a fused projection
    go = torch.randn(B, Tq, Hq, D, device=dev()).to(torch.bfloat16)
    assert flash.supported(q, k, v, True, window)
    f_k = lambda q, k, v: flash.FlashAttention.apply(q, k, v, D ** -0.5, q_offset, window)
    f_r = lambda q, k, v: R.softmax_attention(q, k, v, D ** -0.5, True, q_offset, window)
    (o,), gk = grads(f_k, [q, k, v], go)
    gemm.check_error()
    (o2,), gr = grads(f_r, [q.float(), k.float(), v.float()], go.float())
    close(o, o2, 2e-2, 2e-2, "o")
    for name, a, b in zip(["dq", "dk", "dv"], gk, gr):
        close(a, b, 3e-2, 2e-2 * b.abs().max().item(), name)


def test_ssd_mamba2_on_scalar_kernels():
    """Mamba2 SSD (state 128, head dim 64, heads sharing B/C per group, per-token decay) through the scalar-decay
    kernels against the recurrent fp32 definition."""
    torch.manual_seed(2)
    B, T, H, P, N, G = 2, 300, 4, 64, 128, 2
    x = torch.randn(B, T, H, P, device=dev()).to(torch.bfloat16)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, device=dev()) - 1.0)
    A = -torch.exp(torch.randn(H, device=dev()) * 0.5)
    Bm = (0.3 * torch.randn(B, T, G, N, device=dev())).to(torch.bfloat16)
    Cm = (0.3 * torch.randn(B, T, G, N, device=dev())).to(torch.bfloat16)
    Dskip = torch.randn(H, device=dev())
    go = torch.randn(B, T, H, P, device=dev()).to(torch.bfloat16)
    K.reset_launch_count()
    f_k = lambda x, dt, Bm, Cm: ops.ssd(x, dt, A, Bm, Cm, Dskip, None, 64)[0]
    (o,), gk = grads(f_k, [x, dt, Bm, Cm], go)
    assert K.reset_launch_count() > 0

    f_r = lambda x, dt, Bm, Cm: RL.recurrent_ssd(x, dt, A, Bm, Cm, Dskip)[0]
    (o2,), gr = grads(f_r, [x.float(), dt, Bm.float(), Cm.float()], go.float())
    close(o, o2, 3e-2, 2e-2 * o2.abs().max().item(), "y")
    for name, a, b in zip(["dx", "ddt", "dB", "dC"], gk, gr):
        close(a, b, 5e-2, 3e-2 * b.abs().max().item(), name)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [70, 256, 1000])
@pytest.mark.parametrize("gated,with_state", [(True, False), (False, True), (True, True), (False, False)])
def test_lsm_delta_rule_scan(gated, with_state, T, D):
    """(Gated) delta rule on the GPU (chunk-parallel WY tiles + the scan kernels of csrc/lsm_delta.cu, forward and
    backward) against the token-by-token fp32 recurrence: output, final state and every gradient (relative Frobenius
    error), with and without an initial state / a gradient on the final state."""
    torch.manual_seed(4)
    B, H = 2, 2
    q, v = [(0.5 * torch.randn(B, T, H, D, device=dev())).to(torch.bfloat16) for _ in range(2)]
    k = torch.nn.functional.normalize(torch.randn(B, T, H, D, device=dev()), dim=-1).to(torch.bfloat16)
    beta = torch.rand(B, T, H, device=dev())
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev()) + 2.0) if gated else None
    S0 = 0.2 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    go = torch.randn(B, T, H, D, device=dev()).to(torch.bfloat16)
    gS = 0.05 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    ins = [q, k, v, beta] + ([g] if gated else []) + ([S0] if with_state else [])

    def unpack(a):
        a = list(a)
        q, k, v, beta = a[:4]
        gg = a[4] if gated else None
        s = a[-1] if with_state else None
        return q, k, v, beta, gg, s
    K.reset_launch_count()
    f_k = lambda *a: ops.lsm_delta(*unpack(a)[:5], None, unpack(a)[5], 64)
    f_r = lambda *a: RL.recurrent_lsm(unpack(a)[0], unpack(a)[1], unpack(a)[2], beta=unpack(a)[3], g=unpack(a)[4],
                                      initial_state=unpack(a)[5])
    (o, S), gk = grads(f_k, ins, (go, gS))
    assert K.reset_launch_count() >= 2, "the delta-rule scan kernels did not run"
    (o2, S2), gr = grads(f_r, [t.float() for t in ins], (go.float(), gS))

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()
    assert rel(o, o2) < 2e-2, ("o", rel(o, o2))
    assert rel(S, S2) < 2e-2, ("final state", rel(S, S2))
    for name, a, b in zip(["dq", "dk", "dv", "dbeta", "dg/dS0", "dS0"], gk, gr):
        assert rel(a, b) < 3e-2, (name, rel(a, b))


@pytest.mark.gpu
def test_flash_backward_first_node_of_fresh_process():
    """In a fresh process the autograd worker thread has made no runtime call when the flash backward (whose tensor maps
    are encoded by a driver call) is its first node: the kernel wrapper has to bind the context itself."""
    import subprocess
    import sys
    code = ("import torch\n"
            "from linear_moe_b200.ops import flash\n"
            "q = torch.randn(1, 256, 4, 128, device='cuda').bfloat16().requires_grad_(True)\n"
            "kv = torch.randn(1, 256, 2, 256, device='cuda').bfloat16().requires_grad_(True)\n"
            "k, v = kv.split(128, dim=-1)\n"
            "o = flash.FlashAttention.apply(q, k, v, 128 ** -0.5, 0, None)\n"
            "o.backward(torch.ones_like(o))\n"
            "torch.cuda.synchronize()\n"
            "assert torch.isfinite(q.grad.float()).all() and torch.isfinite(kv.grad.float()).all()\n"
            "print('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("gmode", ["none", "per_head", "per_token"])
@pytest.mark.parametrize("with_state", [False, True])
def test_lsm_scalar_decode_step(D, gmode, with_state):
    """One-token step kernel against the recurrence: S' = e^g S + k^T v, o = scale q S'."""
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.ref.lsm import recurrent_lsm
    torch.manual_seed(0)
    B, H = 3, 5
    dev = "cuda"
    qkv = (0.5 * torch.randn(B, 1, H, 3 * D, device=dev)).bfloat16()
    q, k, v = qkv.split(D, dim=-1)                                  # strided views, as the fused projection gives them
    g = {"none": None, "per_head": -torch.rand(H, device=dev),
         "per_token": -torch.rand(B, 1, H, device=dev)}[gmode]
    S0 = torch.randn(B, H, D, D, device=dev) if with_state else None
    with torch.no_grad():
        o, S = K.lsm_scalar(q, k, v, g, None, S0, 64)
    g_ref = None if g is None else (g[None, None, :].expand(B, 1, H) if g.dim() == 1 else g)
    o_ref, S_ref = recurrent_lsm(q.float(), k.float(), v.float(), g=g_ref, initial_state=S0)
    assert o.shape == (B, 1, H, D) and S.shape == (B, H, D, D)
    assert torch.allclose(S, S_ref, atol=1e-4, rtol=1e-4), (S - S_ref).abs().max()
    assert torch.allclose(o.float(), o_ref, atol=3e-2, rtol=2e-2), (o.float() - o_ref).abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("with_state", [False, True])
def test_lsm_vector_decode_step(D, with_state):
    """One-token step with a decay per key channel (GLA / HGRN2) against the recurrence."""
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.ref.lsm import recurrent_lsm
    torch.manual_seed(1)
    B, H = 2, 3
    dev = "cuda"
    q, k, v = [(0.5 * torch.randn(B, 1, H, D, device=dev)).bfloat16() for _ in range(3)]
    gk = -torch.rand(B, 1, H, D, device=dev)
    S0 = torch.randn(B, H, D, D, device=dev) if with_state else None
    with torch.no_grad():
        o, S = K.lsm_vector(q, k, v, gk, None, S0, None, 16)
    o_ref, S_ref = recurrent_lsm(q.float(), k.float(), v.float(), gk=gk, initial_state=S0)
    assert torch.allclose(S, S_ref, atol=1e-4, rtol=1e-4), (S - S_ref).abs().max()
    assert torch.allclose(o.float(), o_ref, atol=3e-2, rtol=2e-2), (o.float() - o_ref).abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("with_state", [False, True])
def test_lsm_delta_decode_step(D, gated, with_state):
    """One-token (gated) delta-rule step against the recurrence."""
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.ref.lsm import recurrent_lsm
    torch.manual_seed(2)
    B, H = 2, 3
    dev = "cuda"
    q, v = [(0.5 * torch.randn(B, 1, H, D, device=dev)).bfloat16() for _ in range(2)]
    k = torch.nn.functional.normalize(torch.randn(B, 1, H, D, device=dev), dim=-1).bfloat16()
    beta = torch.rand(B, 1, H, device=dev)
    g = -torch.rand(B, 1, H, device=dev) if gated else None
    S0 = 0.5 * torch.randn(B, H, D, D, device=dev) if with_state else None
    with torch.no_grad():
        o, S = K.lsm_delta(q, k, v, beta, g, None, S0, 64)
    o_ref, S_ref = recurrent_lsm(q.float(), k.float(), v.float(), g=g, beta=beta, initial_state=S0)
    assert torch.allclose(S, S_ref, atol=2e-4, rtol=1e-4), (S - S_ref).abs().max()
    assert torch.allclose(o.float(), o_ref, atol=3e-2, rtol=2e-2), (o.float() - o_ref).abs().max()


@pytest.mark.parametrize("D,T,gated", [(64, 70, True), (128, 300, True), (128, 256, False)])
def test_delta_prepare_kernel_matches_torch_tiles(D, T, gated):
    """The chunk-parallel tile kernel (K K^T, triangular inverse by substitution, W, U, Q K^T, scaled Q / K) against the
    same tiles built with torch ops in fp32."""
    torch.manual_seed(3)
    B, H = 2, 3
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev())).to(torch.bfloat16)
    q, k, v = qkv.split(D, dim=-1)                                   # strided views
    k = torch.nn.functional.normalize(k.float(), dim=-1).to(torch.bfloat16)
    beta = torch.rand(B, T, H, device=dev())
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev()) + 1.0) if gated else None
    got = K._delta_prepare_kernel(q, k, v, beta, g, D ** -0.5)
    ref = K._delta_prepare(q, k, v, beta, g, D ** -0.5)
    torch.cuda.synchronize()
    for name, a, b in zip(["W", "U", "Qd", "Kd", "A", "gamma"], got, ref):
        rel = ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()
        assert rel < 1e-2, (name, rel)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("main_grad", [False, True])
def test_embedding_backward_scatter(dtype, main_grad):
    """Embedding backward kernel (atomic scatter-add of gradient rows, repeated and out-of-shard ids included) against
    F.embedding's gradient in fp32."""
    torch.manual_seed(0)
    V, h, T = 500, 256, 3000                           # many repeated ids
    w = torch.randn(V, h, device=dev()).to(dtype).requires_grad_(True)
    ids = torch.randint(0, 2 * V, (3, T // 3), device=dev())          # half of them fall outside the shard [0, V)
    gy = torch.randn(3, T // 3, h, device=dev()).to(dtype)
    if main_grad:
        w.main_grad = torch.zeros(V, h, device=dev())
    K.reset_launch_count()
    y = ops.embedding(ids, w, 0, sharded=True)
    y.backward(gy)
    assert K.reset_launch_count() == 1
    wr = w.detach().float().requires_grad_(True)
    inside = ids < V
    yr = torch.nn.functional.embedding(ids.clamp(max=V - 1), wr) * inside[..., None]
    yr.backward(gy.float())
    assert torch.equal(y.float(), yr.detach().to(dtype).float())
    got = w.main_grad if main_grad else w.grad.float()
    rel = ((got - wr.grad).norm() / wr.grad.norm()).item()
    assert rel < (1e-5 if main_grad or dtype == torch.float32 else 5e-3), rel


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gated_add(dtype):
    """``a + s * sigmoid(g)`` (one gate logit per row), forward and the three gradients, against fp32 PyTorch."""
    torch.manual_seed(6)
    a = torch.randn(3, 70, 256, device=dev()).to(dtype)
    s = torch.randn(3, 70, 256, device=dev()).to(dtype)
    g = torch.randn(3, 70, 1, device=dev()).to(dtype)
    go = torch.randn(3, 70, 256, device=dev()).to(dtype)
    K.reset_launch_count()
    (y,), gk = grads(ops.gated_add, [a, s, g], go)
    assert K.reset_launch_count() == 2
    (y2,), gr = grads(lambda a, s, g: a + s * torch.sigmoid(g), [a.float(), s.float(), g.float()], go.float())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    rel_close(y, y2, tol, "out")
    for name, x_, r_ in zip(["da", "ds", "dg"], gk, gr):
        rel_close(x_, r_, tol, name)


@pytest.mark.parametrize("D,T,with_state", [(64, 130, False), (128, 200, True), (64, 1, True)])
def test_lsm_vector_rwkv6_bonus_on_kernels(D, T, with_state, monkeypatch):
    """RWKV6 (``o_t = r_t (S_{t-1} + diag(u) k_t^T v_t)``) through the key-channel-gated kernels with shifted queries,
    against the token-by-token fp32 recurrence: output, final state and every gradient incl. the bonus."""
    monkeypatch.setenv("LMOE_RWKV6_KERNEL", "1")                               # the kernels also under autograd
    torch.manual_seed(12)
    B, H = 2, 3
    r, k, v = [(0.5 * torch.randn(B, T, H, D, device=dev())).to(torch.bfloat16) for _ in range(3)]
    w = -torch.exp(torch.randn(B, T, H, D, device=dev()) - 1.0)                # RWKV6 log decays, some of them strong
    u = 0.5 * torch.randn(H, D, device=dev())
    S0 = 0.3 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    go = torch.randn(B, T, H, D, device=dev(), dtype=torch.bfloat16)
    gS = 0.1 * torch.randn(B, H, D, D, device=dev()) if with_state else None
    ins = [r, k, v, w, u] + ([S0] if with_state else [])
    K.reset_launch_count()
    f_k = lambda r, k, v, w, u, s=None: ops.lsm_vector(r, k, v, w, 1.0, s, u, 64)
    f_r = lambda r, k, v, w, u, s=None: RL.recurrent_rwkv6(r, k, v, w, u, scale=1.0, initial_state=s)
    (o, S), gk_ = grads(f_k, ins, (go, gS))
    assert K.reset_launch_count() >= 1, "the RWKV6 path did not reach the kernels"
    (o2, S2), gr = grads(f_r, [t.float() for t in ins], (go.float(), gS))
    rel_close(o, o2, 2e-2, "o")
    rel_close(S, S2, 2e-2, "final state")
    # the decay gradient is a reverse cumulative sum of q.dq - k.dk over bf16 dq / dk: a few per cent, the rest is bf16 rounding
    for name, a_, b_ in zip(["dr", "dk", "dv", "dw", "du", "dS0"], gk_, gr):
        rel_close(a_, b_, 8e-2 if name == "dw" else 1e-2, name)
    # forward-only calls take the kernels by default
    monkeypatch.delenv("LMOE_RWKV6_KERNEL")
    K.reset_launch_count()
    with torch.no_grad():
        o3, _ = ops.lsm_vector(r, k, v, w, 1.0, S0, u, 64)
    assert K.reset_launch_count() >= 1 and torch.equal(o3, o)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_vocab_parallel_ce_shard_kernels(dtype):
    """The per-shard pieces of the vocabulary-parallel cross entropy (softmax kernels on each shard, log-sum-exp and target
    logit combined across shards, gradient with the global log-sum-exp) on two emulated shards against
    ``F.cross_entropy`` on the whole vocabulary."""
    from linear_moe_b200.parallel.tensor_parallel import vocab_shard_stats
    torch.manual_seed(7)
    T, V, shards = 300, 4096, 2
    full = (2.0 * torch.randn(T, V, device=dev())).to(dtype)
    labels = torch.randint(0, V, (T,), device=dev())
    labels[::9] = -100
    gl = torch.rand(T, device=dev())
    w = V // shards
    stats = [vocab_shard_stats(full[:, s * w:(s + 1) * w].contiguous(), labels, s * w, -100) for s in range(shards)]
    lse = torch.logsumexp(torch.stack([st[0] for st in stats]), dim=0)
    tgt = torch.stack([st[1] for st in stats]).sum(0)
    loss = torch.where(labels != -100, lse - tgt, torch.zeros_like(lse))
    ref_in = full.float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, labels, ignore_index=-100, reduction="none")
    (ref * gl).sum().backward()
    assert torch.allclose(loss, ref.detach(), atol=2e-3 if dtype == torch.bfloat16 else 1e-4, rtol=1e-3)
    grad = torch.cat([K.softmax_ce_bwd(full[:, s * w:(s + 1) * w].contiguous(), stats[s][2], lse, gl, -100) for s in range(shards)], 1)
    rel_close(grad, ref_in.grad, 1e-2 if dtype == torch.bfloat16 else 1e-5, "dlogits")

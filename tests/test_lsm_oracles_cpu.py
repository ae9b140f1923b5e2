"""CPU oracle tests of the linear-sequence-model math: every chunked form against its token-by-token recurrence
(forward, final state, gradients, state chaining), and LASP-2 over 2 and 4 gloo ranks against one rank on the whole
sequence for the three state-combination kinds (scalar decay, vector decay, delta rule)."""
import pytest
import torch

from linear_moe_b200.ops import lsm_torch as L
from linear_moe_b200.ref import lsm as R

from dist_utils import run_distributed


def _inputs(B, T, H, dk, dv, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, dk, generator=g, dtype=dtype) * 0.5
    k = torch.randn(B, T, H, dk, generator=g, dtype=dtype) * 0.5
    v = torch.randn(B, T, H, dv, generator=g, dtype=dtype)
    return q, k, v, g


def _close(a, b, tol=2e-4):
    err = (a.double() - b.double()).abs().max().item()
    ref = b.double().abs().max().item()
    assert err <= tol * max(ref, 1.0), f"max abs err {err:.3e} (ref max {ref:.3e})"


@pytest.mark.parametrize("T", [64, 192, 1000])
@pytest.mark.parametrize("decay", ["none", "per_head", "per_token"])
def test_chunk_scalar_gated_matches_recurrence(T, decay):
    B, H, dk, dv = 2, 3, 16, 24
    q, k, v, gen = _inputs(B, T, H, dk, dv)
    if decay == "none":
        g_chunk, g_rec = None, None
    elif decay == "per_head":
        g_chunk = -torch.rand(H, generator=gen, dtype=torch.float64) * 0.2
        g_rec = g_chunk[None, None, :].expand(B, T, H)
    else:
        g_chunk = g_rec = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen, dtype=torch.float64)) / 4
    o, S = L.chunk_scalar_gated(q, k, v, g_chunk, chunk_size=64)
    o_ref, S_ref = R.recurrent_lsm(q, k, v, g=g_rec)
    _close(o, o_ref)
    _close(S, S_ref)


@pytest.mark.parametrize("T", [48, 200])
def test_chunk_vector_gated_matches_recurrence(T):
    B, H, dk, dv = 2, 2, 16, 16
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=1)
    gk = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk, generator=gen, dtype=torch.float64)) / 4
    o, S = L.chunk_vector_gated(q, k, v, gk, chunk_size=16)
    o_ref, S_ref = R.recurrent_lsm(q, k, v, gk=gk)
    _close(o, o_ref)
    _close(S, S_ref)


def test_rwkv6_bonus_form_matches_recurrence():
    B, T, H, dk, dv = 1, 80, 2, 16, 16
    r, k, v, gen = _inputs(B, T, H, dk, dv, seed=2)
    w = -torch.rand(B, T, H, dk, generator=gen, dtype=torch.float64) * 0.5
    u = torch.randn(H, dk, generator=gen, dtype=torch.float64) * 0.3
    o, S = L.chunk_vector_gated(r, k, v, w, scale=1.0, chunk_size=16, bonus=u)
    o_ref, S_ref = R.recurrent_rwkv6(r, k, v, w, u, scale=1.0)
    _close(o, o_ref)
    _close(S, S_ref)


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("parallel_scan", [False, True])
@pytest.mark.parametrize("T", [64, 150])
def test_chunk_delta_rule_matches_recurrence(gated, parallel_scan, T):
    B, H, dk, dv = 2, 2, 16, 24
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=3)
    k = torch.nn.functional.normalize(k, dim=-1)
    beta = torch.rand(B, T, H, generator=gen, dtype=torch.float64)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen, dtype=torch.float64)) / 4 if gated else None
    o, S = L.chunk_delta_rule(q, k, v, beta, g, chunk_size=32, parallel_scan=parallel_scan)
    o_ref, S_ref = R.recurrent_lsm(q, k, v, g=g, beta=beta)
    _close(o, o_ref, 5e-4)
    _close(S, S_ref, 5e-4)


def test_ssd_matches_recurrence():
    B, T, H, P, G, N = 2, 130, 4, 16, 2, 8
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(B, T, H, P, generator=gen, dtype=torch.float64)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen, dtype=torch.float64))
    A = -torch.rand(H, generator=gen, dtype=torch.float64)
    Bm = torch.randn(B, T, G, N, generator=gen, dtype=torch.float64) * 0.5
    Cm = torch.randn(B, T, G, N, generator=gen, dtype=torch.float64) * 0.5
    D = torch.randn(H, generator=gen, dtype=torch.float64)
    y, S = L.ssd_chunked(x, dt, A, Bm, Cm, D, chunk_size=32)
    y_ref, S_ref = R.recurrent_ssd(x, dt, A, Bm, Cm, D)
    _close(y, y_ref)
    _close(S, S_ref)


def test_value_gated_matches_recurrence():
    """State decays per value channel (first pass of gated slot attention): the transpose of the key-gated recurrence."""
    B, T, H, dk, dv = 1, 70, 2, 8, 12
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=5)
    gv = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dv, generator=gen, dtype=torch.float64)) / 4
    o, S = L.chunk_value_gated(q, k, v, gv, chunk_size=16)
    S_ref = torch.zeros(B, H, dk, dv, dtype=torch.float64)
    o_ref = torch.empty(B, T, H, dv, dtype=torch.float64)
    for t in range(T):
        S_ref = S_ref * gv[:, t].exp()[:, :, None, :] + k[:, t][..., None] * v[:, t][:, :, None, :]
        o_ref[:, t] = torch.einsum("bhk,bhkv->bhv", q[:, t] * dk ** -0.5, S_ref)
    _close(o, o_ref)
    _close(S, S_ref)


@pytest.mark.parametrize("kind", ["scalar", "vector", "delta"])
def test_state_chaining_equals_whole_sequence(kind):
    """Running two halves with the first half's final state as the second half's initial state equals one run: the
    property that decoding caches and LASP-2 rely on."""
    B, T, H, dk, dv = 1, 96, 2, 16, 16
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=6)
    h = T // 2
    if kind == "scalar":
        g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen, dtype=torch.float64)) / 4
        f = lambda sl, init: L.chunk_scalar_gated(q[:, sl], k[:, sl], v[:, sl], g[:, sl], initial_state=init, chunk_size=16)
    elif kind == "vector":
        gk = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk, generator=gen, dtype=torch.float64)) / 4
        f = lambda sl, init: L.chunk_vector_gated(q[:, sl], k[:, sl], v[:, sl], gk[:, sl], initial_state=init, chunk_size=16)
    else:
        kn = torch.nn.functional.normalize(k, dim=-1)
        beta = torch.rand(B, T, H, generator=gen, dtype=torch.float64)
        f = lambda sl, init: L.chunk_delta_rule(q[:, sl], kn[:, sl], v[:, sl], beta[:, sl], None, initial_state=init, chunk_size=16)
    o_all, S_all = f(slice(0, T), None)
    o1, S1 = f(slice(0, h), None)
    o2, S2 = f(slice(h, T), S1)
    _close(torch.cat([o1, o2], 1), o_all)
    _close(S2, S_all)


@pytest.mark.parametrize("kind", ["scalar", "vector", "delta"])
def test_chunked_gradients_match_recurrence(kind):
    B, T, H, dk, dv = 1, 40, 2, 8, 8
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=7)
    if kind == "delta":
        k = torch.nn.functional.normalize(k, dim=-1)
    extra = {"scalar": torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen, dtype=torch.float64)) / 4,
             "vector": torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk, generator=gen, dtype=torch.float64)) / 4,
             "delta": torch.rand(B, T, H, generator=gen, dtype=torch.float64)}[kind]
    w = torch.randn(B, T, H, dv, generator=gen, dtype=torch.float64)

    def grads(fn):
        xs = [t.clone().requires_grad_(True) for t in (q, k, v, extra)]
        o, S = fn(*xs)
        ((o * w).sum() + S.sum()).backward()
        return [x.grad for x in xs]

    if kind == "scalar":
        a = grads(lambda q, k, v, g: L.chunk_scalar_gated(q, k, v, g, chunk_size=16))
        b = grads(lambda q, k, v, g: R.recurrent_lsm(q, k, v, g=g))
    elif kind == "vector":
        a = grads(lambda q, k, v, gk: L.chunk_vector_gated(q, k, v, gk, chunk_size=8))
        b = grads(lambda q, k, v, gk: R.recurrent_lsm(q, k, v, gk=gk))
    else:
        a = grads(lambda q, k, v, beta: L.chunk_delta_rule(q, k, v, beta, None, chunk_size=16))
        b = grads(lambda q, k, v, beta: R.recurrent_lsm(q, k, v, beta=beta))
    for x, y in zip(a, b):
        _close(x, y, 5e-4)


# ---------------------------------------------------------------------------------------------------------------------
def _lasp_worker(rank, world, kind):
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.parallel.lasp2 import lasp2
    mesh = Mesh(ParallelConfig(context_parallel_size=world))
    B, T, H, dk, dv = 1, 64 * world, 2, 16, 16
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=11, dtype=torch.float32)
    kw = {}
    if kind == "scalar":
        kw["g"] = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen)) / 4
    elif kind == "vector":
        kw["gk"] = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk, generator=gen)) / 4
    else:
        k = torch.nn.functional.normalize(k, dim=-1)
        kw["beta"] = torch.rand(B, T, H, generator=gen)
        kw["g"] = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen)) / 4
    sl = slice(rank * (T // world), (rank + 1) * (T // world))
    loc = [t[:, sl].clone().requires_grad_(True) for t in (q, k, v)]
    kw_loc = {n: t[:, sl] for n, t in kw.items()}
    o, S = lasp2(kind, *loc, group=mesh["cp"], chunk_size=16, **kw_loc)
    w = torch.randn(B, T, H, dv, generator=gen)
    (o * w[:, sl]).sum().backward()
    return o.detach(), S.detach(), [t.grad for t in loc]


@pytest.mark.parametrize("kind", ["scalar", "vector", "delta"])
@pytest.mark.parametrize("world", [2, 4])
def test_lasp2_matches_one_rank(kind, world):
    outs = run_distributed(_lasp_worker, world, kind=kind)
    B, T, H, dk, dv = 1, 64 * world, 2, 16, 16
    q, k, v, gen = _inputs(B, T, H, dk, dv, seed=11, dtype=torch.float32)
    kw = {}
    if kind == "scalar":
        kw["g"] = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen)) / 4
    elif kind == "vector":
        kw["gk"] = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk, generator=gen)) / 4
    else:
        k = torch.nn.functional.normalize(k, dim=-1)
        kw["beta"] = torch.rand(B, T, H, generator=gen)
        kw["g"] = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen)) / 4
    xs = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o_ref, S_ref = R.recurrent_lsm(*xs, **kw)
    w = torch.randn(B, T, H, dv, generator=gen)
    (o_ref * w).sum().backward()
    _close(torch.cat([o[0] for o in outs], 1), o_ref, 1e-3)
    _close(outs[-1][1], S_ref, 1e-3)
    for i, x in enumerate(xs):
        _close(torch.cat([o[2][i] for o in outs], 1), x.grad, 2e-3)


def _dplr_inputs(B, T, H, dk, dv):
    gen = torch.Generator().manual_seed(5)
    rn = lambda *s: torch.randn(*s, generator=gen)
    r, k, v = rn(B, T, H, dk), rn(B, T, H, dk) * 0.5, rn(B, T, H, dv)
    w = -0.6 * torch.sigmoid(rn(B, T, H, dk))                                   # RWKV7's bounded log decay
    kk = torch.nn.functional.normalize(rn(B, T, H, dk), dim=-1)
    a = torch.sigmoid(rn(B, T, H, dk))
    return r, w, k, v, -kk, kk * a, rn(B, T, H, dv)


def _dplr_worker(rank, world):
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.parallel.lasp2 import lasp2
    mesh = Mesh(ParallelConfig(context_parallel_size=world))
    B, T, H, dk, dv = 1, 24 * world, 2, 8, 12
    r, w, k, v, a, b, go = _dplr_inputs(B, T, H, dk, dv)
    sl = slice(rank * (T // world), (rank + 1) * (T // world))
    loc = [t[:, sl].clone().requires_grad_(True) for t in (r, w, k, v, a, b)]
    o, S = lasp2("dplr", loc[0], loc[2], loc[3], group=mesh["cp"], gk=loc[1], scale=1.0, dplr=(loc[4], loc[5]))
    (o * go[:, sl]).sum().backward()
    return o.detach(), S.detach(), [t.grad for t in loc]


@pytest.mark.parametrize("world", [2, 3])
def test_lasp2_dplr_matches_one_rank(world):
    """RWKV7's diagonal-plus-low-rank recurrence with the sequence split over ranks: outputs, final state and every input
    gradient equal the unsplit recurrence."""
    outs = run_distributed(_dplr_worker, world)
    B, T, H, dk, dv = 1, 24 * world, 2, 8, 12
    *xs, go = _dplr_inputs(B, T, H, dk, dv)
    xs = [t.clone().requires_grad_(True) for t in xs]
    o_ref, S_ref = L.recurrent_dplr(*xs, 1.0, None)
    (o_ref * go).sum().backward()
    _close(torch.cat([o[0] for o in outs], 1), o_ref, 1e-4)
    _close(outs[-1][1], S_ref, 1e-4)
    for i, x in enumerate(xs):
        _close(torch.cat([o[2][i] for o in outs], 1), x.grad, 5e-4)


@pytest.mark.parametrize("la", ["retention", "gla", "deltanet", "rwkv6", "hgrn2"])
def test_la_mode_selects_equivalent_forms(la):
    """``--la-mode``: chunk / fused_chunk (chunked form), fused_recurrent (token recurrence) and, for the scalar-decay
    family, parallel (quadratic form) compute the same layer output."""
    from linear_moe_b200.config.model_config import ModelConfig
    from linear_moe_b200.models.transformer import CausalLM
    torch.manual_seed(0)
    ids = torch.randint(0, 512, (2, 96))
    outs = {}
    modes = ["chunk", "fused_chunk", "fused_recurrent"] + (["parallel"] if la == "retention" else [])
    for mode in modes:
        cfg = ModelConfig(num_layers=2, hidden_size=64, num_attention_heads=2, ffn_hidden_size=128, vocab_size=512,
                          use_la_module=True, la_module=la, layer_type_list="LL", la_mode=mode)
        outs[mode] = CausalLM(cfg)(ids)
    for mode in modes[1:]:
        assert torch.allclose(outs[mode], outs["chunk"], atol=2e-4, rtol=1e-3), (la, mode, (outs[mode] - outs["chunk"]).abs().max())
    if la != "retention":
        with pytest.raises(ValueError):
            cfg = ModelConfig(num_layers=1, hidden_size=64, num_attention_heads=2, ffn_hidden_size=128, vocab_size=512,
                              use_la_module=True, la_module=la, layer_type_list="L", la_mode="parallel")
            CausalLM(cfg)(ids)


@pytest.mark.parametrize("T,with_state", [(50, True), (37, False), (1, True)])
def test_rwkv6_shifted_query_identity(T, with_state, monkeypatch):
    """RWKV6 through the gated-scan operator with queries shifted one position to the left (what the CUDA path does around
    its kernels): output, final state and all gradients equal the token-by-token recurrence.  The kernels are stood in
    for by the chunked torch form of the same operator."""
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.ops import lsm_torch as LT
    from linear_moe_b200.ref import lsm as RL

    def inner(q, k, v, gk, scale, init, bonus, chunk):
        assert bonus is None
        return LT.chunk_vector_gated(q, k, v, gk, scale, init, 16, None)
    monkeypatch.setattr(K, "lsm_vector", inner)
    monkeypatch.setattr(K, "_note_strong_decay", lambda gk: None)
    torch.manual_seed(12)
    B, H, D = 2, 3, 16
    f64 = torch.float64
    r, k, v = [0.5 * torch.randn(B, T, H, D, dtype=f64) for _ in range(3)]
    w = -torch.exp(torch.randn(B, T, H, D, dtype=f64) - 1.0)
    u = 0.5 * torch.randn(H, D, dtype=f64)
    S0 = 0.3 * torch.randn(B, H, D, D, dtype=f64) if with_state else None
    ins = [t.clone().requires_grad_(True) for t in ([r, k, v, w, u] + ([S0] if with_state else []))]
    o, S = K._lsm_vector_bonus(ins[0], ins[1], ins[2], ins[3], 1.0, ins[5] if with_state else None, ins[4], 64)
    go, gS = torch.randn_like(o), 0.1 * torch.randn_like(S)
    ((o * go).sum() + (S * gS).sum()).backward()
    ref_in = [t.detach().clone().float().requires_grad_(True) for t in ins]
    o2, S2 = RL.recurrent_rwkv6(ref_in[0], ref_in[1], ref_in[2], ref_in[3], ref_in[4], scale=1.0,
                                initial_state=ref_in[5] if with_state else None)
    ((o2 * go.float()).sum() + (S2 * gS.float()).sum()).backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()
    assert rel(o, o2) < 1e-5 and rel(S, S2) < 1e-5
    for a, b in zip(ins, ref_in):
        assert rel(a.grad, b.grad) < 1e-4

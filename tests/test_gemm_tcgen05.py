"""tcgen05 GEMM against torch.matmul in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 768, 520), (4096, 2048, 2048), (300, 264, 72)])
def test_gemm_nt(M, N, K):
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    c = gemm.gemm_nt(a, b)
    torch.cuda.synchronize()
    gemm.check_error()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


def test_gemm_nt_swiglu():
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    M, f, K = 520, 512, 256
    a = (0.5 * torch.randn(M, K, device=dev)).to(torch.bfloat16)
    w = (0.1 * torch.randn(2 * f, K, device=dev)).to(torch.bfloat16)
    y = gemm.gemm_nt(a, gemm.tile_swiglu_weight(w), swiglu=True)
    torch.cuda.synchronize()
    gemm.check_error()
    z = a.float() @ w.float().t()
    ref = torch.nn.functional.silu(z[:, :f]) * z[:, f:]
    err = (y.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (384, 320, 200)])
def test_gemm_layouts(a_mn, b_mn, M, N, K, pairs):
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    c = gemm.gemm_general(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn, b_mn, pairs=pairs)
    torch.cuda.synchronize()
    gemm.check_error()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


@pytest.mark.parametrize("pairs", [False, True])
def test_grouped_mlp_matches_loop(pairs, monkeypatch):
    from linear_moe_b200.ops import gemm
    from linear_moe_b200.ref import ops as R
    monkeypatch.setattr(gemm, "PAIRS", pairs)                # single-CTA kernels (128-row tiles) or CTA pairs (256)
    monkeypatch.setattr(gemm, "ROW_ALIGN", 256 if pairs else 128)
    dev = torch.device("cuda", 0)
    torch.manual_seed(2)
    E, h, f = 6, 256, 192
    counts = torch.tensor([300, 0, 17, 128, 511, 64], device=dev)
    T = int(counts.sum())
    x = (0.5 * torch.randn(T, h, device=dev)).to(torch.bfloat16).requires_grad_(True)
    w1 = (0.05 * torch.randn(E, h, 2 * f, device=dev)).to(torch.bfloat16).requires_grad_(True)
    w2 = (0.05 * torch.randn(E, f, h, device=dev)).to(torch.bfloat16).requires_grad_(True)
    gy = torch.randn(T, h, device=dev).to(torch.bfloat16)
    y = gemm.grouped_mlp(x, counts, w1, w2)
    y.backward(gy)
    torch.cuda.synchronize()
    gemm.check_error()
    xr, w1r, w2r = (t.detach().float().requires_grad_(True) for t in (x, w1, w2))
    yr = R.grouped_mlp(xr, counts, w1r, w2r)
    yr.backward(gy.float())
    for name, a, b in (("y", y, yr), ("dx", x.grad, xr.grad), ("dw1", w1.grad, w1r.grad), ("dw2", w2.grad, w2r.grad)):
        err = (a.float() - b).abs().max().item()
        assert err <= 3e-2 * b.abs().max().item() + 1e-3, (name, err, b.abs().max().item())
    assert w1.grad[1].abs().max().item() == 0.0          # expert without tokens: exact zero gradient


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (1000 // 16 * 16, 328 // 8 * 8, 272), (128, 256, 128)])
def test_fp8_gemm_and_quantisation(M, N, K):
    """e4m3 tcgen05 GEMM with per-row scales against the fp32 product of the de-quantised operands (exact up to
    accumulation order and the bf16 output), and the quantisers against torch's float8 cast."""
    from linear_moe_b200.ops import fp8, gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    a = (torch.randn(M, K, device=dev) * torch.rand(M, 1, device=dev) * 3).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    aq, sa = fp8.quant_rows(a)
    bq, sb = fp8.quant_rows(b)
    # quantiser: scale = amax / 448 and round-to-nearest e4m3
    assert torch.allclose(sa, a.float().abs().amax(1) / 448.0, rtol=1e-6)
    want = (a.float() / sa[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    assert (aq != want).float().mean().item() < 1e-3          # ties may round differently
    ref = fp8.dequant_rows(aq, sa) @ fp8.dequant_rows(bq, sb).t()
    for pairs in (False, True):                              # single-CTA and CTA-pair kernels
        c = fp8.gemm_nt(aq, sa, bq, sb, pairs=pairs)
        gemm.check_error()
        err = (c.float() - ref).abs().max().item()
        assert err <= 1e-2 * ref.abs().max().item(), (pairs, err, ref.abs().max().item())
    # transposed column-wise quantisation = row-wise quantisation of the transpose
    tq, ts = fp8.quant_cols_t(a)
    tq2, ts2 = fp8.quant_rows(a.t().contiguous())
    assert torch.allclose(ts, ts2, rtol=1e-6) and (tq != tq2).float().mean().item() < 1e-3


def test_fp8_linear_close_to_bf16():
    from linear_moe_b200.ops import fp8
    dev = torch.device("cuda", 0)
    torch.manual_seed(2)
    x = torch.randn(4, 256, 512, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (0.05 * torch.randn(768, 512, device=dev)).to(torch.bfloat16).requires_grad_(True)
    go = torch.randn(4, 256, 768, device=dev).to(torch.bfloat16)
    y = fp8.Fp8Linear.apply(x, w)
    y.backward(go)
    g1 = (x.grad.clone(), w.grad.clone())
    x.grad = w.grad = None
    y2 = torch.nn.functional.linear(x, w)
    y2.backward(go)
    for name, p, q in (("y", y, y2), ("dx", g1[0], x.grad), ("dw", g1[1], w.grad)):
        rel = (p.float() - q.float()).norm() / q.float().norm()
        assert rel < 6e-2, (name, rel.item())           # e4m3 has 3 mantissa bits: ~4 % relative error per GEMM


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 512), (1000, 328, 200), (4096, 2048, 1024), (128, 256, 2048)])
def test_gemm_2cta_pairs(M, N, K):
    """tcgen05.mma.cta_group::2 GEMM (256 x 256 tile per CTA pair) against the fp32 product."""
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    for _ in range(2):
        c = gemm.gemm_nt_2cta(a, b)
    torch.cuda.synchronize()
    gemm.check_error()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, (err, ref.abs().max().item())


def test_grouped_wgrad_into_fp32_accumulator():
    """The grouped weight-gradient GEMM writes (first call) and then accumulates (second call) into ``main_grad``."""
    from linear_moe_b200.ops import gemm
    if not gemm.PAIRS:
        pytest.skip("needs the CTA-pair grouped kernels")
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    E, h, f = 4, 256, 320
    counts = torch.tensor([256, 0, 512, 256], device=dev)
    offs = gemm.padded_offsets(counts)
    rows = int(offs[-1])
    x = (0.5 * torch.randn(rows, h, device=dev)).to(torch.bfloat16).requires_grad_(True)
    w = (0.05 * torch.randn(E, h, f, device=dev)).to(torch.bfloat16).requires_grad_(True)
    gy = torch.randn(rows, f, device=dev).to(torch.bfloat16)
    ref = torch.autograd.grad(gemm.GroupedLinear.apply(x, w, offs), w, gy)[0].float()
    w.main_grad = torch.full((E, h, f), 7.0, dtype=torch.float32, device=dev)     # stale content: the first write overwrites
    w._main_grad_fresh = True
    for n in (1, 2):
        gemm.GroupedLinear.apply(x, w, offs).backward(gy)
        torch.cuda.synchronize()
        gemm.check_error()
        assert w.grad is None
        err = (w.main_grad - n * ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() * n + 1e-3, (n, err)


def _dense_case(M, N, K, a_mn, b_mn, seed=0):
    dev = torch.device("cuda", 0)
    torch.manual_seed(seed)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    return a, b, (a.t().contiguous() if a_mn else a), (b.t().contiguous() if b_mn else b), a.float() @ b.float().t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (1000, 520, 200), (72, 40, 8), (2304, 1280, 1032)])
def test_gemm_dense_layouts(a_mn, b_mn, M, N, K):
    """Dense CTA-pair kernel, bf16 output through TMA stores, against the fp32 product (ragged M, N and K included)."""
    from linear_moe_b200.ops import gemm
    a, b, aa, bb, ref = _dense_case(M, N, K, a_mn, b_mn)
    for band in (1, 3, 8):
        c = gemm.dense(aa, bb, a_mn, b_mn, band=band)
        torch.cuda.synchronize()
        gemm.check_error()
        err = (c.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-3, (band, err)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(512, 768, 320), (1000, 264, 4104)])
def test_gemm_dense_fp32_out_and_accumulate(a_mn, b_mn, M, N, K):
    """fp32 output (TMA store) and fp32 accumulation (TMA reduce-add) of the dense kernel; relative Frobenius error."""
    from linear_moe_b200.ops import gemm
    a, b, aa, bb, ref = _dense_case(M, N, K, a_mn, b_mn, seed=3)
    c = torch.full((M, N), 7.0, device=a.device)
    gemm.dense(aa, bb, a_mn, b_mn, out=c)
    torch.cuda.synchronize()
    assert ((c - ref).norm() / ref.norm()).item() < 1e-5
    gemm.dense(aa, bb, a_mn, b_mn, out=c, accumulate=True)
    gemm.dense(aa, bb, a_mn, b_mn, out=c, accumulate=True)
    torch.cuda.synchronize()
    gemm.check_error()
    assert ((c - 3 * ref).norm() / (3 * ref).norm()).item() < 1e-5
    # a strided fp32 destination (a slice of a flat gradient buffer)
    big = torch.zeros(M, N + 12, device=a.device)
    gemm.dense(aa, bb, a_mn, b_mn, out=big[:, 4:4 + N], accumulate=True)
    torch.cuda.synchronize()
    assert ((big[:, 4:4 + N] - ref).norm() / ref.norm()).item() < 1e-5
    assert big[:, :4].abs().max().item() == 0 and big[:, 4 + N:].abs().max().item() == 0


@pytest.mark.parametrize("M,F,K,want_pre", [(520, 512, 256, True), (300, 136, 72, True), (1024, 384, 128, False)])
def test_gemm_dense_swiglu(M, F, K, want_pre):
    """fc1 + SwiGLU epilogue on the ordinary [gate; up] weight layout; also returns the pre-activations."""
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = (0.5 * torch.randn(M, K, device=dev)).to(torch.bfloat16)
    w = (0.1 * torch.randn(2 * F, K, device=dev)).to(torch.bfloat16)
    act, pre = gemm.dense_swiglu(x, w, want_pre=want_pre)
    torch.cuda.synchronize()
    gemm.check_error()
    z = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(z[:, :F]) * z[:, F:]
    assert (act.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
    if want_pre:
        assert (pre.float() - z).abs().max().item() <= 2e-2 * z.abs().max().item() + 1e-3
    else:
        assert pre is None


@pytest.mark.parametrize("main_grad", [False, True])
def test_linear_autograd_on_dense_kernel(main_grad):
    """ops.linear on bf16 CUDA tensors: y, dx, dW against fp32 autograd; with main_grad two backward passes accumulate."""
    from linear_moe_b200 import ops
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    x = torch.randn(3, 100, 264, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (0.1 * torch.randn(520, 264, device=dev)).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(520, device=dev).to(torch.bfloat16)
    gy = torch.randn(3, 100, 520, device=dev).to(torch.bfloat16)
    if main_grad:
        w.main_grad = torch.empty(520, 264, device=dev)
        w._main_grad_fresh = True
    reps = 2 if main_grad else 1
    for _ in range(reps):
        y = ops.linear(x, w, bias)
        y.backward(gy)
    torch.cuda.synchronize()
    gemm.check_error()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr, bias.float())
    yr.backward(gy.float())
    assert (y.float() - yr).abs().max().item() <= 2e-2 * yr.abs().max().item()
    assert ((x.grad.float() - reps * xr.grad).norm() / (reps * xr.grad).norm()).item() < 1e-2
    dw = w.main_grad if main_grad else w.grad.float()
    assert ((dw - reps * wr.grad).norm() / (reps * wr.grad).norm()).item() < (1e-5 if main_grad else 1e-2)


@pytest.mark.parametrize("M,F,H", [(520, 512, 256), (300, 192, 136), (2048, 1024, 512)])
def test_gemm_dense_dswiglu(M, F, H):
    """fc2 data-gradient GEMM with the SwiGLU backward in its epilogue against fp32 autograd of swiglu(pre) @ W2^T."""
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    dy = (0.5 * torch.randn(M, H, device=dev)).to(torch.bfloat16)
    w2 = (0.1 * torch.randn(H, F, device=dev)).to(torch.bfloat16)
    pre = torch.randn(M, 2 * F, device=dev).to(torch.bfloat16)
    dpre = gemm.dense_dswiglu(dy, w2, pre)
    torch.cuda.synchronize()
    gemm.check_error()
    p = pre.float().requires_grad_(True)
    act = torch.nn.functional.silu(p[:, :F]) * p[:, F:]
    (act @ w2.float().t()).backward(dy.float())
    rel = ((dpre.float() - p.grad).norm() / p.grad.norm()).item()
    assert rel < 1e-2, rel


def test_mlp_swiglu_autograd():
    """The fused SwiGLU MLP node (fc1 + SwiGLU epilogue, fc2, dSwiGLU epilogue) against fp32 autograd: y, dx, dW1, dW2."""
    from linear_moe_b200 import ops
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    h, f = 256, 384
    x = torch.randn(2, 150, h, device=dev).to(torch.bfloat16).requires_grad_(True)
    w1 = (0.08 * torch.randn(2 * f, h, device=dev)).to(torch.bfloat16).requires_grad_(True)
    w2 = (0.08 * torch.randn(h, f, device=dev)).to(torch.bfloat16).requires_grad_(True)
    gy = torch.randn(2, 150, h, device=dev).to(torch.bfloat16)
    y = ops.mlp_swiglu(x, w1, w2)
    y.backward(gy)
    torch.cuda.synchronize()
    gemm.check_error()
    xr, w1r, w2r = (t.detach().float().requires_grad_(True) for t in (x, w1, w2))
    z = xr @ w1r.t()
    yr = (torch.nn.functional.silu(z[..., :f]) * z[..., f:]) @ w2r.t()
    yr.backward(gy.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(y, yr) < 1e-2 and rel(x.grad, xr.grad) < 2e-2 and rel(w1.grad, w1r.grad) < 2e-2 and rel(w2.grad, w2r.grad) < 2e-2


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (8, 6144, 2048), (5, 2056, 8192), (16, 128256, 2048), (11, 40, 64)])
def test_skinny_gemm_for_decode_rows(M, N, K):
    """The weight-streaming GEMM of one-token decode steps (up to 16 rows) against fp32 matmul; also through
    ``ops.linear`` without autograd, which must route to it."""
    from linear_moe_b200 import ops
    from linear_moe_b200.ops import cuda as K_
    torch.manual_seed(M + N)
    dev = torch.device("cuda", 0)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    y = K_.linear_skinny(x, w)
    torch.cuda.synchronize()
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 5e-3, rel
    K_.reset_launch_count()
    with torch.no_grad():
        y2 = ops.linear(x.view(1, M, K), w)
    assert K_.reset_launch_count() == 1 and y2.shape == (1, M, N)
    assert torch.equal(y2.view(M, N), y)                       # deterministic: no atomics
    # with autograd on a parameter the regular (differentiable) path runs instead
    wp = w.clone().requires_grad_(True)
    assert not K_._skinny_ok(x, wp)


def test_linear_with_bias_in_the_gemm_epilogue():
    """``ops.linear`` with a bf16 bias: the bias is added in the GEMM epilogue (one launch forward); output and all three
    gradients against fp32 PyTorch."""
    from linear_moe_b200 import ops
    from linear_moe_b200.ops import cuda as K_
    torch.manual_seed(5)
    dev = torch.device("cuda", 0)
    x = torch.randn(3, 700, 512, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(1032, 512, device=dev) / 512 ** 0.5).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(1032, device=dev).to(torch.bfloat16).requires_grad_(True)
    gy = torch.randn(3, 700, 1032, device=dev).to(torch.bfloat16)
    K_.reset_launch_count()
    y = ops.linear(x, w, b)
    assert K_.reset_launch_count() == 1, "the bias add is a separate launch"
    y.backward(gy)
    xf, wf, bf = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    yr = torch.nn.functional.linear(xf, wf, bf)
    yr.backward(gy.float())
    rel = lambda a, r: ((a.float() - r).norm() / r.norm()).item()
    assert rel(y, yr) < 5e-3, rel(y, yr)
    assert rel(x.grad, xf.grad) < 5e-3 and rel(w.grad, wf.grad) < 5e-3 and rel(b.grad, bf.grad) < 5e-3

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


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (384, 320, 200)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    from linear_moe_b200.ops import gemm
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    c = gemm.gemm_general(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn, b_mn)
    torch.cuda.synchronize()
    gemm.check_error()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


def test_grouped_mlp_matches_loop():
    from linear_moe_b200.ops import gemm
    from linear_moe_b200.ref import ops as R
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

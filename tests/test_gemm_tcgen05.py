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

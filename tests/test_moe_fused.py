"""The peer-memory MoE exchange kernels on one GPU (a one-rank workspace) against the permute / grouped-MLP / un-permute
definition in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from linear_moe_b200.ref import ops as R


@pytest.mark.parametrize("T,k,E,hid,f,drop", [(1000, 2, 4, 256, 128, False), (333, 8, 16, 512, 64, True), (64, 1, 2, 128, 256, False)])
def test_fused_moe_one_rank(T, k, E, hid, f, drop):
    from linear_moe_b200.models.moe import permute, unpermute
    from linear_moe_b200.ops import gemm
    from linear_moe_b200.ops.moe_fused import fused_moe
    from linear_moe_b200.parallel import fused_comm
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    ws = fused_comm.MoeWorkspace(None, E, hid, T * k + 256 * E, dev)
    h = torch.randn(T, hid, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev)
    probs, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    if drop:
        dropped = torch.rand(T, k, device=dev) < 0.2
        idx = torch.where(dropped, torch.full_like(idx, -1), idx)
        probs = probs * (~dropped)
    w1 = (0.05 * torch.randn(E, hid, 2 * f, device=dev)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(E, f, hid, device=dev)).to(torch.bfloat16)
    go = torch.randn(T, hid, device=dev).to(torch.bfloat16)

    def run(fused):
        hh, pp = h.clone().requires_grad_(True), probs.clone().requires_grad_(True)
        a, b = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        if fused:
            out = fused_moe(hh, pp, idx, a, b, ws)
            out.backward(go)
        else:
            hf, af, bf = hh.float(), a.float(), b.float()
            permuted, order, counts = permute(hf, idx, E)
            y = R.grouped_mlp(permuted, counts, af, bf)
            out = unpermute(y, order, pp, T, k)
            out.backward(go.float())
        return out, hh.grad, pp.grad, a.grad, b.grad

    for rep in range(2):                                    # twice: epochs and buffer reuse
        got = run(True)
        torch.cuda.synchronize()
        fused_comm.check_status("moe test")
        gemm.check_error()
    ref = run(False)
    for name, x, y in zip(["out", "dh", "dprobs", "dw1", "dw2"], got, ref):
        x, y = x.float(), y.float()
        err, scale = (x - y).abs().max().item(), y.abs().max().item()
        assert err <= 3e-2 * scale + 1e-3, f"{name}: err {err:.3e} scale {scale:.3e}"

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


def test_bounded_wait_expiry_and_overflow_are_reported():
    """Failure reporting of the exchange kernels without faulting anything: (a) a pull that waits for an epoch nobody
    signals gives up after its spin limit, sets the status word and returns; (b) routing more rows to a rank than its
    receive buffer holds sets the status word and sends nothing.  The context stays usable afterwards."""
    import ctypes
    from linear_moe_b200.ops import cuda as K
    from linear_moe_b200.parallel import fused_comm
    from linear_moe_b200.train.watchdog import CommTimeout
    dev = torch.device("cuda", 0)
    E, hid, T, k = 4, 128, 64, 2
    ws = fused_comm.MoeWorkspace(None, E, hid, T * k + 256 * E, dev, spin_limit=2000)
    idx = torch.randint(0, E, (T, k), device=dev)
    route = ws.route(idx)
    torch.cuda.synchronize()
    fused_comm.check_status("clean")                                   # nothing wrong so far
    # (a) wait for an epoch that is never signalled: ~2000 polls of 64 ns, then status + return
    a = ws._args()
    a.epoch = ws.ep_pull + 5
    out = torch.empty(T, hid, dtype=torch.bfloat16, device=dev)
    w = torch.ones(T, k, dtype=torch.float32, device=dev)
    a.w, a.out, a.rows = w.data_ptr(), out.data_ptr(), 0
    a.dest_rank, a.dest_row = route.dest_rank.data_ptr(), route.dest_row.data_ptr()
    a.n_assign, a.k = T * k, k
    ws._run(5, a, "moe_pull")
    torch.cuda.synchronize()
    with pytest.raises(CommTimeout):
        fused_comm.check_status("expired wait")
    fused_comm.check_status("cleared")                                 # the status word was reset
    # (b) receive buffer too small for the routed rows
    small = fused_comm.MoeWorkspace(None, E, hid, 256, dev)
    r2 = small.route(torch.zeros(1024, k, dtype=torch.int64, device=dev))      # 2048 rows to expert 0, capacity 256
    torch.cuda.synchronize()
    assert int((r2.dest_rank >= 0).sum()) == 0                         # nothing is sent
    with pytest.raises(CommTimeout):
        fused_comm.check_status("overflow")
    # the context is intact: a normal exchange still works
    x = torch.randn(T, hid, device=dev).to(torch.bfloat16)
    recv = ws.push(x, route, None)
    torch.cuda.synchronize()
    fused_comm.check_status("after")
    assert torch.isfinite(recv[: int(route.offs[-1])].float()).all()

"""Per-kernel timing and roofline harness.

  python -m linear_moe_b200.bench.kernels [--kernel all|gemm|gemm_dense|lsm|flash|families|moe|decode|norm|headnorm|swiglu|ce|adam|conv] [--size small|full]

Each kernel is timed with CUDA events on the launching stream after warm-up, with an L2 flush (a 256 MiB write)
between iterations; the median is reported together with the algorithmic bytes / FLOPs and the fraction of the
measured peaks (``MEASURED_PEAKS.json`` at the repository root: STREAM-style copy bandwidth and cuBLAS bf16
throughput; fallback 6650 GB/s and 1590 TFLOPS when the file is absent).  ``--size small`` keeps the working set
at a few hundred MB (larger than L2), which is the case to run under ``ncu``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters=10, warmup=3):
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def report(name, ms, bytes_=None, flops=None):
    bw, tf, kind = peaks()
    line = f"{name:38s} {ms * 1e3:9.1f} us"
    if bytes_ is not None:
        g = bytes_ / ms / 1e6
        line += f" | {g:7.0f} GB/s = {g / bw:5.2f} of {kind} copy bw"
    if flops is not None:
        t = flops / ms / 1e9
        line += f" | {t:7.0f} TFLOPS = {t / tf:5.2f} of {kind} cuBLAS bf16"
    print(line, flush=True)


def bench_gemm(size):
    from ..ops import gemm
    dev = torch.device("cuda", 0)
    shapes = [(4096, 4096, 2048)] if size == "small" else [(16384, 8192, 2048), (16384, 16384, 2048), (16384, 2048, 8192)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        report(f"gemm tcgen05 {M}x{N}x{K}", timeit(lambda: gemm.gemm_nt(a, b, out=c)), flops=2.0 * M * N * K)
        report(f"gemm tcgen05 2-CTA {M}x{N}x{K}", timeit(lambda: gemm.gemm_nt_2cta(a, b, out=c)), flops=2.0 * M * N * K)
        report(f"gemm cuBLAS  {M}x{N}x{K}", timeit(lambda: torch.mm(a, b.t(), out=c)), flops=2.0 * M * N * K)
    from ..ops import fp8
    for M, N, K in shapes:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        aq, sa = fp8.quant_rows(a)
        bq, sb = fp8.quant_rows(b)
        report(f"gemm fp8 tcgen05 {M}x{N}x{K}", timeit(lambda: fp8.gemm_nt(aq, sa, bq, sb, pairs=False)), flops=2.0 * M * N * K)
        report(f"gemm fp8 tcgen05 2-CTA {M}x{N}x{K}", timeit(lambda: fp8.gemm_nt(aq, sa, bq, sb, pairs=True)), flops=2.0 * M * N * K)
        report(f"fp8 quant rows {M}x{K}", timeit(lambda: fp8.quant_rows(a)), bytes_=3.0 * M * K)
        report(f"fp8 quant cols^T {M}x{K}", timeit(lambda: fp8.quant_cols_t(a)), bytes_=5.0 * M * K)
    gemm.check_error()


def bench_gemm_dense(size):
    """The dense CTA-pair kernel under every plain linear (``csrc/gemm_dense.cu``) in its three operand layouts, next to
    the library GEMM on the same operands.  ``small``: one 4096 x 4096 x 2048 problem per layout (what ``ncu`` captures)."""
    from ..ops import gemm
    dev = torch.device("cuda", 0)
    if size == "small":
        shapes = [("fwd  x W^T", 4096, 4096, 2048, 0, 0, 0), ("dgrad dy W", 4096, 2048, 4096, 0, 1, 0),
                  ("wgrad dy^T x (fp32)", 4096, 2048, 4096, 1, 1, 1)]
    else:
        shapes = [("fc1 fwd", 16384, 16384, 2048, 0, 0, 0), ("fc2 fwd", 16384, 2048, 8192, 0, 0, 0),
                  ("qkv fwd", 16384, 6144, 2048, 0, 0, 0), ("fc1 dgrad", 16384, 2048, 16384, 0, 1, 0),
                  ("fc2 dgrad", 16384, 8192, 2048, 0, 1, 0), ("fc1 wgrad (fp32)", 16384, 2048, 16384, 1, 1, 1),
                  ("fc2 wgrad (fp32)", 2048, 8192, 16384, 1, 1, 1), ("LM head fwd", 16384, 128256, 2048, 0, 0, 0)]
    for name, M, N, K, amn, bmn, f32 in shapes:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        aa, bb = (a.t().contiguous() if amn else a), (b.t().contiguous() if bmn else b)
        del a, b
        c = torch.empty(M, N, device=dev, dtype=torch.float32 if f32 else torch.bfloat16)
        at, bt = (aa.t() if amn else aa), (bb if bmn else bb.t())
        fl = 2.0 * M * N * K
        report(f"gemm_dense {name} {M}x{N}x{K}", timeit(lambda: gemm.dense(aa, bb, bool(amn), bool(bmn), out=c)), flops=fl)
        lib = (lambda: torch.mm(at, bt, out_dtype=torch.float32, out=c)) if f32 else (lambda: torch.mm(at, bt, out=c))
        report(f"cuBLAS     {name} {M}x{N}x{K}", timeit(lib), flops=fl)
        del aa, bb, c, at, bt
    if size != "small":
        M, F_, K = 16384, 8192, 2048
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (0.1 * torch.randn(2 * F_, K, device=dev)).bfloat16()
        from .. import ops
        report("fc1 + SwiGLU, fused epilogue (writes act + pre)", timeit(lambda: gemm.dense_swiglu(x, w, want_pre=True)),
               flops=2.0 * M * 2 * F_ * K)
        report("fc1 cuBLAS + SwiGLU kernel", timeit(lambda: ops.swiglu(torch.mm(x, w.t()))), flops=2.0 * M * 2 * F_ * K)
    gemm.check_error()


def bench_skinny(size):
    """Linears of a one-token decode step (batch 8): the weight-streaming kernel against the library call.  Each
    measurement loops once over enough copies of the weight (>= 512 MB) that no call finds its weight in L2, inside one
    pair of events, so launch gaps of a few microseconds do not dominate kernels of a few microseconds."""
    from ..ops import cuda as K
    dev = torch.device("cuda", 0)
    M = 8
    shapes = [("qkv", 6144, 2048), ("gate / out proj", 2048, 2048), ("fc1", 16384, 2048), ("fc2", 2048, 8192),
              ("LM head", 128256, 2048)]
    for name, N, Kd in shapes:
        x = torch.randn(M, Kd, device=dev).bfloat16()
        n = max(2, (512 << 20) // (N * Kd * 2) + 1)
        ws = [(torch.randn(N, Kd, device=dev) / Kd ** 0.5).bfloat16() for _ in range(n)]

        def loop(fn):
            def run():
                for w_ in ws:
                    fn(x, w_)
            return run
        with torch.no_grad():
            for label, fn in (("gemm_skinny", K.linear_skinny), ("cuBLAS     ", torch.nn.functional.linear)):
                ms = timeit(loop(fn), iters=5) / n
                report(f"{label} {name} {M}x{N}x{Kd}", ms, bytes_=N * Kd * 2)
        del ws


def bench_lsm(size):
    from .. import ops
    dev = torch.device("cuda", 0)
    B, H, D = 1, 16, 128
    T = 4096 if size == "small" else 16384
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev)).bfloat16().requires_grad_(True)
    g = -torch.linspace(0.01, 0.3, H, device=dev)
    go = torch.randn(B, T, H, D, device=dev).bfloat16()
    elt = B * T * H * D * 2

    def fwd():
        q, k, v = qkv.split(D, dim=-1)
        return ops.lsm_scalar(q, k, v, g, 1.0, None, 64)[0]
    intra = 2.0 * B * H * T * (2 * 64 * D + 2 * D * D)          # per token: QK^T, PV (64-wide) + QS, K^T V
    with torch.no_grad():
        report(f"lsm_scalar fwd T={T} H={H} D={D}", timeit(fwd), bytes_=6 * elt, flops=1.5 * intra)
    o = fwd()

    def bwd():
        qkv.grad = None
        o.backward(go, retain_graph=True)
    report(f"lsm_scalar bwd T={T} H={H} D={D}", timeit(bwd), bytes_=15 * elt, flops=3.5 * intra)


def bench_elementwise(which, size):
    from .. import ops
    from ..ops import cuda as K
    dev = torch.device("cuda", 0)
    T = 8192 if size == "small" else 16384
    h, f, H, D = 2048, 8192, 16, 128
    if which in ("norm", "all"):
        x = torch.randn(T, h, device=dev).bfloat16().requires_grad_(True)
        r = torch.randn(T, h, device=dev).bfloat16().requires_grad_(True)
        w = torch.ones(h, device=dev).bfloat16().requires_grad_(True)
        with torch.no_grad():
            report("add_rms_norm fwd", timeit(lambda: ops.add_rms_norm(x, r, w, 1e-6)), bytes_=4 * T * h * 2)
        y, ro = ops.add_rms_norm(x, r, w, 1e-6)
        gy = torch.randn_like(y)
        report("add_rms_norm bwd", timeit(lambda: torch.autograd.grad([y, ro], [x, w], [gy, gy], retain_graph=True)),
               bytes_=4 * T * h * 2)
    if which in ("headnorm", "all"):
        o = torch.randn(1, T, H, D, device=dev).bfloat16().requires_grad_(True)
        gt = torch.randn(1, T, H * D, device=dev).bfloat16().requires_grad_(True)
        w = torch.ones(D, device=dev).bfloat16().requires_grad_(True)
        with torch.no_grad():
            report("head_norm_gate fwd", timeit(lambda: ops.head_norm_gate(o, w, gt, 1e-5)), bytes_=3 * T * h * 2)
        y = ops.head_norm_gate(o, w, gt, 1e-5)
        gy = torch.randn_like(y)
        report("head_norm_gate bwd", timeit(lambda: torch.autograd.grad(y, [o, gt, w], gy, retain_graph=True)),
               bytes_=5 * T * h * 2)
    if which in ("swiglu", "all"):
        x = torch.randn(T, 2 * f, device=dev).bfloat16().requires_grad_(True)
        with torch.no_grad():
            report("swiglu fwd", timeit(lambda: ops.swiglu(x)), bytes_=3 * T * f * 2)
        y = ops.swiglu(x)
        gy = torch.randn_like(y)
        report("swiglu bwd", timeit(lambda: torch.autograd.grad(y, x, gy, retain_graph=True)), bytes_=5 * T * f * 2)
    if which in ("ce", "all"):
        V, Tc = 128256, 2048 if size == "small" else 4096
        logits = torch.randn(Tc, V, device=dev).bfloat16()
        lab = torch.randint(0, V, (Tc,), device=dev)
        loss, lse = torch.empty(Tc, device=dev), torch.empty(Tc, device=dev)
        report("softmax_ce fwd", timeit(lambda: K.softmax_ce_fwd(logits, lab, loss, lse, -100)), bytes_=Tc * V * 2)
        gl = torch.ones(Tc, device=dev)
        report("softmax_ce bwd (in place)", timeit(lambda: K.softmax_ce_bwd(logits, lab, lse, gl, -100)), bytes_=2 * Tc * V * 2)
    if which in ("adam", "all"):
        n = (64 << 20) if size == "small" else (512 << 20)
        p = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        m32, g, m, v = (torch.zeros(n, device=dev) for _ in range(4))
        report(f"fused_adam n={n >> 20}Mi", timeit(lambda: K.fused_adam(p, m32, g, m, v, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0)),
               bytes_=n * 30)
    if which in ("conv", "all"):
        Dc = 6144
        x = torch.randn(1, T, Dc, device=dev).bfloat16().requires_grad_(True)
        w = torch.randn(Dc, 4, device=dev).bfloat16().requires_grad_(True)
        with torch.no_grad():
            report("causal_conv1d fwd", timeit(lambda: ops.causal_conv1d(x, w)), bytes_=2 * T * Dc * 2)
        y = ops.causal_conv1d(x, w)[0]
        gy = torch.randn_like(y)
        report("causal_conv1d bwd", timeit(lambda: torch.autograd.grad(y, [x, w], gy, retain_graph=True)), bytes_=3 * T * Dc * 2)


def bench_flash(size):
    from ..ops import flash, attention
    dev = torch.device("cuda", 0)
    B, Hq, Hkv, D = 1, 16, 4, 128
    T = 4096 if size == "small" else 16384
    q = torch.randn(B, T, Hq, D, device=dev).bfloat16().requires_grad_(True)
    kv = torch.randn(B, T, Hkv, 2 * D, device=dev).bfloat16().requires_grad_(True)
    go = torch.randn(B, T, Hq, D, device=dev).bfloat16()
    fl = 4.0 * B * Hq * T * T * D / 2                      # causal: half of QK^T + PV

    def fwd(fn):
        k, v = kv.split(D, dim=-1)
        return fn(q, k, v)
    mine = lambda q, k, v: flash.FlashAttention.apply(q, k, v, D ** -0.5, 0, None)
    lib = lambda q, k, v: attention.sdpa_reference(q, k, v, D ** -0.5, True, 0, None)
    for name, fn in (("flash_attn (own)", mine), ("sdpa (library)", lib)):
        with torch.no_grad():
            report(f"{name} fwd T={T} {Hq}q/{Hkv}kv D={D}", timeit(lambda: fwd(fn)), flops=fl)
        o = fwd(fn)

        def bwd():
            q.grad = kv.grad = None
            o.backward(go, retain_graph=True)
        report(f"{name} bwd T={T} {Hq}q/{Hkv}kv D={D}", timeit(bwd), flops=2.5 * fl)


def bench_lsm_families(size):
    """GLA and the gated delta rule, forward and backward.  ``--size small`` runs every operator once (one forward, one
    backward, 4 x 4096 tokens so that the inputs exceed L2) and is the case to put under a profiler; ``full`` times them."""
    from .. import ops
    dev = torch.device("cuda", 0)
    B, H, D = 4, 8, 128
    T = 4096
    q, k, v = [(0.5 * torch.randn(B, T, H, D, device=dev)).bfloat16().requires_grad_(True) for _ in range(3)]
    gk = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, D, device=dev)) / 16).requires_grad_(True)
    g = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev)) / 16).requires_grad_(True)
    beta = torch.rand(B, T, H, device=dev).requires_grad_(True)
    go = torch.randn(B, T, H, D, device=dev).bfloat16()
    kn = torch.nn.functional.normalize(k.detach().float(), dim=-1).bfloat16().requires_grad_(True)
    cases = {
        "gla (lsm_vector.cu)": lambda: ops.lsm_vector(q, k, v, gk, None, None, None, 64)[0],
        "gated delta rule (lsm_delta.cu)": lambda: ops.lsm_delta(q, kn, v, beta, g, None, None, 64)[0],
    }
    for name, fn in cases.items():
        if size == "small":
            fn().backward(go)
            torch.cuda.synchronize()
            print(f"{name}: one forward + backward, B={B} T={T} H={H} D={D}")
            continue
        with torch.no_grad():
            report(f"{name} fwd B={B} T={T} H={H} D={D}", timeit(fn, iters=5))
        o = fn()

        def bwd():
            for t in (q, k, v, gk, g, beta, kn):
                t.grad = None
            o.backward(go, retain_graph=True)
        report(f"{name} bwd B={B} T={T} H={H} D={D}", timeit(bwd, iters=5))


def bench_moe(size):
    """Expert MLPs of the A0.3B-2B GLA preset on one rank: 8 local experts, hidden 1024, ffn 896, top-8."""
    from ..ops import gemm
    from ..ops.moe_fused import fused_moe
    from ..parallel import fused_comm
    dev = torch.device("cuda", 0)
    T, k, E, hid, f = (2048, 8, 8, 1024, 896) if size == "small" else (8192, 8, 8, 1024, 896)
    ws = fused_comm.MoeWorkspace(None, E, hid, T * k + 256 * E, dev)
    h = torch.randn(T, hid, device=dev).bfloat16().requires_grad_(True)
    probs, idx = torch.topk(torch.softmax(torch.randn(T, E, device=dev), -1), k, dim=-1)
    probs = probs.requires_grad_(True)
    w1 = (0.05 * torch.randn(E, hid, 2 * f, device=dev)).bfloat16().requires_grad_(True)
    w2 = (0.05 * torch.randn(E, f, hid, device=dev)).bfloat16().requires_grad_(True)
    go = torch.randn(T, hid, device=dev).bfloat16()
    fl = 2.0 * T * k * hid * 3 * f
    fn = lambda: fused_moe(h, probs, idx, w1, w2, ws)
    with torch.no_grad():
        report(f"fused moe fwd T={T} k={k} E={E} h={hid} f={f}", timeit(fn), flops=fl)
    o = fn()

    def bwd():
        h.grad = probs.grad = w1.grad = w2.grad = None
        o.backward(go, retain_graph=True)
    report(f"fused moe bwd T={T} k={k} E={E} h={hid} f={f}", timeit(bwd), flops=2 * fl)
    # the grouped GEMM alone (fc1 of all experts)
    x = torch.randn(T * k, hid, device=dev).bfloat16()
    offs = torch.arange(0, E + 1, device=dev, dtype=torch.int32) * (T * k // E)
    with torch.no_grad():
        report(f"grouped gemm fc1 rows={T * k} E={E}", timeit(lambda: gemm.GroupedLinear.apply(x, w1, offs)), flops=2.0 * T * k * hid * 2 * f)
    gemm.check_error()
    fused_comm.check_status("bench")


def bench_decode(size):
    """One-token decode steps of the LASP-2 Linear-Llama3-1B preset (all layers lightning attention, O(1) state):
    eager launches against replay of the captured CUDA graph.  The floor is reading the bf16 weights once per token."""
    from ..config.presets import get_preset
    from ..infer.generation import GraphedDecodeStep
    from ..models.transformer import CausalLM
    dev = torch.device("cuda", 0)
    cfg = get_preset("bench-lasp2-llama3-1b")
    if size == "small":
        cfg.num_layers = 4
        cfg.layer_type_list = "LLLL"
    model = CausalLM(cfg, device=dev).to(dev).eval()
    weight_bytes = sum(p.numel() * p.element_size() for n, p in model.named_parameters() if "word_embeddings" not in n)
    B = 8
    with torch.no_grad():
        caches = model.new_cache()
        model(torch.randint(0, cfg.vocab_size, (B, 64), device=dev), caches=caches)
        tok = torch.randint(0, cfg.vocab_size, (B, 1), device=dev)
        for _ in range(3):
            model(tok, caches=caches, position_offset=0)
        t_eager = timeit(lambda: model(tok, caches=caches, position_offset=0))
        step = GraphedDecodeStep(model, caches, B, dev)
        step(tok)
        t_graph = timeit(lambda: step(tok))
    for name, t in (("eager", t_eager), ("CUDA graph", t_graph)):
        report(f"decode step, batch {B}, {cfg.num_layers} layers, {name}", t, bytes_=weight_bytes)
    print(f"  tokens/s: eager {B / t_eager * 1e3:.0f}, graph {B / t_graph * 1e3:.0f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--size", default="full", choices=["small", "full"])
    a = ap.parse_args()
    torch.cuda.set_device(0)
    print(f"peaks: {peaks()}")
    if a.kernel in ("gemm", "all"):
        bench_gemm(a.size)
    if a.kernel in ("gemm_dense", "all"):
        bench_gemm_dense(a.size)
    if a.kernel in ("skinny", "all"):
        bench_skinny(a.size)
    if a.kernel in ("lsm", "all"):
        bench_lsm(a.size)
    if a.kernel in ("flash", "all"):
        bench_flash(a.size)
    if a.kernel in ("families", "all"):
        bench_lsm_families(a.size)
    if a.kernel in ("moe", "all"):
        bench_moe(a.size)
    if a.kernel in ("decode", "all"):
        bench_decode(a.size)
    if a.kernel in ("norm", "headnorm", "swiglu", "ce", "adam", "conv", "all"):
        bench_elementwise(a.kernel, a.size)


if __name__ == "__main__":
    main()

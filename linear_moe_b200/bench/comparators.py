"""Per-kernel yardsticks: this repository's kernels next to the engines the reference calls for the same operator.

  python -m linear_moe_b200.bench.comparators [--only lightning,gla,gdn,delta,flash,gemm] [--iters 10]

The reference reaches its sequence-mixing kernels through ``flash-linear-attention`` (``fla.ops.simple_gla`` for
lightning attention / retention, ``fla.ops.gla``, ``fla.ops.gated_delta_rule``, ``fla.ops.delta_rule``;
gla/gla.py:94, gated_deltanet.py:112, retention.py:91) and softmax attention through ``flash_attn`` / TransformerEngine.
Both packages are Triton / CUDA libraries; they are imported here only as comparators and never by the framework.
Shapes are the per-GPU shapes of the benchmark configurations.  Every row is timed the same way: CUDA events on the
launching stream, 3 warm-up calls, an L2 flush (256 MiB write) before every timed call, median of ``--iters``.
Forward and forward+backward are reported; a comparator that is missing or fails prints the reason in its cell.
"""
from __future__ import annotations

import argparse
import statistics

import torch


def _time(fn, iters):
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
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
    return statistics.median(ts) * 1e3          # microseconds


def _fwd_bwd(op, inputs, iters):
    """(forward us, forward+backward us) of ``op(*inputs)`` whose first result is differentiated."""
    leaves = [t.detach().clone().requires_grad_(t.is_floating_point()) for t in inputs]

    def fwd():
        with torch.no_grad():
            op(*leaves)
    out = op(*leaves)
    out = out[0] if isinstance(out, (tuple, list)) else out
    go = torch.randn_like(out)

    def both():
        o = op(*leaves)
        o = o[0] if isinstance(o, (tuple, list)) else o
        o.backward(go)
        for t in leaves:
            t.grad = None
    return _time(fwd, iters), _time(both, iters)


def _cell(fn):
    try:
        f, fb = fn()
        return f"{f:8.0f} / {fb:8.0f}"
    except Exception as e:                                   # noqa: BLE001 - a comparator may be absent or refuse a shape
        return f"n/a ({type(e).__name__}: {str(e)[:60]})"


def bench_lightning(iters):
    """Config LASP-2 Linear-Llama3-1B: lightning attention, T=16384, 16 heads x 128, constant decay per head."""
    from .. import ops
    from ..ref import lsm as RL
    B, T, H, D = 1, 16384, 16, 128
    dev = torch.device("cuda", 0)
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev)).bfloat16()
    q, k, v = (t.contiguous() for t in qkv.split(D, dim=-1))
    g = -RL.lightning_slopes(H).to(dev)
    ours = lambda q, k, v: ops.lsm_scalar(q, k, v, g, 1.0, None, 64)

    def fla_op(q, k, v):
        from fla.ops.simple_gla import chunk_simple_gla
        return chunk_simple_gla(q, k, v, g_gamma=g, scale=1.0)
    return [("lightning attention T=16384 H=16 D=128", _cell(lambda: _fwd_bwd(ours, [q, k, v], iters)),
             "fla chunk_simple_gla", _cell(lambda: _fwd_bwd(fla_op, [q, k, v], iters)))]


def bench_gla(iters):
    """Config A0.3B-2B: GLA, 8 sequences of 2048, 8 heads x 128."""
    from .. import ops
    B, T, H, D = 8, 2048, 8, 128
    dev = torch.device("cuda", 0)
    q, k, v = [(0.5 * torch.randn(B, T, H, D, device=dev)).bfloat16() for _ in range(3)]
    gk = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, D, device=dev)) / 16).bfloat16()
    ours = lambda q, k, v, gk: ops.lsm_vector(q, k, v, gk.float(), None, None, None, 64)

    def fla_op(q, k, v, gk):
        from fla.ops.gla import chunk_gla
        return chunk_gla(q, k, v, gk)
    return [("GLA B=8 T=2048 H=8 D=128", _cell(lambda: _fwd_bwd(ours, [q, k, v, gk], iters)),
             "fla chunk_gla", _cell(lambda: _fwd_bwd(fla_op, [q, k, v, gk], iters)))]


def bench_gdn(iters, gated=True):
    """Config A1B-7B hybrid: (gated) delta rule, 2 sequences of 4096, 8 heads x 128 (16 heads under TP2)."""
    from .. import ops
    B, T, H, D = 2, 4096, 8, 128
    dev = torch.device("cuda", 0)
    q, v = [(0.5 * torch.randn(B, T, H, D, device=dev)).bfloat16() for _ in range(2)]
    k = torch.nn.functional.normalize(torch.randn(B, T, H, D, device=dev), dim=-1).bfloat16()
    beta = torch.rand(B, T, H, device=dev).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev) + 2.0)
    if gated:
        ours = lambda q, k, v, beta, g: ops.lsm_delta(q, k, v, beta.float(), g, None, None, 64)

        def fla_op(q, k, v, beta, g):
            from fla.ops.gated_delta_rule import chunk_gated_delta_rule
            return chunk_gated_delta_rule(q, k, v, g, beta)
        ins, name, fname = [q, k, v, beta, g], "gated delta rule", "fla chunk_gated_delta_rule"
    else:
        ours = lambda q, k, v, beta: ops.lsm_delta(q, k, v, beta.float(), None, None, None, 64)

        def fla_op(q, k, v, beta):
            from fla.ops.delta_rule import chunk_delta_rule
            return chunk_delta_rule(q, k, v, beta)
        ins, name, fname = [q, k, v, beta], "delta rule", "fla chunk_delta_rule"
    return [(f"{name} B=2 T=4096 H=8 D=128", _cell(lambda: _fwd_bwd(ours, ins, iters)), fname,
             _cell(lambda: _fwd_bwd(fla_op, ins, iters)))]


def bench_flash(iters):
    """Softmax attention layers of the hybrid configs: causal GQA, head dim 128."""
    from ..ops import attention
    rows = []
    for B, T, Hq, Hkv in ((2, 4096, 8, 2), (1, 16384, 16, 4)):
        dev = torch.device("cuda", 0)
        q = (0.5 * torch.randn(B, T, Hq, 128, device=dev)).bfloat16()
        k = (0.5 * torch.randn(B, T, Hkv, 128, device=dev)).bfloat16()
        v = (0.5 * torch.randn(B, T, Hkv, 128, device=dev)).bfloat16()
        ours = lambda q, k, v: attention.flash_attention(q, k, v, 128 ** -0.5, True, 0, None)

        def fa(q, k, v):
            from flash_attn import flash_attn_func
            return flash_attn_func(q, k, v, causal=True)

        def sdpa(q, k, v):
            o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                 is_causal=True, enable_gqa=True)
            return o.transpose(1, 2)
        rows.append((f"flash attention B={B} T={T} {Hq}q/{Hkv}kv D=128", _cell(lambda: _fwd_bwd(ours, [q, k, v], iters)),
                     "flash_attn 2.8 | torch SDPA",
                     _cell(lambda: _fwd_bwd(fa, [q, k, v], iters)) + " | " + _cell(lambda: _fwd_bwd(sdpa, [q, k, v], iters))))
    return rows


def bench_gemm(iters):
    """The three GEMMs of one fc1 / fc2 linear of the headline model (16384 tokens, 2048 <-> 8192/16384)."""
    from ..ops import gemm
    dev = torch.device("cuda", 0)
    rows = []
    for name, M, N, K, amn, bmn, f32 in (("fc1 forward", 16384, 16384, 2048, 0, 0, 0), ("fc2 forward", 16384, 2048, 8192, 0, 0, 0),
                                         ("fc1 dgrad", 16384, 2048, 16384, 0, 1, 0), ("fc1 wgrad (fp32 out)", 16384, 2048, 16384, 1, 1, 1)):
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        aa, bb = (a.t().contiguous() if amn else a), (b.t().contiguous() if bmn else b)
        c = torch.empty(M, N, device=dev, dtype=torch.float32 if f32 else torch.bfloat16)
        at, bt = (aa.t() if amn else aa), (bb if bmn else bb.t())
        t_o = _time(lambda: gemm.dense(aa, bb, bool(amn), bool(bmn), out=c), iters)
        t_c = _time((lambda: torch.mm(at, bt, out_dtype=torch.float32, out=c)) if f32 else (lambda: torch.mm(at, bt, out=c)), iters)
        fl = 2.0 * M * N * K
        rows.append((f"GEMM {name} {M}x{N}x{K}", f"{t_o:8.0f} us = {fl / t_o / 1e6:5.0f} TFLOP/s", "cuBLAS (torch.mm)",
                     f"{t_c:8.0f} us = {fl / t_c / 1e6:5.0f} TFLOP/s"))
        del a, b, aa, bb, c
    gemm.check_error()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", type=str, default="lightning,gla,gdn,delta,flash,gemm")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    only = set(args.only.split(","))
    rows = []
    if "lightning" in only:
        rows += bench_lightning(args.iters)
    if "gla" in only:
        rows += bench_gla(args.iters)
    if "gdn" in only:
        rows += bench_gdn(args.iters, True)
    if "delta" in only:
        rows += bench_gdn(args.iters, False)
    if "flash" in only:
        rows += bench_flash(args.iters)
    if "gemm" in only:
        rows += bench_gemm(args.iters)
    print("| operator (per-GPU shape) | this repository: fwd / fwd+bwd (us) | comparator | comparator: fwd / fwd+bwd (us) |")
    print("|---|---|---|---|")
    for r in rows:
        print("| " + " | ".join(r) + " |", flush=True)


if __name__ == "__main__":
    main()

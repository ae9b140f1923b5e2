"""Per-kernel yardsticks: this repository's kernels next to the engines the reference calls for the same operator.

  python -m linear_moe_b200.bench.comparators [--only lightning,gla,gdn,delta,flash4k,flash16k,gemm] [--iters 10]

The reference reaches its sequence-mixing kernels through ``flash-linear-attention`` (``fla.ops.simple_gla`` for
lightning attention / retention, ``fla.ops.gla``, ``fla.ops.gated_delta_rule``, ``fla.ops.delta_rule``;
gla/gla.py:94, gated_deltanet.py:112, retention.py:91) and softmax attention through ``flash_attn`` / TransformerEngine.
Both packages are Triton / CUDA libraries; they are imported here only as comparators and never by the framework.
Shapes are the per-GPU shapes of the benchmark configurations.  Every row is timed the same way: CUDA events on the
launching stream, 3 warm-up calls, an L2 flush (256 MiB write) before every timed call, median of ``--iters``.
Forward and forward+backward are reported.  Every measurement runs in a process of its own, so a comparator that is
missing or fails prints the reason in its cell and the table goes on.
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


def _inputs_lightning():
    from ..ref import lsm as RL
    B, T, H, D = 1, 16384, 16, 128
    dev = torch.device("cuda", 0)
    qkv = (0.5 * torch.randn(B, T, H, 3 * D, device=dev)).bfloat16()
    q, k, v = (t.contiguous() for t in qkv.split(D, dim=-1))
    return [q, k, v], -RL.lightning_slopes(H).to(dev)


def cell_lightning(impl, iters):
    """Config LASP-2 Linear-Llama3-1B: lightning attention, T=16384, 16 heads x 128, constant decay per head."""
    from .. import ops
    ins, g = _inputs_lightning()
    if impl == "ours":
        return _fwd_bwd(lambda q, k, v: ops.lsm_scalar(q, k, v, g, 1.0, None, 64), ins, iters)
    from fla.ops.simple_gla import chunk_simple_gla
    return _fwd_bwd(lambda q, k, v: chunk_simple_gla(q, k, v, g_gamma=g, scale=1.0), ins, iters)


def cell_gla(impl, iters):
    """Config A0.3B-2B: GLA, 8 sequences of 2048, 8 heads x 128."""
    from .. import ops
    B, T, H, D = 8, 2048, 8, 128
    dev = torch.device("cuda", 0)
    q, k, v = [(0.5 * torch.randn(B, T, H, D, device=dev)).bfloat16() for _ in range(3)]
    gk = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, D, device=dev)) / 16).bfloat16()
    if impl == "ours":
        return _fwd_bwd(lambda q, k, v, gk: ops.lsm_vector(q, k, v, gk.float(), None, None, None, 64), [q, k, v, gk], iters)
    from fla.ops.gla import chunk_gla
    return _fwd_bwd(lambda q, k, v, gk: chunk_gla(q, k, v, gk), [q, k, v, gk], iters)


def _cell_delta(impl, iters, gated):
    """Config A1B-7B hybrid: (gated) delta rule, 2 sequences of 4096, 8 heads x 128 (16 heads under TP2)."""
    from .. import ops
    B, T, H, D = 2, 4096, 8, 128
    dev = torch.device("cuda", 0)
    q, v = [(0.5 * torch.randn(B, T, H, D, device=dev)).bfloat16() for _ in range(2)]
    k = torch.nn.functional.normalize(torch.randn(B, T, H, D, device=dev), dim=-1).bfloat16()
    beta = torch.rand(B, T, H, device=dev).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev) + 2.0)
    if impl == "ours":
        if gated:
            return _fwd_bwd(lambda q, k, v, beta, g: ops.lsm_delta(q, k, v, beta.float(), g, None, None, 64), [q, k, v, beta, g], iters)
        return _fwd_bwd(lambda q, k, v, beta: ops.lsm_delta(q, k, v, beta.float(), None, None, None, 64), [q, k, v, beta], iters)
    if impl == "eager":                                          # the batched-matmul + parallel-scan form this kernel replaced
        import os
        os.environ["LMOE_DELTA_KERNEL"] = "0"
        if gated:
            return _fwd_bwd(lambda q, k, v, beta, g: ops.lsm_delta(q, k, v, beta.float(), g, None, None, 64), [q, k, v, beta, g], iters)
        return _fwd_bwd(lambda q, k, v, beta: ops.lsm_delta(q, k, v, beta.float(), None, None, None, 64), [q, k, v, beta], iters)
    if gated:
        from fla.ops.gated_delta_rule import chunk_gated_delta_rule
        return _fwd_bwd(lambda q, k, v, beta, g: chunk_gated_delta_rule(q, k, v, g, beta), [q, k, v, beta, g], iters)
    from fla.ops.delta_rule import chunk_delta_rule
    return _fwd_bwd(lambda q, k, v, beta: chunk_delta_rule(q, k, v, beta), [q, k, v, beta], iters)


def cell_gdn(impl, iters):
    return _cell_delta(impl, iters, True)


def cell_delta(impl, iters):
    return _cell_delta(impl, iters, False)


def _cell_flash(impl, iters, shape):
    from ..ops import attention
    B, T, Hq, Hkv = shape
    dev = torch.device("cuda", 0)
    q = (0.5 * torch.randn(B, T, Hq, 128, device=dev)).bfloat16()
    k = (0.5 * torch.randn(B, T, Hkv, 128, device=dev)).bfloat16()
    v = (0.5 * torch.randn(B, T, Hkv, 128, device=dev)).bfloat16()
    if impl == "ours":
        return _fwd_bwd(lambda q, k, v: attention.flash_attention(q, k, v, 128 ** -0.5, True, 0, None), [q, k, v], iters)
    if impl == "flash_attn":
        from flash_attn import flash_attn_func
        return _fwd_bwd(lambda q, k, v: flash_attn_func(q, k, v, causal=True), [q, k, v], iters)

    def sdpa(q, k, v):
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                             is_causal=True, enable_gqa=True)
        return o.transpose(1, 2)
    return _fwd_bwd(sdpa, [q, k, v], iters)


def cell_flash4k(impl, iters):
    return _cell_flash(impl, iters, (2, 4096, 8, 2))


def cell_flash16k(impl, iters):
    return _cell_flash(impl, iters, (1, 16384, 16, 4))


# operator -> (row title, cell function, implementations; "ours" first).  A comparator that faulted the GPU in an
# earlier run is listed in SKIP with the record of that run and is not started again.
TABLE = {
    "lightning": ("lightning attention T=16384 H=16 D=128", cell_lightning, ["ours", "fla"]),
    "gla": ("GLA B=8 T=2048 H=8 D=128", cell_gla, ["ours", "fla"]),
    "gdn": ("gated delta rule B=2 T=4096 H=8 D=128", cell_gdn, ["ours", "eager", "fla"]),
    "delta": ("delta rule B=2 T=4096 H=8 D=128", cell_delta, ["ours", "eager", "fla"]),
    "flash4k": ("flash attention B=2 T=4096 8q/2kv D=128", cell_flash4k, ["ours", "flash_attn", "sdpa"]),
    "flash16k": ("flash attention B=1 T=16384 16q/4kv D=128", cell_flash16k, ["ours", "flash_attn", "sdpa"]),
}
SKIP = {
    ("gdn", "fla"): "not run: a run that included fla.ops.gated_delta_rule.chunk_gated_delta_rule at this shape ended in "
                    "'CUDA error: misaligned address' (Triton 3.6 on sm_100a); it is not started again",
}


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
    import subprocess
    import sys
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", type=str, default="lightning,gla,gdn,delta,flash4k,flash16k,gemm")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--cell", type=str, default=None, help="internal: run one <operator>:<implementation> measurement")
    args = ap.parse_args()
    if args.cell:
        op, impl = args.cell.split(":")
        f, fb = TABLE[op][1](impl, args.iters)
        print(f"RESULT {f:.1f} {fb:.1f}", flush=True)
        return
    print("| operator (per-GPU shape) | implementation | forward (us) | forward + backward (us) |")
    print("|---|---|---|---|")
    for op in args.only.split(","):
        if op == "gemm":
            for r in bench_gemm(args.iters):
                print(f"| {r[0]} | this repository | {r[1]} | |")
                print(f"| {r[0]} | {r[2]} | {r[3]} | |", flush=True)
            continue
        title, _, impls = TABLE[op]
        for impl in impls:
            name = "this repository" if impl == "ours" else impl
            if (op, impl) in SKIP:
                print(f"| {title} | {name} | {SKIP[(op, impl)]} | |", flush=True)
                continue
            # one process per measurement: a comparator that fails cannot take the rest of the table with it
            r = subprocess.run([sys.executable, "-m", "linear_moe_b200.bench.comparators", "--cell", f"{op}:{impl}",
                                "--iters", str(args.iters)], capture_output=True, text=True)
            line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")]
            if r.returncode == 0 and line:
                _, f, fb = line[-1].split()
                print(f"| {title} | {name} | {float(f):.0f} | {float(fb):.0f} |", flush=True)
            else:
                err = (r.stderr.strip().splitlines() or ["failed"])[-1][:120]
                print(f"| {title} | {name} | n/a ({err}) | |", flush=True)


if __name__ == "__main__":
    main()

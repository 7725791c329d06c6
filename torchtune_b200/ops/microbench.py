"""Single-op micro-benchmarks for the sm_100a kernels, timed with CUDA events.

    python -m torchtune_b200.ops.microbench gemm --m 8192 --n 4096 --k 4096 --layout nt
    python -m torchtune_b200.ops.microbench attention --batch 4 --seq 2048 --doc 512
    python -m torchtune_b200.ops.microbench rmsnorm --rows 8192 --dim 4096
    python -m torchtune_b200.ops.microbench adamw --numel 268435456

Each command prints one JSON line: median milliseconds over ``--iters`` launches (an L2 flush
of 256 MiB between launches), the algorithmic FLOP/s or bytes/s, and the same figure for the
PyTorch library op on identical inputs.  ``--iters`` and ``--warmup`` are small by default so
the same command line can be placed under a profiler.
"""
from __future__ import annotations

import argparse
import json

import torch


def _time(fn, iters: int, warmup: int, flush: torch.Tensor) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(args, flush):
    from ._cuda import gemm

    m, n, k = args.m, args.n, args.k
    bf = dict(device="cuda", dtype=torch.bfloat16)
    if args.layout == "nt":  # forward: Y[m,n] = X[m,k] · W[n,k]ᵀ
        a, b = torch.randn(m, k, **bf), torch.randn(n, k, **bf)
        ours = lambda: gemm(a, b, out=out)
        lib = lambda: torch.matmul(a, b.t(), out=out)
    elif args.layout == "nn":  # dgrad: dX[m,n] = dY[m,k] · W[k,n]
        a, b = torch.randn(m, k, **bf), torch.randn(k, n, **bf)
        ours = lambda: gemm(a, b, b_mn=True, out=out)
        lib = lambda: torch.matmul(a, b, out=out)
    else:  # tn, wgrad: dW[m,n] = dY[k,m]ᵀ · X[k,n]
        a, b = torch.randn(k, m, **bf), torch.randn(k, n, **bf)
        ours = lambda: gemm(a, b, a_mn=True, b_mn=True, out=out)
        lib = lambda: torch.matmul(a.t(), b, out=out)
    out = torch.empty(m, n, **bf)
    flops = 2.0 * m * n * k
    t = _time(ours, args.iters, args.warmup, flush)
    res = {"op": f"gemm_{args.layout}", "m": m, "n": n, "k": k, "ms": t, "tflops": flops / t / 1e9}
    if not args.no_lib:
        t_lib = _time(lib, args.iters, args.warmup, flush)
        res.update(lib_ms=t_lib, lib_tflops=flops / t_lib / 1e9)
    return res


def bench_gemm_fp8(args, flush):
    """fp8 (e4m3 × e4m3, tensorwise scales) GEMM alone, and the whole fp8 linear forward (amax + cast + GEMM) against the bf16 GEMM."""
    from ._cuda import fp8_cast, fp8_linear, fp8_scales, gemm, gemm_fp8

    m, n, k = args.m, args.n, args.k
    bf = dict(device="cuda", dtype=torch.bfloat16)
    a, b = torch.randn(m, k, **bf), torch.randn(n, k, **bf) * 0.05
    sa, _ = fp8_scales(a, False, False)
    sb, _ = fp8_scales(b, False, False)
    aq, _ = fp8_cast(a, sa, sa, want_t=False)
    bq, _ = fp8_cast(b, sb, sb, want_t=False)
    ia, ib = 1.0 / sa, 1.0 / sb
    out = torch.empty(m, n, **bf)
    flops = 2.0 * m * n * k
    t = _time(lambda: gemm_fp8(aq, bq, ia, ib, out=out), args.iters, args.warmup, flush)
    t_cast = _time(lambda: fp8_cast(a, sa, sa), args.iters, args.warmup, flush)
    with torch.no_grad():
        t_lin = _time(lambda: fp8_linear(a, b, None, False), args.iters, args.warmup, flush)
    t_bf16 = _time(lambda: gemm(a, b, out=out), args.iters, args.warmup, flush)
    return {"op": "gemm_fp8_nt", "m": m, "n": n, "k": k, "ms": t, "tflops": flops / t / 1e9, "cast_transpose_ms": t_cast,
            "cast_gbs": (m * k * 4) / t_cast / 1e6, "fp8_linear_fwd_ms": t_lin, "bf16_gemm_ms": t_bf16, "bf16_tflops": flops / t_bf16 / 1e9}


def bench_attention(args, flush):
    from . import attention
    from .mask import AttentionMask

    b, s, h, hk, d = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
    bf = dict(device="cuda", dtype=torch.bfloat16)
    q = torch.randn(b, s, h, d, requires_grad=True, **bf)
    k = torch.randn(b, s, hk, d, requires_grad=True, **bf)
    v = torch.randn(b, s, hk, d, requires_grad=True, **bf)
    doc = args.doc or s
    doc_ids = (torch.arange(s, device="cuda", dtype=torch.int32) // doc).unsqueeze(0).expand(b, s).contiguous()
    mask = AttentionMask(causal=True, doc_ids=doc_ids if doc < s else None)
    # block-causal: each query sees (pos_in_doc + 1) keys
    pairs = b * h * (s // doc) * doc * (doc + 1) / 2
    fwd_flops = 4.0 * pairs * d
    res = {"op": "attention", "batch": b, "seq": s, "doc": doc, "heads": h, "kv_heads": hk, "head_dim": d}
    with torch.no_grad():
        t = _time(lambda: attention(q, k, v, mask), args.iters, args.warmup, flush)
    res.update(fwd_ms=t, fwd_tflops=fwd_flops / t / 1e9)
    out = attention(q, k, v, mask)
    go = torch.randn_like(out)
    t = _time(lambda: torch.autograd.grad(out, (q, k, v), go, retain_graph=True), args.iters, args.warmup, flush)
    res.update(bwd_ms=t, bwd_tflops=2.5 * fwd_flops / t / 1e9)
    return res


def bench_rmsnorm(args, flush):
    from . import rms_norm

    x = torch.randn(args.rows, args.dim, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(args.dim, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        t = _time(lambda: rms_norm(x, w, 1e-5), args.iters, args.warmup, flush)
    nbytes = 2.0 * x.numel() * 2
    return {"op": "rmsnorm_fwd", "rows": args.rows, "dim": args.dim, "ms": t, "gbs": nbytes / t / 1e6}


def bench_adamw(args, flush):
    from ._cuda import adamw_multi

    n = args.numel
    p = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    m = torch.zeros(n, device="cuda", dtype=torch.bfloat16)  # moments are kept in the parameter dtype
    v = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    state = {"step": 0, "exp_avg": m, "exp_avg_sq": v}

    def run():
        state["step"] += 1
        adamw_multi([(p, g, state)], lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)

    t = _time(run, args.iters, args.warmup, flush)
    nbytes = n * (2 + 2 + 2 + 4 * 2)  # p r/w, g r, m and v r/w (all bf16)
    return {"op": "adamw", "numel": n, "ms": t, "gbs": nbytes / t / 1e6}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--layout", choices=["nt", "nn", "tn"], default="nt")
    g.add_argument("--no-lib", action="store_true")
    f = sub.add_parser("gemm_fp8")
    f.add_argument("--m", type=int, default=8192)
    f.add_argument("--n", type=int, default=4096)
    f.add_argument("--k", type=int, default=4096)
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=4)
    a.add_argument("--seq", type=int, default=2048)
    a.add_argument("--doc", type=int, default=512)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    r = sub.add_parser("rmsnorm")
    r.add_argument("--rows", type=int, default=8192)
    r.add_argument("--dim", type=int, default=4096)
    o = sub.add_parser("adamw")
    o.add_argument("--numel", type=int, default=1 << 28)
    args = ap.parse_args()
    from ._lib import check_device_errors

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = {"gemm": bench_gemm, "gemm_fp8": bench_gemm_fp8, "attention": bench_attention, "rmsnorm": bench_rmsnorm, "adamw": bench_adamw}[args.op]
    res = fn(args, flush)
    check_device_errors()
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()

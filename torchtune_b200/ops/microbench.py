"""Single-op micro-benchmarks for the sm_100a kernels, timed with CUDA events.

    python -m torchtune_b200.ops.microbench gemm --m 8192 --n 4096 --k 4096 --layout nt
    python -m torchtune_b200.ops.microbench attention --batch 4 --seq 2048 --doc 512
    python -m torchtune_b200.ops.microbench rmsnorm --rows 8192 --dim 4096
    python -m torchtune_b200.ops.microbench adamw --numel 268435456
    python -m torchtune_b200.ops.microbench adamw8bit --numel 268435456
    python -m torchtune_b200.ops.microbench gate_up --tokens 8192 --dim 4096 --hidden 14336
    python -m torchtune_b200.ops.microbench comm --world 8 --numel 268435456             (peer-memory kernels, ranks emulated on one GPU)
    python -m torchtune_b200.ops.microbench suite --tokens 8192      (norm, RoPE, SwiGLU, loss, embedding, LoRA, grouped GEMM, NF4, offload copies)

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


def bench_gemm_mxfp8(args, flush):
    """Block-scaled fp8 GEMM alone, its two quantisers, and the whole linear forward (2 quantisations + GEMM) against the bf16 GEMM."""
    from ._cuda import gemm, gemm_mxfp8, mx_quantize, mxfp8_linear

    m, n, k = args.m, args.n, args.k
    bf = dict(device="cuda", dtype=torch.bfloat16)
    a, b = torch.randn(m, k, **bf), torch.randn(n, k, **bf) * 0.05
    aq, asf = mx_quantize(a)
    bq, bsf = mx_quantize(b)
    out = torch.empty(m, n, **bf)
    flops = 2.0 * m * n * k
    t = _time(lambda: gemm_mxfp8(aq, asf, bq, bsf, out=out), args.iters, args.warmup, flush)
    t_q = _time(lambda: mx_quantize(a), args.iters, args.warmup, flush)
    t_qt = _time(lambda: mx_quantize(a, transpose=True), args.iters, args.warmup, flush)
    from ._cuda import mx_quantize_both

    t_qb = _time(lambda: mx_quantize_both(a), args.iters, args.warmup, flush)
    with torch.no_grad():
        t_lin = _time(lambda: mxfp8_linear(a, b, None), args.iters, args.warmup, flush)
    t_bf16 = _time(lambda: gemm(a, b, out=out), args.iters, args.warmup, flush)
    return {"op": "gemm_mxfp8_nt", "m": m, "n": n, "k": k, "ms": t, "tflops": flops / t / 1e9, "quantize_ms": t_q, "quantize_gbs": (m * k * 3) / t_q / 1e6,
            "quantize_transposed_ms": t_qt, "quantize_both_ms": t_qb, "mxfp8_linear_fwd_ms": t_lin, "bf16_gemm_ms": t_bf16, "bf16_tflops": flops / t_bf16 / 1e9}


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
    import torch.nn.functional as F

    from . import rms_norm

    x = torch.randn(args.rows, args.dim, device="cuda", dtype=torch.bfloat16).requires_grad_()
    w = torch.ones(args.dim, device="cuda", dtype=torch.bfloat16).requires_grad_()
    go = torch.randn(args.rows, args.dim, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        t = _time(lambda: rms_norm(x, w, 1e-5), args.iters, args.warmup, flush)
        t_lib = _time(lambda: F.rms_norm(x, (args.dim,), w, 1e-5), args.iters, args.warmup, flush)

    def both(fn):
        def run():
            x.grad = w.grad = None
            fn().backward(go)
        return run

    t2 = _time(both(lambda: rms_norm(x, w, 1e-5)), args.iters, args.warmup, flush)
    t2_lib = _time(both(lambda: F.rms_norm(x, (args.dim,), w, 1e-5)), args.iters, args.warmup, flush)
    nbytes = 2.0 * x.numel() * 2
    return {"op": "rmsnorm", "rows": args.rows, "dim": args.dim, "ms": t, "gbs": nbytes / t / 1e6, "lib_ms": t_lib,
            "fwd_bwd_ms": t2, "fwd_bwd_gbs": 2.5 * nbytes / t2 / 1e6, "lib_fwd_bwd_ms": t2_lib}


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


def bench_adamw8bit(args, flush):
    from ._cuda import adamw8bit

    n = args.numel
    p = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    mq, vq = torch.zeros(n, device="cuda", dtype=torch.int8), torch.zeros(n, device="cuda", dtype=torch.uint8)
    ms, vs = torch.zeros((n + 255) // 256, device="cuda"), torch.zeros((n + 255) // 256, device="cuda")
    step = [0]

    def run():
        step[0] += 1
        adamw8bit(p, g, mq, vq, ms, vs, step[0], 1e-4, 0.9, 0.999, 1e-8, 0.01)

    t = _time(run, args.iters, args.warmup, flush)
    nbytes = n * (2 * 2 + 2 + 2 * 2) + 4 * ms.numel() * 4  # p r/w, g r, one-byte codes of both moments r/w, block scales r/w
    return {"op": "adamw8bit", "numel": n, "ms": t, "gbs": nbytes / t / 1e6, "state_bytes_per_param": 2 + 8 / 256}


def bench_gate_up(args, flush):
    """Gate / up projections + SwiGLU of one MLP: the fused CTA-pair kernel against two GEMMs followed by the SwiGLU kernel,
    without (inference / first checkpointed forward) and with (recomputed forward) the pre-activations kept for backward."""
    from . import _cuda

    T, D, H = args.tokens, args.dim, args.hidden
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16) * 0.5
    w1 = torch.randn(H, D, device="cuda", dtype=torch.bfloat16) * 0.02
    w3 = torch.randn(H, D, device="cuda", dtype=torch.bfloat16) * 0.02
    flops = 2 * 2.0 * T * D * H
    out = {"op": "gate_up", "tokens": T, "dim": D, "hidden": H}

    def unfused():
        return _cuda.swiglu(_cuda.gemm(x, w1), _cuda.gemm(x, w3))

    with torch.no_grad():
        t = _time(lambda: _cuda.gate_up_swiglu(x, w1, w3), args.iters, args.warmup, flush)
        out["fused_nograd_ms"], out["fused_nograd_tflops"] = t, flops / t / 1e9
        t = _time(unfused, args.iters, args.warmup, flush)
        out["unfused_nograd_ms"], out["unfused_nograd_tflops"] = t, flops / t / 1e9
    xg, w1g, w3g = x.clone().requires_grad_(), w1.clone().requires_grad_(), w3.clone().requires_grad_()
    t = _time(lambda: _cuda.gate_up_swiglu(xg, w1g, w3g), args.iters, args.warmup, flush)
    out["fused_grad_ms"], out["fused_grad_tflops"] = t, flops / t / 1e9
    t = _time(lambda: _cuda.swiglu(_cuda.linear(xg, w1g, None), _cuda.linear(xg, w3g, None)), args.iters, args.warmup, flush)
    out["unfused_grad_ms"], out["unfused_grad_tflops"] = t, flops / t / 1e9
    return out


def bench_comm(args, flush):
    """The two peer-memory communication kernels with every rank's buffers on this one GPU (no peer sits behind NVLink here, so the
    figures are the kernels' own HBM efficiency): the fused reduce → AdamW → broadcast bucket kernel of rank 0 over ``--world``
    gradient / parameter buffers, its reduce-scatter → AdamW form (no broadcast: the ZeRO-3 update) and the ZeRO-3 bucket gather."""
    import ctypes
    import math

    from ..parallel.dp import _declare_dp
    from ._lib import check, lib, stream_ptr

    L = lib()
    _declare_dp(L)
    world, shard = args.world, args.numel // args.world // 8 * 8
    total = shard * world
    params = [torch.randn(total, device="cuda", dtype=torch.bfloat16) * 0.1 for _ in range(world)]
    grads = [torch.randn(total, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    m, v = torch.zeros(shard, device="cuda", dtype=torch.bfloat16), torch.zeros(shard, device="cuda", dtype=torch.bfloat16)
    gp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in grads])
    pp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in params])

    def update(bcast):
        check(L.ttb_dp_reduce_adamw_bcast(gp, pp, world, 0, 0, shard, m.data_ptr(), v.data_ptr(), None, None, None, 1.0, 1e-4, 0.9, 0.999, 1e-8, 0.01, 10.0, 1.0 / math.sqrt(1 - 0.999), 0,
                                          None, 0, 0, None, 0, int(bcast), 0, stream_ptr()), "dp kernel")

    out = {"op": "comm", "world": world, "shard_numel": shard}
    t = _time(lambda: update(True), args.iters, args.warmup, flush)
    nbytes = shard * 2 * (world + 3 + 2 + world)  # gradient rows of all ranks, own parameter + moments read; moments + parameter copies of all ranks written
    out["reduce_adamw_bcast_ms"], out["reduce_adamw_bcast_gbs"] = t, nbytes / t / 1e6
    t = _time(lambda: update(False), args.iters, args.warmup, flush)
    nbytes = shard * 2 * (world + 3 + 3)
    out["reduce_scatter_adamw_ms"], out["reduce_scatter_adamw_gbs"] = t, nbytes / t / 1e6
    dst = torch.empty(total, device="cuda", dtype=torch.bfloat16)
    shards = [p[:shard] for p in params]
    sp = (ctypes.c_void_p * world)(*[t_.data_ptr() for t_ in shards])
    t = _time(lambda: check(L.ttb_zero3_gather(sp, world, 0, shard, dst.data_ptr(), None, 0, 0, None, 0, stream_ptr()), "gather"), args.iters, args.warmup, flush)
    out["zero3_gather_ms"], out["zero3_gather_gbs"] = t, 2 * total * 2 / t / 1e6
    return out


def bench_suite(args, flush):
    """The memory-bound and fused operators of one Llama-3.1-8B training step (``--tokens`` rows, width 4096, MLP 14336,
    vocabulary 128256) and of a Llama-4-Scout MoE layer (16 experts, 5120 → 8192), each against the PyTorch library expression of
    the same maths on identical inputs.  Prints one JSON line per operator."""
    import torch.nn.functional as F

    from . import embedding, grouped_matmul, linear_cross_entropy, lora_linear, rms_norm, rope, swiglu

    T, D, H, V = args.tokens, 4096, 14336, 128256
    bf = dict(device="cuda", dtype=torch.bfloat16)
    it, wu = args.iters, args.warmup
    rows = []

    def emit(op, ours_ms, lib_ms, **kw):
        r = {"op": op, "ms": round(ours_ms, 4), "lib_ms": round(lib_ms, 4), "speedup_vs_lib": round(lib_ms / ours_ms, 2), **kw}
        for key in ("gbs", "tflops"):
            if key in r:
                r[key] = round(r[key], 1)
        rows.append(r)
        print(json.dumps(r), flush=True)

    def fwd_bwd(fn, inputs, go):
        def run():
            for t in inputs:
                t.grad = None
            fn().backward(go)
        return run

    # RMSNorm forward + backward: x read twice, y and dx written, dy read
    x = torch.randn(T, D, **bf).requires_grad_()
    w = torch.ones(D, **bf).requires_grad_()
    go = torch.randn(T, D, **bf)
    t_o = _time(fwd_bwd(lambda: rms_norm(x, w, 1e-5), (x, w), go), it, wu, flush)
    t_l = _time(fwd_bwd(lambda: F.rms_norm(x, (D,), w, 1e-5), (x, w), go), it, wu, flush)
    emit("rmsnorm_fwd_bwd", t_o, t_l, rows=T, dim=D, gbs=5.0 * T * D * 2 / t_o / 1e6)

    # RoPE forward on q ([b, s, 32, 128])
    b, sq = T // 2048, 2048
    q = torch.randn(b, sq, 32, 128, **bf)
    half = torch.arange(64, device="cuda", dtype=torch.float32)
    ang = torch.arange(sq, device="cuda", dtype=torch.float32)[:, None] * (500000.0 ** (-half / 64))[None]
    cache = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()

    def rope_lib():
        xf = q.float().reshape(b, sq, 32, 64, 2)
        c = cache.view(1, sq, 1, 64, 2)
        return torch.stack([xf[..., 0] * c[..., 0] - xf[..., 1] * c[..., 1], xf[..., 1] * c[..., 0] + xf[..., 0] * c[..., 1]], -1).flatten(3).to(q.dtype)

    with torch.no_grad():
        t_o = _time(lambda: rope(q, cache), it, wu, flush)
        t_l = _time(rope_lib, it, wu, flush)
    emit("rope_fwd", t_o, t_l, shape=[b, sq, 32, 128], gbs=2.0 * q.numel() * 2 / t_o / 1e6)

    # SwiGLU forward + backward: gate, up, dy read; y, dgate, dup written (+ gate, up re-read in backward)
    g1 = torch.randn(T, H, **bf).requires_grad_()
    u1 = torch.randn(T, H, **bf).requires_grad_()
    goh = torch.randn(T, H, **bf)
    t_o = _time(fwd_bwd(lambda: swiglu(g1, u1), (g1, u1), goh), it, wu, flush)
    t_l = _time(fwd_bwd(lambda: F.silu(g1) * u1, (g1, u1), goh), it, wu, flush)
    emit("swiglu_fwd_bwd", t_o, t_l, rows=T, dim=H, gbs=8.0 * T * H * 2 / t_o / 1e6)
    del g1, u1, goh

    # fused linear + cross-entropy, forward + backward (3 GEMMs of 2·T·D·V)
    hid = (torch.randn(T, D, **bf) * 0.5).requires_grad_()
    wv = (torch.randn(V, D, **bf) * 0.02).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    one = torch.ones((), device="cuda")

    def ce_ours():
        hid.grad = wv.grad = None
        linear_cross_entropy(hid, wv, labels)[0].backward(one)

    def ce_lib():
        hid.grad = wv.grad = None
        F.cross_entropy(F.linear(hid, wv).float(), labels, reduction="sum").backward(one)

    t_o = _time(ce_ours, it, wu, flush)
    t_l = _time(ce_lib, it, wu, flush)
    emit("linear_cross_entropy_fwd_bwd", t_o, t_l, tokens=T, dim=D, vocab=V, tflops=6.0 * T * D * V / t_o / 1e9)
    del wv, hid

    # embedding gather + gradient
    table = (torch.randn(V, D, **bf) * 0.02).requires_grad_()
    toks = torch.randint(0, V, (T,), device="cuda")
    t_o = _time(fwd_bwd(lambda: embedding(toks, table), (table,), go), it, wu, flush)
    t_l = _time(fwd_bwd(lambda: F.embedding(toks, table), (table,), go), it, wu, flush)
    emit("embedding_fwd_bwd", t_o, t_l, tokens=T, dim=D, vocab=V)
    del table

    # LoRA-fused linear (rank 64) forward: base GEMM + adapter in one kernel
    xl = torch.randn(T, D, **bf)
    wl = torch.randn(D, D, **bf) * 0.02
    la, lb = torch.randn(64, D, **bf) * 0.02, torch.randn(D, 64, **bf) * 0.02
    with torch.no_grad():
        t_o = _time(lambda: lora_linear(xl, xl, wl, None, la, lb, 2.0), it, wu, flush)
        t_l = _time(lambda: F.linear(xl, wl) + 2.0 * F.linear(F.linear(xl, la), lb), it, wu, flush)
    emit("lora_linear_fwd", t_o, t_l, m=T, n=D, k=D, rank=64, tflops=2.0 * T * D * (D + 128) / t_o / 1e9)

    # grouped expert GEMM, Scout shapes: 16 experts, top-1, uneven loads
    E, Dm, Hm = 16, 5120, 8192
    gen = torch.Generator(device="cuda").manual_seed(0)
    assign = torch.multinomial(torch.rand(E, device="cuda", generator=gen) + 0.2, T, replacement=True, generator=gen)
    counts = torch.bincount(assign, minlength=E).to(torch.int32)
    xe = torch.randn(T, Dm, **bf)
    we = torch.randn(E, Dm, Hm, **bf) * 0.02
    sizes = counts.tolist()

    def grouped_lib():
        outs, st = [], 0
        for e, n in enumerate(sizes):
            outs.append(xe[st : st + n] @ we[e])
            st += n
        return torch.cat(outs)

    with torch.no_grad():
        t_o = _time(lambda: grouped_matmul(xe, we, counts), it, wu, flush)
        t_l = _time(grouped_lib, it, wu, flush)
    emit("grouped_gemm_fwd", t_o, t_l, tokens=T, experts=E, k=Dm, n=Hm, tflops=2.0 * T * Dm * Hm / t_o / 1e9)
    del we, xe

    # NF4 dequantise (4096 × 14336): 0.5 B read + 2 B written per element
    from ..modules.low_precision.nf4 import NF4Weight

    nf4 = NF4Weight(H, D, device="cuda")
    nf4.quantize_(torch.randn(H, D, **bf) * 0.02)
    t_o = _time(lambda: nf4.dequantize(torch.bfloat16), it, wu, flush)
    emit("nf4_dequantize", t_o, t_o, shape=[H, D], gbs=2.53 * H * D / t_o / 1e6)

    # activation offload path: pinned host <-> device copies of 1 GiB on a side stream
    n = 1 << 30
    dev_buf = torch.empty(n, dtype=torch.uint8, device="cuda")
    host = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    t_d2h = _time(lambda: host.copy_(dev_buf, non_blocking=True), it, wu, flush)
    t_h2d = _time(lambda: dev_buf.copy_(host, non_blocking=True), it, wu, flush)
    r = {"op": "offload_copy_1GiB", "d2h_ms": round(t_d2h, 3), "h2d_ms": round(t_h2d, 3), "d2h_gbs": round(n / t_d2h / 1e6, 1), "h2d_gbs": round(n / t_h2d / 1e6, 1)}
    print(json.dumps(r), flush=True)
    rows.append(r)
    return {"op": "suite", "tokens": T, "operators": len(rows)}


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
    fm = sub.add_parser("gemm_mxfp8")
    fm.add_argument("--m", type=int, default=8192)
    fm.add_argument("--n", type=int, default=4096)
    fm.add_argument("--k", type=int, default=4096)
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
    o8 = sub.add_parser("adamw8bit")
    o8.add_argument("--numel", type=int, default=1 << 28)
    gu = sub.add_parser("gate_up")
    gu.add_argument("--tokens", type=int, default=8192)
    gu.add_argument("--dim", type=int, default=4096)
    gu.add_argument("--hidden", type=int, default=14336)
    co = sub.add_parser("comm")
    co.add_argument("--world", type=int, default=8)
    co.add_argument("--numel", type=int, default=1 << 28)
    su = sub.add_parser("suite")
    su.add_argument("--tokens", type=int, default=8192)
    args = ap.parse_args()
    from ._lib import check_device_errors

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = {"gemm": bench_gemm, "gemm_fp8": bench_gemm_fp8, "gemm_mxfp8": bench_gemm_mxfp8, "attention": bench_attention, "rmsnorm": bench_rmsnorm, "adamw": bench_adamw, "adamw8bit": bench_adamw8bit, "gate_up": bench_gate_up, "comm": bench_comm, "suite": bench_suite}[args.op]
    res = fn(args, flush)
    check_device_errors()
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()

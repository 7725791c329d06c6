"""Multi-rank micro-benchmarks of the fused collective GEMMs against NCCL + plain GEMM.

Launch one process per GPU, e.g.::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29555 \
        -m torchtune_b200.parallel.microbench --rows 4096 --dim 8192 --hidden 28672 --iters 20

Per shape it times, with CUDA events on the compute stream and the maximum over ranks:

* ``ag_gemm``  — fused all-gather → GEMM           vs ``all_gather_into_tensor`` + tcgen05 GEMM,
* ``gemm_rs``  — fused GEMM → reduce-scatter(+sum) vs tcgen05 GEMM + ``reduce_scatter_tensor``.

``--rows`` is the total number of tokens (all ranks), ``--dim`` the model width and ``--hidden`` the *global*
MLP width (each rank holds ``hidden / world`` of it), i.e. the shapes of one Megatron-style MLP block
(column-parallel w1/w3 then row-parallel w2, torchtune/models/llama3/_parallelism.py:33-59).
Rank 0 prints one JSON line per measurement.

``--op ep`` times the expert-parallel MoE layer instead (``--rows`` tokens over all ranks, ``--dim``, ``--hidden`` expert width,
``--experts``, ``--top-k``): the plan / push / pull kernels, the layer forward and forward+backward.  ``--op wg`` times the
sharded-parameter forward (``--rows`` tokens per rank, weight ``[--hidden, --dim]`` split over the ranks).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters: int, warmup: int, flush: torch.Tensor) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.zero_()  # evict L2 between timed iterations
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_ep(args, dev, world, rank) -> None:
    """Expert-parallel MoE layer (Llama-4 Scout shapes by default): the exchange steps alone, the whole layer forward and
    forward+backward, and NCCL ``all_to_all_single`` moving the same number of rows as a reference for the exchange."""
    from ..models.llama4 import llama4_moe
    from ..ops._lib import check_device_errors
    from .ep import ExpertParallelContext, ExpertParallelMoE

    T, dim, hid, E, k = args.rows // world, args.dim, args.hidden, args.experts, args.top_k
    torch.manual_seed(0)
    full = llama4_moe(dim=dim, hidden_dim=hid, num_experts=E, experts_per_token=k).to(dev).bfloat16()
    ep = ExpertParallelContext(dev, None, num_experts=E, dim=dim, max_pairs=T * k, capacity_factor=args.capacity_factor)
    moe = ExpertParallelMoE(full, ep)
    del full
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = (torch.randn(1, T, dim, generator=g, device=dev) * 0.5).bfloat16().requires_grad_()
    dy = (torch.randn(1, T, dim, generator=g, device=dev) * 0.1).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flat = x.detach().reshape(T, dim)
    with torch.no_grad():
        scores, token_idx, counts = moe.router(flat)
    plan = ep.plan(counts, T * k)
    y_local = torch.zeros(ep.capacity, dim, dtype=torch.bfloat16, device=dev)
    send = torch.empty(T * k, dim, dtype=torch.bfloat16, device=dev)
    recv = torch.empty_like(send)

    def fwd_bwd():
        x.grad = None
        moe(x).backward(dy)

    def fwd():
        with torch.no_grad():
            moe(x)

    def nccl_a2a():  # balanced all-to-all of the same number of rows (gather + send; no re-permutation)
        torch.index_select(flat, 0, token_idx, out=send)
        dist.all_to_all_single(recv, send)

    results = []
    for name, fn in (
        ("ep_plan", lambda: ep.plan(counts, T * k)),
        ("ep_dispatch_push", lambda: ep.push(flat, token_idx, scores, plan)),
        ("ep_combine_publish_pull", lambda: (ep.publish_result(y_local), ep.pull(plan, torch.bfloat16))),
        ("nccl_gather_all_to_all", nccl_a2a),
        ("ep_moe_forward", fwd),
        ("ep_moe_forward_backward", fwd_bwd),
    ):
        ms = _time(fn, args.iters, args.warmup, flush)
        results.append({"op": name, "world": world, "tokens_per_rank": T, "dim": dim, "hidden": hid, "experts": E, "top_k": k, "ms": round(ms, 4)})
    check_device_errors()
    row_bytes = T * k * dim * 2 * (world - 1) / world
    if rank == 0:
        for r in results:
            if r["op"] in ("ep_dispatch_push", "nccl_gather_all_to_all"):
                r["nvlink_gbs_per_gpu"] = round(row_bytes / r["ms"] / 1e6, 1)
            print(json.dumps(r))
    ep.close()


def bench_wg(args, dev, world, rank) -> None:
    """Sharded-parameter forward: fused weight all-gather → GEMM against NCCL ``all_gather_into_tensor`` of the weight + GEMM and
    against the GEMM alone.  ``--rows`` tokens per rank, weight ``[--hidden, --dim]`` split by rows over the ranks."""
    from ..ops._cuda import gemm
    from ..ops._lib import check_device_errors
    from .fsdp import ShardedWeightContext

    T, K, N = args.rows, args.dim, args.hidden
    rows = N // world
    sw = ShardedWeightContext(dev, None, store_numel=rows * K, max_weight_numel=N * K, max_out_features=N)
    g = torch.Generator(device="cuda").manual_seed(rank)
    shard = sw.place((torch.randn(rows, K, generator=g, device=dev) * 0.02).bfloat16())
    x = (torch.randn(T, K, generator=g, device=dev) * 0.3).bfloat16()
    w_local = (torch.randn(N, K, generator=g, device=dev) * 0.02).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sw.barrier()

    def nccl_path():
        return gemm(x, sw.gather(shard))

    a, b = sw.linear(x, shard, None), nccl_path()
    torch.cuda.synchronize()
    err = float((a.float() - b.float()).abs().max() / b.float().abs().max())
    flops = 2.0 * T * K * N
    results = []
    for name, fn in (("wg_gemm_fused", lambda: sw.linear(x, shard, None)), ("wg_gemm_nccl", nccl_path), ("gemm_only_local", lambda: gemm(x, w_local))):
        ms = _time(fn, args.iters, args.warmup, flush)
        results.append({"op": name, "world": world, "tokens": T, "dim": K, "out_features": N, "ms": round(ms, 4), "tflops_per_gpu": round(flops / ms / 1e9, 1)})
    check_device_errors()
    if rank == 0:
        print(json.dumps({"rel_err_fused_vs_nccl": err, "weight_bytes_over_nvlink_per_gpu": (world - 1) * rows * K * 2}))
        for r in results:
            print(json.dumps(r))
    sw.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["tp", "ep", "wg"], default="tp")
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=1)
    ap.add_argument("--capacity-factor", type=float, default=None)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--dim", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", local)

    if args.op in ("ep", "wg"):
        (bench_ep if args.op == "ep" else bench_wg)(args, dev, world, rank)
        dist.destroy_process_group()
        return

    from ..ops._cuda import gemm
    from ..ops._lib import check_device_errors
    from .tp import TensorParallelContext

    rows = args.rows // world
    hid = args.hidden // world
    tp = TensorParallelContext(dev, None, max_rows_per_rank=rows, max_width=max(args.dim, hid))
    g = torch.Generator(device="cuda").manual_seed(rank)
    x_shard = (torch.randn(rows, args.dim, generator=g, device=dev) * 0.3).bfloat16()
    w_col = (torch.randn(hid, args.dim, generator=g, device=dev) * 0.02).bfloat16()  # column-parallel [N_r, K]
    h_full = (torch.randn(rows * world, hid, generator=g, device=dev) * 0.3).bfloat16()
    w_row = (torch.randn(args.dim, hid, generator=g, device=dev) * 0.02).bfloat16()  # row-parallel [N, K_r]
    x_full_local = (torch.randn(rows * world, args.dim, generator=g, device=dev) * 0.3).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def nccl_ag_gemm():
        full = torch.empty(rows * world, args.dim, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, x_shard)
        return gemm(full, w_col)

    def nccl_gemm_rs():
        part = gemm(h_full, w_row)
        out = torch.empty(rows, args.dim, dtype=torch.bfloat16, device=dev)
        dist.reduce_scatter_tensor(out, part)
        return out

    # numerics of the fused paths against the NCCL paths (bf16 reduction order differs)
    a, b = tp.ag_gemm(x_shard, w_col), nccl_ag_gemm()
    c, d = tp.gemm_rs(h_full, w_row), nccl_gemm_rs()
    torch.cuda.synchronize()
    err_ag = float((a.float() - b.float()).abs().max() / b.float().abs().max())
    err_rs = float((c.float() - d.float()).abs().max() / d.float().abs().max())

    flops_col = 2.0 * rows * world * args.dim * hid
    results = []
    for name, fn, flops in (
        ("ag_gemm_fused", lambda: tp.ag_gemm(x_shard, w_col), flops_col),
        ("ag_gemm_nccl", nccl_ag_gemm, flops_col),
        ("gemm_rs_fused", lambda: tp.gemm_rs(h_full, w_row), flops_col),
        ("gemm_rs_nccl", nccl_gemm_rs, flops_col),
        ("gemm_only_local", lambda: gemm(x_full_local, w_col), flops_col),
    ):
        ms = _time(fn, args.iters, args.warmup, flush)
        results.append({"op": name, "world": world, "rows": rows * world, "dim": args.dim, "hidden_per_rank": hid, "ms": round(ms, 4),
                        "tflops_per_gpu": round(flops / ms / 1e9, 1)})
    check_device_errors()
    if rank == 0:
        print(json.dumps({"rel_err_ag_vs_nccl": err_ag, "rel_err_rs_vs_nccl": err_rs}))
        for r in results:
            print(json.dumps(r))
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

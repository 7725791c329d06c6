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


def main() -> None:
    ap = argparse.ArgumentParser()
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

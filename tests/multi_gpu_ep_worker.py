"""Worker for the 2-GPU expert-parallel check: bf16 MoE layer with experts spread over the ranks (peer-memory push / pull,
grouped tcgen05 GEMMs) against an fp32 single-device evaluation of the same layer on the concatenated batch."""
import os

import torch
import torch.distributed as dist


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()

    from torchtune_b200 import ops
    from torchtune_b200.models.llama4 import llama4_moe
    from torchtune_b200.ops._lib import check_device_errors
    from torchtune_b200.parallel.ep import ExpertParallelContext, ExpertParallelMoE

    DIM, HID, E, K, TOK = 256, 512, 8, 2, 192
    torch.manual_seed(0)
    full = llama4_moe(dim=DIM, hidden_dim=HID, num_experts=E, experts_per_token=K).to(dev)
    with torch.no_grad():
        for p in full.parameters():
            p.copy_((torch.randn_like(p) * 0.05).bfloat16().float())
    xs = [(torch.randn(1, TOK, DIM, generator=torch.Generator().manual_seed(50 + r)) * 0.5).bfloat16() for r in range(world)]
    dys = [(torch.randn(1, TOK, DIM, generator=torch.Generator().manual_seed(80 + r)) * 0.1).bfloat16() for r in range(world)]

    # fp32 oracle on all tokens
    with ops.use_reference_ops():
        xr = torch.cat(xs, dim=1).float().to(dev).requires_grad_()
        yr = full(xr)
        yr.backward(torch.cat(dys, dim=1).float().to(dev))
        sel_ref = full.router.selected_experts_indices.sort(dim=1).values

    import copy

    ep = ExpertParallelContext(dev, None, num_experts=E, dim=DIM, max_pairs=TOK * K)
    moe = ExpertParallelMoE(copy.deepcopy(full).bfloat16(), ep)
    for p in moe.parameters():
        p.grad = None
    x = xs[rank].to(dev).requires_grad_()
    for _ in range(2):  # second pass reuses the exchange buffers
        x.grad = None
        for p in moe.parameters():
            p.grad = None
        y = moe(x)
        y.backward(dys[rank].to(dev))
    torch.cuda.synchronize()
    check_device_errors()

    sl = slice(rank * TOK, (rank + 1) * TOK)
    # tokens whose bf16 routing differs from the fp32 oracle (near-ties) are excluded from the comparison
    same = (moe.router.selected_experts_indices.sort(dim=1).values == sel_ref[sl]).all(dim=1)
    assert same.float().mean() > 0.8, same.float().mean()

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9))

    e_y = rel(y[0][same], yr[0, sl][same])
    e_dx = rel(x.grad[0][same], xr.grad[0, sl][same])
    assert e_y < 3e-2 and e_dx < 5e-2, (e_y, e_dx)
    if bool(same.all()):
        flags = torch.tensor([1.0], device=dev)
    else:
        flags = torch.tensor([0.0], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if flags.item() == 1.0:  # identical routing everywhere: expert weight gradients are comparable too
        epr = E // world
        e_w = rel(moe.experts.gate_proj.grad, full.experts.gate_proj.grad[rank * epr : (rank + 1) * epr])
        assert e_w < 5e-2, e_w
    ep.close()
    dist.barrier()
    if rank == 0:
        print("EP_OK", e_y, e_dx)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

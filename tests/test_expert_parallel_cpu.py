"""Expert-parallel MoE on CPU (gloo, 2 ranks): every rank routes its own tokens to experts spread over the ranks; outputs,
input gradients, replicated-parameter gradients (after the group sum) and the expert gradients of each owner must equal one
process that holds all experts and sees the concatenated batch."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torchtune_b200.models.llama4 import llama4_moe
from torchtune_b200.parallel.ep import ExpertParallelContext, ExpertParallelMoE, expert_parallelize

DIM, HID, E, K, TOK = 16, 24, 4, 2, 12


def _moe():
    torch.manual_seed(0)
    moe = llama4_moe(dim=DIM, hidden_dim=HID, num_experts=E, experts_per_token=K)
    with torch.no_grad():
        for p in moe.parameters():
            p.copy_(torch.randn_like(p) * 0.2)
    return moe


def _data(rank):
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randn(1, TOK, DIM, generator=g), torch.randn(1, TOK, DIM, generator=g)


def _worker(rank, world, port, results, capacity_factor):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ep = ExpertParallelContext(torch.device("cpu"), num_experts=E, dim=DIM, max_pairs=TOK * K, capacity_factor=capacity_factor)
        holder = torch.nn.ModuleDict({"moe": _moe()})
        expert_parallelize(holder, ep)
        assert isinstance(holder["moe"], ExpertParallelMoE)
        x, dy = _data(rank)
        x.requires_grad_()
        y = holder["moe"](x)
        y.backward(dy)
        holder.sync_replicated_grads()
        m = holder["moe"]
        results[rank] = dict(
            y=y.detach().clone(), dx=x.grad.clone(), gate=m.router.gate.weight.grad.clone(), shared=m.shared_expert.w1.weight.grad.clone(),
            experts={n: getattr(m.experts, n).grad.clone() for n in ("gate_proj", "up_proj", "down_proj")},
            sd={k: v.clone() for k, v in holder.full_state_dict().items()},
        )
    finally:
        dist.destroy_process_group()


def _reference(world):
    moe = _moe()
    xs, dys = zip(*[_data(r) for r in range(world)])
    x = torch.cat(xs, dim=1).requires_grad_()
    y = moe(x)
    y.backward(torch.cat(dys, dim=1))
    return moe, x, y


def test_expert_parallel_moe_matches_single_process():
    world = 2
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29571, results, None), nprocs=world, join=True)
    moe, x, y = _reference(world)
    epr = E // world
    for rank in range(world):
        r = results[rank]
        sl = slice(rank * TOK, (rank + 1) * TOK)
        torch.testing.assert_close(r["y"], y[:, sl].detach(), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["dx"], x.grad[:, sl], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["gate"], moe.router.gate.weight.grad, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["shared"], moe.shared_expert.w1.weight.grad, rtol=1e-4, atol=1e-5)
        for n, g in r["experts"].items():
            torch.testing.assert_close(g, getattr(moe.experts, n).grad[rank * epr : (rank + 1) * epr], rtol=1e-4, atol=1e-5)
        ref_sd = {f"moe.{k}": v for k, v in moe.state_dict().items()}
        assert set(r["sd"]) == set(ref_sd)
        for k in ref_sd:
            assert torch.equal(r["sd"][k], ref_sd[k]), k


def test_expert_parallel_single_rank_and_bounded_capacity():
    moe = _moe()
    x, _ = _data(0)
    want = moe(x)
    ep = ExpertParallelContext(torch.device("cpu"), num_experts=E, dim=DIM, max_pairs=TOK * K)
    got = ExpertParallelMoE(_moe(), ep)(x)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    # a bounded capacity keeps the buffers small; with world 1 nothing can overflow, the result is unchanged
    ep2 = ExpertParallelContext(torch.device("cpu"), num_experts=E, dim=DIM, max_pairs=TOK * K, capacity_factor=4.0)
    torch.testing.assert_close(ExpertParallelMoE(_moe(), ep2)(x), want, rtol=1e-5, atol=1e-6)

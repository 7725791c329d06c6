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


def _layerwise_worker(rank, world, port, results):
    import weakref

    from torchtune_b200 import parallel as par
    from torchtune_b200 import training
    from torchtune_b200.models.llama4 import llama4_decoder
    from torchtune_b200.modules.moe import GroupedExperts
    from torchtune_b200.training import _distributed as td

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = {"expert_parallel_dim": 2, "batch_size": 1}
        strategy = par.ParallelStrategy(cfg, torch.device("cpu"))
        with training.set_default_dtype(torch.float32), torch.device("meta"):
            model = llama4_decoder(vocab_size=64, num_layers=4, num_heads=2, num_kv_heads=1, embed_dim=16, hidden_dim=24, max_seq_len=32, num_experts=4)
        seen, alive_before = [], []
        original = td.LayerwisePreparer.__call__

        def counting(self, module, prefix=""):
            # full-size expert stacks of the layers prepared so far that are still alive when the next layer gets its storage
            alive_before.append(sum(1 for r in seen if r() is not None and not any(p.is_meta for p in r().parameters())))
            out = original(self, module, prefix)
            seen.extend(weakref.ref(m) for m in module.modules() if isinstance(m, GroupedExperts) and m.num_experts == 4)
            return out

        td.LayerwisePreparer.__call__ = counting
        try:
            strategy.shard_model(model, cfg, None)
        finally:
            td.LayerwisePreparer.__call__ = original
        results[rank] = max(alive_before)
    finally:
        dist.destroy_process_group()


def test_layerwise_expert_sharding_keeps_no_full_expert_stack_alive():
    """While a meta-device MoE model is cut into expert-parallel shards layer by layer, the full expert stacks of an earlier
    layer must be gone before the next layer gets storage (a 109B model never exists in full on one GPU)."""
    results = mp.Manager().dict()
    mp.spawn(_layerwise_worker, args=(2, 29615, results), nprocs=2, join=True)
    assert results[0] == 0 and results[1] == 0

"""Host-side logic of the data-parallel engine on CPU (gloo, world size 2) and mesh arithmetic."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torchtune_b200.parallel import DataParallelEngine, ParallelDims


def test_parallel_dims_validation_and_layout():
    pd = ParallelDims(dp_replicate=2, dp_shard=-1, tp=2, cp=1, world_size=8)
    assert pd.dp_shard == 2 and pd.dp_size == 4 and pd.non_data_parallel_size == 2
    assert pd.min_seq_len_divisor == 2
    assert ParallelDims(dp_shard=-1, tp=2, cp=2, world_size=8).min_seq_len_divisor == 8
    assert pd.coordinates(5) == {"dp_replicate": 1, "dp_shard": 0, "cp": 0, "tp": 1, "dp": 2}
    assert sorted(map(tuple, pd.groups_along("tp"))) == [(0, 1), (2, 3), (4, 5), (6, 7)]
    assert sorted(map(tuple, pd.groups_along("dp"))) == [(0, 2, 4, 6), (1, 3, 5, 7)]
    with pytest.raises(AssertionError):
        ParallelDims(dp_shard=3, tp=2, world_size=8)
    with pytest.raises(AssertionError):
        ParallelDims(dp_shard=-1, tp=3, world_size=8)


def _tiny_model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = _tiny_model()
        eng = DataParallelEngine(torch.device("cpu"))
        eng.prepare(model)
        opt = eng.build_optimizer(model, lr=1e-2, weight_decay=0.1)
        g = torch.Generator().manual_seed(100)
        xs = torch.randn(3, 8, 16, generator=g)
        ys = torch.randn(3, 8, 4, generator=g)
        for step in range(3):
            lo = rank * (8 // world)
            x, y = xs[step, lo : lo + 8 // world], ys[step, lo : lo + 8 // world]
            loss = ((model(x) - y) ** 2).sum()
            loss.backward()
            n = torch.tensor(float(x.shape[0]))
            eng.all_reduce_sum_(n)
            eng.optimizer_step(model, opt, 1.0 / n, clip_grad_norm=1.0 if step == 2 else None)
        results[rank] = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).clone()
        eng.shutdown()
    finally:
        dist.destroy_process_group()


def test_dp_engine_matches_single_process_training():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29650 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    # single-process oracle: whole batch, plain torch AdamW, mean over the global batch
    model = _tiny_model()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1)
    g = torch.Generator().manual_seed(100)
    xs = torch.randn(3, 8, 16, generator=g)
    ys = torch.randn(3, 8, 4, generator=g)
    for step in range(3):
        loss = ((model(xs[step]) - ys[step]) ** 2).sum() / 8
        loss.backward()
        if step == 2:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
    want = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    torch.testing.assert_close(results[0], want, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(results[1], want, rtol=1e-5, atol=1e-6)

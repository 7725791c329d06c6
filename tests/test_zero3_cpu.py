"""Fully sharded parameters (ZeRO-3 engine) on two gloo ranks against one process with ``torch.optim.AdamW``:
the fused per-bucket update during backward, and the deferred update with clipping over two micro-batches.  Also the
gathered checkpoint and a gradient-free forward pass in between."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from helpers import fixed_init_
from torchtune_b200 import training
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.modules import TransformerSelfAttentionLayer
from torchtune_b200.parallel.zero3 import Zero3Engine

ARCH = dict(vocab_size=64, num_layers=3, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48, norm_eps=1e-5, rope_base=10000)
LR, CLIP, STEPS = 1e-2, 0.5, 3


def _batch(rank: int, step: int, micro: int = 0):
    g = torch.Generator().manual_seed(1000 * micro + 100 * rank + step)
    return torch.randint(0, 64, (2, 8), generator=g), torch.randint(0, 64, (2, 8), generator=g)


def _loss(model, tokens, labels):
    return F.cross_entropy(model(tokens).reshape(-1, 64), labels.reshape(-1), reduction="sum")


def _single_process(mode: str, world: int):
    model = llama3_1(**ARCH)
    fixed_init_(model, std=0.1)
    opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=0.01)
    micros = 2 if mode == "deferred" else 1
    norms = []
    for step in range(STEPS):
        total = 0.0
        for micro in range(micros):
            for rank in range(world):
                total = total + _loss(model, *_batch(rank, step, micro))
        (total / (16 * world * micros)).backward()
        if mode in ("deferred", "hsdp"):
            norms.append(float(torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)))
        opt.step()
        opt.zero_grad()
    return {k: v.clone() for k, v in model.state_dict().items()}, norms


def _worker(rank, world, port, mode, ac, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = llama3_1(**ARCH)
        fixed_init_(model, std=0.1)
        if ac:
            training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
        if mode == "hsdp":  # 2 shard groups of 2 ranks: parameters cut in two, the halves replicated across the groups
            from torchtune_b200.parallel.mesh import ParallelDims

            groups = ParallelDims(dp_replicate=2, dp_shard=2, world_size=world).build_groups(("dp_shard", "dp_replicate"))
            engine = Zero3Engine(torch.device("cpu"), groups["dp_shard"], groups["dp_replicate"])
            assert engine.dp_size == 4 and engine.world == 2 and not engine.wants_backward_overlap(None)
        else:
            engine = Zero3Engine(torch.device("cpu"))
        model = engine.prepare(model)
        opt = engine.build_optimizer(model, lr=LR, weight_decay=0.01)
        assert all(p.untyped_storage().size() == 0 for p in model.parameters()), "parameters must not be resident between steps"
        micros = 2 if mode == "deferred" else 1
        scale = 1.0 / (16 * world * micros)
        clipped = mode in ("deferred", "hsdp")
        norms = []
        for step in range(STEPS):
            for micro in range(micros):
                loss = _loss(model, *_batch(rank, step, micro))
                if mode == "fused":
                    assert engine.arm_backward_overlap(opt, scale, None)
                loss.backward()
            norm = engine.optimizer_step(model, opt, scale, CLIP if clipped else None)
            if norm is not None:
                norms.append(float(norm))
            if step == 1:
                with torch.no_grad():  # a gradient-free pass between steps gathers and releases without touching any state
                    model(_batch(rank, 0)[0])
        sd = engine.full_state_dict(model)
        results[rank] = dict(sd=sd, norms=norms, resident=sum(p.untyped_storage().size() for p in model.parameters()))
        engine.shutdown()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,ac", [("fused", True), ("fused", False), ("deferred", True), ("hsdp", True)])
def test_zero3_engine_matches_single_process(mode, ac):
    world = 4 if mode == "hsdp" else 2
    want_sd, want_norms = _single_process(mode, world)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, 29581 + (mode == "deferred") + 2 * ac + 5 * (mode == "hsdp"), mode, ac, results), nprocs=world, join=True)
    for rank in range(world):
        got = results[rank]
        if want_norms:
            torch.testing.assert_close(torch.tensor(got["norms"]), torch.tensor(want_norms), rtol=1e-4, atol=1e-5)
        for k, v in want_sd.items():
            torch.testing.assert_close(got["sd"][k], v, rtol=2e-4, atol=2e-5, msg=lambda m, k=k: f"{k}: {m}")

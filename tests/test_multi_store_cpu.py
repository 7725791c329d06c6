"""The fused sharded optimizer over two flat stores (replicated parameters summed over the job, tensor-parallel shards
summed over their replicas) on a 2 × 2 gloo mesh must train like one process with ``torch.optim.AdamW`` and global-norm
clipping, and its checkpoint form must restore the moments."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from helpers import fixed_init_
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.parallel.stores import MultiStoreAdamW, StoreSpec
from torchtune_b200.parallel.tp import TensorParallelContext
from torchtune_b200.parallel.tp_model import tensor_parallelize

ARCH = dict(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48, norm_eps=1e-5, rope_base=10000)
LR, CLIP, STEPS = 1e-2, 0.5, 3


def _batch(replica: int, step: int):
    g = torch.Generator().manual_seed(100 * replica + step)
    tokens = torch.randint(0, 64, (2, 8), generator=g)
    labels = torch.randint(0, 64, (2, 8), generator=g)
    return tokens, labels


def _single_process():
    model = llama3_1(**ARCH)
    fixed_init_(model, std=0.1)
    opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=0.01)
    norms = []
    for step in range(STEPS):
        loss = 0.0
        for replica in range(2):
            tokens, labels = _batch(replica, step)
            loss = loss + F.cross_entropy(model(tokens).reshape(-1, 64), labels.reshape(-1), reduction="sum")
        (loss / 32).backward()
        norms.append(float(torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)))
        opt.step()
        opt.zero_grad()
    return {k: v.clone() for k, v in model.state_dict().items()}, norms


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
        dp_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
        tp_group, dp_group, replica = tp_groups[rank // 2], dp_groups[rank % 2], rank // 2
        model = llama3_1(**ARCH)
        fixed_init_(model, std=0.1)
        tp = TensorParallelContext(torch.device("cpu"), tp_group, max_rows_per_rank=8, max_width=48)
        tpm = tensor_parallelize(model, tp)
        replicated = {id(p) for p in tpm._replicated}
        named = list(tpm.named_parameters())
        specs = [StoreSpec("replicated", [(n, p) for n, p in named if id(p) in replicated], None),
                 StoreSpec("local", [(n, p) for n, p in named if id(p) not in replicated], dp_group)]
        opt = MultiStoreAdamW(torch.device("cpu"), specs, lr=LR, weight_decay=0.01, shard_group=tp_group)
        norms = []
        for step in range(STEPS):
            tokens, labels = _batch(replica, step)
            logits = tpm(tokens)
            loss = F.cross_entropy(logits.reshape(-1, 64), tpm.shard_rows(labels).reshape(-1), reduction="sum")
            loss.backward()
            opt.collect_grads()
            opt.step(grad_scale=1.0 / 32, max_grad_norm=CLIP)
            opt.zero_grad()
            norms.append(float(opt.last_grad_norm))
            if step == 1:  # checkpoint round trip in mid-training: wipe the moments, restore them from the gathered form
                saved = opt.full_state_dict(True)
                for o in opt.opts:
                    o.exp_avg.zero_()
                    o.exp_avg_sq.zero_()
                opt.load_full_state_dict(saved)
        results[rank] = dict(norms=norms, sd={k: v.clone() for k, v in tpm.full_state_dict().items()})
    finally:
        dist.destroy_process_group()


def test_multi_store_adamw_on_a_2x2_mesh_matches_single_process():
    want_sd, want_norms = _single_process()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(4, 29611, results), nprocs=4, join=True)
    for rank in range(4):
        got = results[rank]
        torch.testing.assert_close(torch.tensor(got["norms"]), torch.tensor(want_norms), rtol=1e-4, atol=1e-5)
        for k, v in want_sd.items():
            torch.testing.assert_close(got["sd"][k], v, rtol=2e-4, atol=2e-5, msg=lambda m, k=k: f"{k}: {m}")

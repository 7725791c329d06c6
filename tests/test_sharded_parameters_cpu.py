"""Sharded linear weights (ZeRO-3 for the GEMM weights) on CPU (gloo, 2 ranks): every rank trains on its own batch with half of
every linear weight's rows; loss, shard gradients (after the reduce-scatter), replicated gradients (after the sum) and the
re-assembled checkpoint must equal one process that sees both batches."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from helpers import fixed_init_
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.parallel.fsdp import ShardedLinear, shard_linear_weights

ARCH = dict(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48, norm_eps=1e-5, rope_base=10000)


def _data(rank):
    g = torch.Generator().manual_seed(70 + rank)
    return torch.randint(0, 64, (2, 8), generator=g), torch.randint(0, 64, (2, 8), generator=g)


def _loss(model, tokens, labels):
    return F.cross_entropy(model(tokens).reshape(-1, 64).float(), labels.reshape(-1), reduction="sum")


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = llama3_1(**ARCH)
        fixed_init_(model, std=0.1)
        shard_linear_weights(model, torch.device("cpu"), min_numel=1)
        assert isinstance(model.layers[0].attn.q_proj, ShardedLinear) and model.layers[0].attn.q_proj.weight.shape == (16, 32)
        loss = _loss(model, *_data(rank))
        loss.backward()
        model.sync_replicated_grads()
        total = loss.detach().clone()
        dist.all_reduce(total)
        l0 = model.layers[0]
        results[rank] = dict(loss=total.item(), q=l0.attn.q_proj.weight.grad.clone(), w2=l0.mlp.w2.weight.grad.clone(), norm=l0.sa_norm.scale.grad.clone(),
                             emb=model.tok_embeddings.weight.grad.clone(), sd={k: v.clone() for k, v in model.full_state_dict().items()})
    finally:
        dist.destroy_process_group()


def test_sharded_linear_weights_match_single_process():
    world = 2
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29591, results), nprocs=world, join=True)
    model = llama3_1(**ARCH)
    fixed_init_(model, std=0.1)
    loss = sum(_loss(model, *_data(r)) for r in range(world))
    loss.backward()
    grads = {k: p.grad for k, p in model.named_parameters()}
    sd = model.state_dict()
    for rank in range(world):
        r = results[rank]
        assert abs(r["loss"] - loss.item()) < 1e-4 * abs(loss.item())
        torch.testing.assert_close(r["q"], grads["layers.0.attn.q_proj.weight"][rank * 16 : (rank + 1) * 16], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["w2"], grads["layers.0.mlp.w2.weight"][rank * 16 : (rank + 1) * 16], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["norm"], grads["layers.0.sa_norm.scale"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["emb"], grads["tok_embeddings.weight"], rtol=1e-4, atol=1e-5)
        assert set(r["sd"]) == set(sd)
        for k in sd:
            assert torch.equal(r["sd"][k], sd[k]), k

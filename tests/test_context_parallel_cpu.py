"""Context parallelism on CPU (gloo): sequence-sharded decoder with the head/sequence exchange around attention must give
the loss and the (summed) gradients of one process that sees whole sequences — with a packed-document mask and with
fewer K/V heads than ranks."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from helpers import fixed_init_
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.ops.mask import AttentionMask
from torchtune_b200.parallel.cp import ContextParallelContext, context_parallelize


def _arch(kv_heads):
    return dict(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=kv_heads, embed_dim=32, max_seq_len=32, intermediate_dim=48, norm_eps=1e-5, rope_base=10000)


def _batch():
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, 64, (2, 16), generator=g)
    labels = torch.randint(0, 64, (2, 16), generator=g)
    labels[1, 3:6] = -100
    mask = AttentionMask.from_seq_lens([[5, 11], [9, 7]])
    pos = torch.tensor([list(range(5)) + list(range(11)), list(range(9)) + list(range(7))])
    return dict(tokens=tokens, labels=labels, mask=mask, input_pos=pos)


def _run(model, batch):
    labels = batch.pop("labels")
    logits = model(**batch)
    loss = F.cross_entropy(logits.reshape(-1, 64).float(), labels.reshape(-1), ignore_index=-100, reduction="sum")
    loss.backward()
    return loss


def _worker(rank, world, port, kv_heads, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = llama3_1(**_arch(kv_heads))
        fixed_init_(model, std=0.1)
        cp = ContextParallelContext()
        context_parallelize(model, cp)
        batch = cp.shard_batch(_batch())
        assert batch["tokens"].shape == (2, 16 // world)
        loss = _run(model, batch).detach()
        dist.all_reduce(loss)
        grads = {}
        for k, p in model.named_parameters():
            g = p.grad.clone()
            dist.all_reduce(g)
            grads[k] = g
        results[rank] = dict(loss=loss.item(), grads=grads)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,kv_heads,port", [(2, 2, 29581), (4, 2, 29583)])
def test_context_parallel_decoder_matches_single_process(world, kv_heads, port):
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, kv_heads, results), nprocs=world, join=True)
    model = llama3_1(**_arch(kv_heads))
    fixed_init_(model, std=0.1)
    ref_loss = _run(model, _batch()).item()
    for rank in range(world):
        r = results[rank]
        assert abs(r["loss"] - ref_loss) < 1e-4 * abs(ref_loss)
        for k, p in model.named_parameters():
            torch.testing.assert_close(r["grads"][k], p.grad, rtol=1e-4, atol=1e-5, msg=k)

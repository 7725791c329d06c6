"""Worker for ``test_gpu_multi.py``: tensor-parallel tiny Llama on 2 GPUs (fused all-gather→GEMM and
GEMM→reduce-scatter kernels over peer memory) against the same model run unsharded on each rank."""
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from helpers import fixed_init_
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.ops._lib import check_device_errors
from torchtune_b200.parallel.tp import TensorParallelContext
from torchtune_b200.parallel.tp_model import tensor_parallelize

ARCH = dict(vocab_size=512, num_layers=2, num_heads=8, num_kv_heads=4, embed_dim=256, max_seq_len=256, intermediate_dim=512, norm_eps=1e-5, rope_base=10000)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, 512, (2, 128), generator=g).to(dev)
    labels = torch.randint(0, 512, (2, 128), generator=g).to(dev)

    ref = llama3_1(**ARCH)
    fixed_init_(ref, std=0.05)
    ref = ref.to(dev).bfloat16()
    ref_loss = F.cross_entropy(ref(tokens).float().reshape(-1, 512), labels.reshape(-1), reduction="sum")
    ref_loss.backward()

    model = llama3_1(**ARCH)
    fixed_init_(model, std=0.05)
    model = model.to(dev).bfloat16()
    tp = TensorParallelContext(dev, max_rows_per_rank=2 * 128 // world, max_width=512)
    tpm = tensor_parallelize(model, tp)
    for step in range(2):  # twice: exercises the double-buffered shard / staging buffers
        tpm.zero_grad()
        logits = tpm(tokens)
        loss = F.cross_entropy(logits.float().reshape(-1, 512), tpm.shard_rows(labels).reshape(-1), reduction="sum")
        loss.backward()
        tpm.sync_replicated_grads()
    total = loss.detach().clone()
    dist.all_reduce(total)
    torch.cuda.synchronize()
    check_device_errors()
    rel = abs(total.item() - ref_loss.item()) / abs(ref_loss.item())
    assert rel < 2e-2, (total.item(), ref_loss.item())
    per = 512 // world
    want = torch.cat([ref.layers[0].mlp.w1.weight.grad[rank * per : (rank + 1) * per], ref.layers[0].mlp.w3.weight.grad[rank * per : (rank + 1) * per]]).float()
    got = tpm.layers[0].mlp.w13.grad.float()
    err = (got - want).norm() / want.norm()
    assert err < 5e-2, err.item()
    emb_err = (tpm.tok_embeddings.weight.grad.float() - ref.tok_embeddings.weight.grad.float()).norm() / ref.tok_embeddings.weight.grad.float().norm()
    assert emb_err < 5e-2, emb_err.item()
    sd = tpm.full_state_dict()
    assert sd["layers.1.attn.q_proj.weight"].shape == (256, 256) and sd["layers.1.mlp.w2.weight"].shape == (256, 512)
    tp.close()
    dist.barrier()
    if rank == 0:
        print("TP_OK", total.item(), ref_loss.item(), err.item())
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

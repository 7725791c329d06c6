"""Worker for the 2-GPU sharded-parameter check: a bf16 decoder whose large linear weights are split over the ranks (fused weight
all-gather → GEMM in forward) against an fp32 single-device evaluation on both ranks' batches."""
import copy
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()

    from helpers import fixed_init_
    from torchtune_b200 import ops
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.ops._lib import check_device_errors
    from torchtune_b200.parallel.fsdp import ShardedLinear, shard_linear_weights

    arch = dict(vocab_size=512, num_layers=2, num_heads=4, num_kv_heads=4, embed_dim=512, max_seq_len=256, intermediate_dim=1024, norm_eps=1e-5, rope_base=10000)
    full = llama3_1(**arch)
    fixed_init_(full, std=0.05)
    full = full.to(dev)
    with torch.no_grad():
        for p in full.parameters():
            p.copy_(p.bfloat16().float())
    batches = [(torch.randint(0, 512, (2, 128), generator=torch.Generator().manual_seed(5 + r)), torch.randint(0, 512, (2, 128), generator=torch.Generator().manual_seed(9 + r))) for r in range(world)]

    with ops.use_reference_ops():
        ref_loss = sum(F.cross_entropy(full(t.to(dev)).reshape(-1, 512).float(), l.to(dev).reshape(-1), reduction="sum") for t, l in batches)
        ref_loss.backward()
    ref_grads = {k: p.grad for k, p in full.named_parameters()}

    model = copy.deepcopy(full).bfloat16()
    for p in model.parameters():
        p.grad = None
    shard_linear_weights(model, dev)
    n_sharded = sum(isinstance(m, ShardedLinear) for m in model.modules())
    assert n_sharded >= 10, n_sharded
    tokens, labels = batches[rank]
    for _ in range(2):
        for p in model.parameters():
            p.grad = None
        loss = F.cross_entropy(model(tokens.to(dev)).reshape(-1, 512).float(), labels.to(dev).reshape(-1), reduction="sum")
        loss.backward()
    model.sync_replicated_grads()
    total = loss.detach().clone()
    dist.all_reduce(total)
    torch.cuda.synchronize()
    check_device_errors()

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9))

    assert abs(total.item() - ref_loss.item()) < 2e-2 * abs(ref_loss.item()), (total.item(), ref_loss.item())
    q = model.layers[0].attn.q_proj
    rows = q.weight.shape[0]
    e_q = rel(q.weight.grad, ref_grads["layers.0.attn.q_proj.weight"][rank * rows : (rank + 1) * rows])
    w2 = model.layers[1].mlp.w2
    r2 = w2.weight.shape[0]
    e_w2 = rel(w2.weight.grad, ref_grads["layers.1.mlp.w2.weight"][rank * r2 : (rank + 1) * r2])
    e_norm = rel(model.layers[0].sa_norm.scale.grad, ref_grads["layers.0.sa_norm.scale"])
    assert e_q < 6e-2 and e_w2 < 6e-2 and e_norm < 6e-2, (e_q, e_w2, e_norm)
    sd = model.full_state_dict()
    assert torch.equal(sd["layers.0.attn.q_proj.weight"].float(), full.state_dict()["layers.0.attn.q_proj.weight"])
    model._sw.close()
    dist.barrier()
    if rank == 0:
        print("ZERO3_OK", e_q, e_w2, e_norm)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""A frozen 4-bit base cut over two ranks (gloo): each rank keeps half of every weight's codes and block scales, gathers and expands
them per use; loss, adapter gradients and the re-assembled checkpoint must equal one process that holds the whole base — also when
the model is built without storage first and filled from a checkpoint afterwards (the path a base larger than one GPU takes)."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from torchtune_b200.models.llama3_1 import lora_llama3_1
from torchtune_b200.modules.low_precision import NF4Weight, ShardedNF4Weight
from torchtune_b200.parallel.fsdp import shard_linear_weights, shard_nf4_bases

ARCH = dict(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=256, max_seq_len=32, intermediate_dim=256, norm_eps=1e-5, rope_base=10000)
LORA = dict(lora_attn_modules=["q_proj", "v_proj"], apply_lora_to_mlp=True, lora_rank=4, lora_alpha=8.0, quantize_base=True)


def _model():
    torch.manual_seed(11)
    model = lora_llama3_1(**LORA, **ARCH)
    with torch.no_grad():  # lora_b starts at zero; give the adapters something to do
        for name, p in model.named_parameters():
            if "lora_b" in name:
                p.normal_(0.0, 0.05)
    return model


def _data(rank):
    g = torch.Generator().manual_seed(170 + rank)
    return torch.randint(0, 64, (2, 8), generator=g), torch.randint(0, 64, (2, 8), generator=g)


def _loss(model, tokens, labels):
    return F.cross_entropy(model(tokens).reshape(-1, 64).float(), labels.reshape(-1), reduction="sum")


def _worker(rank, world, port, results, checkpoint):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = _model()
        for p in model.parameters():
            p.requires_grad_("lora" in [n for n, q in model.named_parameters() if q is p][0])
        whole_bytes = sum(m.nbytes() for m in model.modules() if isinstance(m, NF4Weight))
        shard_linear_weights(model, torch.device("cpu"), min_numel=1)
        l0 = model.layers[0]
        kinds = {name: type(getattr(mod, "nf4", None)).__name__ for name, mod in (("q", l0.attn.q_proj), ("k", l0.attn.k_proj), ("w1", l0.mlp.w1))}
        part_bytes = sum(m.nbytes() for m in model.modules() if isinstance(m, (NF4Weight, ShardedNF4Weight)))
        loss = _loss(model, *_data(rank))
        loss.backward()
        model.sync_replicated_grads()
        total = loss.detach().clone()
        dist.all_reduce(total)
        out = dict(loss=total.item(), kinds=kinds, whole=whole_bytes, part=part_bytes, qa=l0.attn.q_proj.lora_a.weight.grad.clone(), w2b=l0.mlp.w2.lora_b.weight.grad.clone(),
                   sd={k: v.clone() for k, v in model.full_state_dict().items()})

        # the same model without storage first: parts are allocated directly, values come from the checkpoint
        with torch.device("meta"):
            late = lora_llama3_1(**LORA, **ARCH)
        cut = shard_nf4_bases(late, torch.device("cpu"), min_numel=1)
        from torchtune_b200.training._distributed import materialize

        materialize(late, torch.device("cpu"))
        missing, unexpected = late.load_state_dict(checkpoint, strict=False)
        out["late_cut"], out["late_unexpected"] = cut, list(unexpected)
        out["late_missing_non_lora"] = [k for k in missing if "lora" not in k]
        out["late_w1"] = late.layers[1].mlp.w1.nf4.dequantize().clone()
        out["late_part_numel"] = late.layers[1].mlp.w1.nf4.weight_nf4.numel()
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_sharded_nf4_base_matches_single_process():
    world = 2
    model = _model()
    for name, p in model.named_parameters():
        p.requires_grad_("lora" in name)
    checkpoint = {k: v.clone() for k, v in model.state_dict().items() if "lora" not in k}
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29641, results, checkpoint), nprocs=world, join=True)
    loss = sum(_loss(model, *_data(r)) for r in range(world))
    loss.backward()
    grads = {k: p.grad for k, p in model.named_parameters() if p.grad is not None}
    sd = model.state_dict()
    for rank in range(world):
        r = results[rank]
        # k_proj (128 x 256 = two scale groups... one per rank) and the others all split; every base is now a part
        assert r["kinds"] == {"q": "ShardedNF4Weight", "k": "ShardedNF4Weight", "w1": "ShardedNF4Weight"}
        assert r["part"] * 2 <= r["whole"] + 64  # half of the codes and scales (+ the replicated scalar means)
        assert abs(r["loss"] - loss.item()) < 1e-5 * abs(loss.item())
        torch.testing.assert_close(r["qa"], grads["layers.0.attn.q_proj.lora_a.weight"], rtol=1e-4, atol=1e-6)
        torch.testing.assert_close(r["w2b"], grads["layers.0.mlp.w2.lora_b.weight"], rtol=1e-4, atol=1e-6)
        assert set(r["sd"]) == set(sd)
        for k in sd:
            assert torch.equal(r["sd"][k], sd[k]), k
        assert r["late_cut"] == 14 and not r["late_unexpected"] and not r["late_missing_non_lora"]
        recoded = NF4Weight(256, 256, dtype=torch.float32)
        recoded.quantize_(checkpoint["layers.1.mlp.w1.weight"])  # what one process makes of the same checkpoint tensor
        assert torch.equal(r["late_w1"], recoded.dequantize(r["late_w1"].dtype))
        assert r["late_part_numel"] == 256 * 256 // 2 // world


def test_weights_that_do_not_split_at_scale_group_boundaries_stay_whole():
    assert ShardedNF4Weight.divisible(128, 256, 2) and not ShardedNF4Weight.divisible(128, 128, 2) and not ShardedNF4Weight.divisible(128, 256, 3)
    full = NF4Weight(128, 256)
    torch.manual_seed(0)
    dense = torch.randn(128, 256, dtype=torch.bfloat16)
    full.quantize_(dense)
    parts = [ShardedNF4Weight.from_full(full, rank=r, world=2) for r in range(2)]
    assert torch.equal(torch.cat([p.weight_nf4 for p in parts]), full.weight_nf4)
    assert torch.equal(torch.cat([p.scaler_q for p in parts]), full.scaler_q)
    assert torch.equal(torch.cat([p.scaler_factor for p in parts]), full.scaler_factor)
    again = ShardedNF4Weight(128, 256, rank=1, world=2)
    again.quantize_(dense)  # coding the whole weight and keeping a part gives the same part
    assert torch.equal(again.weight_nf4, parts[1].weight_nf4) and torch.equal(again.scaler_q, parts[1].scaler_q)

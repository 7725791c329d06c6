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


def test_fusion_model_built_without_storage_is_sharded_from_the_checkpoint():
    """Llama-3.2-Vision-shaped model on the meta device: every linear weight goes from the checkpoint straight into a shard (fusion
    layers keep the ``layer.`` level out of their state-dict keys, which the sharding has to look through), the rest is given
    storage and loaded afterwards, and the result computes what the ordinary model computes."""
    from torchtune_b200.models.llama3_2_vision import llama3_2_vision_decoder, llama3_2_vision_encoder
    from torchtune_b200.modules.model_fusion import DeepFusionModel
    from torchtune_b200.training._distributed import materialize

    def build():
        enc = llama3_2_vision_encoder(patch_size=4, num_heads=4, clip_embed_dim=32, clip_num_layers=2, clip_hidden_states=[1], num_layers_projection=1, decoder_embed_dim=64, tile_size=16,
                                      max_num_tiles=4, in_channels=3)
        dec = llama3_2_vision_decoder(vocab_size=128, num_layers=4, fusion_interval=2, num_special_tokens=8, num_heads=4, num_kv_heads=2, embed_dim=64, max_seq_len=64, encoder_max_seq_len=68,
                                      rope_base=500000, intermediate_dim=96)
        return DeepFusionModel(encoder=enc, decoder=dec)

    torch.manual_seed(0)
    whole = build().eval()
    with torch.no_grad():
        for name, p in whole.named_parameters():
            if p.numel() == 1:
                p.fill_(0.7)  # open the gates
    state = {k: v.clone() for k, v in whole.state_dict().items()}

    with torch.device("meta"):
        late = build()
    late = shard_linear_weights(late, torch.device("cpu"), min_numel=1, state_dict=state)
    fused_layer = late.decoder.layers[1]
    assert isinstance(fused_layer.layer.attn.q_proj, ShardedLinear) and isinstance(fused_layer.fusion_layer.attn.q_proj, ShardedLinear)
    assert "decoder.layers.1.attn.q_proj.weight" in late._sharded_keys  # found under the key without `layer.`
    rest = {k: v for k, v in state.items() if k not in late._sharded_keys}
    materialize(late, torch.device("cpu"))
    missing, unexpected = late.load_state_dict(rest, strict=False)
    assert not unexpected and set(missing) <= late._sharded_keys, (missing, unexpected)
    late.refresh_replicated()
    assert not any(p.is_meta for p in late.parameters())

    tokens = torch.randint(0, 128, (2, 9))
    images = torch.randn(2, 1, 4, 3, 16, 16)
    kwargs = dict(encoder_input={"images": images, "aspect_ratio": torch.tensor([[[2, 2]], [[2, 2]]])}, encoder_mask=torch.ones(2, 9, 68, dtype=torch.bool))
    with torch.no_grad():
        torch.testing.assert_close(late.eval()(tokens, **kwargs), whole(tokens, **kwargs), rtol=1e-5, atol=1e-5)

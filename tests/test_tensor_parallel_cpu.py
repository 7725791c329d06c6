"""Tensor-parallel decoder on CPU (gloo, 2 ranks): token-sharded loss, parameter gradients and the
re-assembled checkpoint must equal the single-process model."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from helpers import fixed_init_
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.parallel.tp import TensorParallelContext
from torchtune_b200.parallel.tp_model import tensor_parallelize

ARCH = dict(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48, norm_eps=1e-5, rope_base=10000)


def _data():
    g = torch.Generator().manual_seed(7)
    tokens = torch.randint(0, 64, (2, 8), generator=g)
    labels = torch.randint(0, 64, (2, 8), generator=g)
    labels[0, :2] = -100
    return tokens, labels


def _reference():
    model = llama3_1(**ARCH)
    fixed_init_(model, std=0.1)
    tokens, labels = _data()
    loss = F.cross_entropy(model(tokens).reshape(-1, 64), labels.reshape(-1), ignore_index=-100, reduction="sum")
    loss.backward()
    return loss.item(), {k: p.grad.clone() for k, p in model.named_parameters()}, {k: v.clone() for k, v in model.state_dict().items()}


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = llama3_1(**ARCH)
        fixed_init_(model, std=0.1)
        tp = TensorParallelContext(torch.device("cpu"), max_rows_per_rank=8, max_width=48)
        tpm = tensor_parallelize(model, tp)
        tokens, labels = _data()
        logits = tpm(tokens)  # [1, rows, vocab] for this rank's rows
        my_labels = tpm.shard_rows(labels)
        loss = F.cross_entropy(logits.reshape(-1, 64), my_labels.reshape(-1), ignore_index=-100, reduction="sum")
        loss.backward()
        tpm.sync_replicated_grads()
        total = loss.detach().clone()
        dist.all_reduce(total)
        # inference path: replicated activations + per-rank KV cache must reproduce the unsharded logits
        full = llama3_1(**ARCH)
        fixed_init_(full, std=0.1)
        with torch.no_grad():
            want = full(tokens)
            got = tpm.forward_inference(tokens)
            tpm.setup_caches(batch_size=2, dtype=torch.float32, decoder_max_seq_len=8)
            causal = torch.tril(torch.ones(8, 8, dtype=torch.bool))
            pos = torch.arange(8)
            steps = [tpm.forward_inference(tokens[:, :5], mask=causal[None, :5].expand(2, -1, -1), input_pos=pos[None, :5].expand(2, -1))]
            for t in range(5, 8):
                steps.append(tpm.forward_inference(tokens[:, t : t + 1], mask=causal[None, t : t + 1].expand(2, -1, -1), input_pos=pos[None, t : t + 1].expand(2, -1)))
            cached = torch.cat(steps, dim=1)
        infer_err = (got - want).abs().max().item()
        cache_err = (cached - want).abs().max().item()
        l0 = tpm.layers[0]
        results[rank] = dict(
            infer_err=infer_err, cache_err=cache_err,
            loss=total.item(),
            wqkv_grad=l0.attn.wqkv.grad.clone(), wo_grad=l0.attn.wo.grad.clone(), w13_grad=l0.mlp.w13.grad.clone(), w2_grad=l0.mlp.w2.grad.clone(),
            emb_grad=tpm.tok_embeddings.weight.grad.clone(), norm_grad=l0.sa_norm.scale.grad.clone(), out_grad=tpm.output.weight.grad.clone(),
            sd={k: v.clone() for k, v in tpm.full_state_dict().items()},
        )
    finally:
        dist.destroy_process_group()


def test_tp_decoder_matches_single_process():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, 29561, results), nprocs=world, join=True)
    ref_loss, ref_grads, ref_sd = _reference()
    hd, heads, kv = 8, 2, 1  # per rank
    for rank in range(world):
        r = results[rank]
        assert abs(r["loss"] - ref_loss) < 1e-3 * abs(ref_loss)
        assert r["infer_err"] < 1e-4 and r["cache_err"] < 1e-4
        q = ref_grads["layers.0.attn.q_proj.weight"][rank * heads * hd : (rank + 1) * heads * hd]
        k = ref_grads["layers.0.attn.k_proj.weight"][rank * kv * hd : (rank + 1) * kv * hd]
        v = ref_grads["layers.0.attn.v_proj.weight"][rank * kv * hd : (rank + 1) * kv * hd]
        torch.testing.assert_close(r["wqkv_grad"], torch.cat([q, k, v]), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["wo_grad"], ref_grads["layers.0.attn.output_proj.weight"][:, rank * 16 : (rank + 1) * 16], rtol=1e-4, atol=1e-5)
        w1 = ref_grads["layers.0.mlp.w1.weight"][rank * 24 : (rank + 1) * 24]
        w3 = ref_grads["layers.0.mlp.w3.weight"][rank * 24 : (rank + 1) * 24]
        torch.testing.assert_close(r["w13_grad"], torch.cat([w1, w3]), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["w2_grad"], ref_grads["layers.0.mlp.w2.weight"][:, rank * 24 : (rank + 1) * 24], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["emb_grad"], ref_grads["tok_embeddings.weight"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["norm_grad"], ref_grads["layers.0.sa_norm.scale"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["out_grad"], ref_grads["output.weight"], rtol=1e-4, atol=1e-5)
        assert set(r["sd"]) == set(ref_sd)
        for key in ref_sd:
            assert torch.equal(r["sd"][key], ref_sd[key]), key


# ----------------------------------------------------------------------------- mixture of experts under tensor parallelism
MOE_ARCH = dict(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, hidden_dim=48, max_seq_len=32, num_experts=4, experts_per_token=2, rope_base=10000)


def _moe_model():
    from torchtune_b200.models.llama4 import llama4_decoder

    model = llama4_decoder(**MOE_ARCH)
    fixed_init_(model, std=0.1)
    return model


def _moe_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = TensorParallelContext(torch.device("cpu"), max_rows_per_rank=8, max_width=48)
        tpm = tensor_parallelize(_moe_model(), tp)
        tokens, labels = _data()
        logits = tpm(tokens)
        loss = F.cross_entropy(logits.reshape(-1, 64), tpm.shard_rows(labels).reshape(-1), ignore_index=-100, reduction="sum")
        loss.backward()
        tpm.sync_replicated_grads()
        total = loss.detach().clone()
        dist.all_reduce(total)
        with torch.no_grad():
            infer = tpm.forward_inference(tokens)
        mlp = tpm.layers[0].mlp
        results[rank] = dict(
            loss=total.item(), infer=infer, gate=mlp.experts.gate_proj.grad.clone(), down=mlp.experts.down_proj.grad.clone(), router=mlp.router.gate.weight.grad.clone(),
            shared_w2=mlp.shared_expert.w2.grad.clone(), sd={k: v.clone() for k, v in tpm.full_state_dict().items()},
        )
    finally:
        dist.destroy_process_group()


def test_tp_moe_decoder_matches_single_process():
    world = 2
    results = mp.Manager().dict()
    mp.spawn(_moe_worker, args=(world, 29563, results), nprocs=world, join=True)
    model = _moe_model()
    tokens, labels = _data()
    logits = model(tokens)
    loss = F.cross_entropy(logits.reshape(-1, 64), labels.reshape(-1), ignore_index=-100, reduction="sum")
    loss.backward()
    grads = {k: p.grad for k, p in model.named_parameters()}
    sd = model.state_dict()
    per = 48 // world
    for rank in range(world):
        r = results[rank]
        assert abs(r["loss"] - loss.item()) < 1e-3 * abs(loss.item())
        torch.testing.assert_close(r["infer"], logits.detach().float(), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(r["gate"], grads["layers.0.mlp.experts.gate_proj"][:, :, rank * per : (rank + 1) * per], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["down"], grads["layers.0.mlp.experts.down_proj"][:, rank * per : (rank + 1) * per], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["router"], grads["layers.0.mlp.router.gate.weight"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(r["shared_w2"], grads["layers.0.mlp.shared_expert.w2.weight"][:, rank * per : (rank + 1) * per], rtol=1e-4, atol=1e-5)
        assert set(r["sd"]) == set(sd), set(r["sd"]) ^ set(sd)
        for key in sd:
            assert torch.equal(r["sd"][key], sd[key]), key


# ----------------------------------------------------------------------------- fp8 training under tensor parallelism
def _fp8_model():
    from torchtune_b200.training.quantization import convert_to_float8_training

    model = llama3_1(**ARCH)
    fixed_init_(model, std=0.1)
    return convert_to_float8_training(model, "tensorwise")


def _fp8_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = TensorParallelContext(torch.device("cpu"), max_rows_per_rank=8, max_width=48)
        tpm = tensor_parallelize(_fp8_model(), tp)
        assert all(layer.attn.fp8 and layer.mlp.fp8 for layer in tpm.layers)
        tokens, labels = _data()
        loss = F.cross_entropy(tpm(tokens).reshape(-1, 64), tpm.shard_rows(labels).reshape(-1), ignore_index=-100, reduction="sum")
        loss.backward()
        tpm.sync_replicated_grads()
        total = loss.detach().clone()
        dist.all_reduce(total)
        l0 = tpm.layers[0]
        results[rank] = dict(loss=total.item(), w13_grad=l0.mlp.w13.grad.clone(), wo_grad=l0.attn.wo.grad.clone(), emb_grad=tpm.tok_embeddings.weight.grad.clone())
    finally:
        dist.destroy_process_group()


def test_tp_fp8_decoder_tracks_single_process_fp8():
    """Float8 linears under tensor parallelism: every rank scales its own weight shard, so the numbers differ from the
    single-process fp8 model only by quantisation noise; a rowwise recipe is refused."""
    import pytest

    world = 2
    results = mp.Manager().dict()
    mp.spawn(_fp8_worker, args=(world, 29563, results), nprocs=world, join=True)
    model = _fp8_model()
    tokens, labels = _data()
    loss = F.cross_entropy(model(tokens).reshape(-1, 64), labels.reshape(-1), ignore_index=-100, reduction="sum")
    loss.backward()
    grads = {k: p.grad for k, p in model.named_parameters()}
    cos = lambda a, b: F.cosine_similarity(a.reshape(1, -1), b.reshape(1, -1)).item()
    for rank in range(world):
        r = results[rank]
        assert abs(r["loss"] - loss.item()) < 2e-2 * abs(loss.item())
        w1 = grads["layers.0.mlp.w1.weight"][rank * 24 : (rank + 1) * 24]
        w3 = grads["layers.0.mlp.w3.weight"][rank * 24 : (rank + 1) * 24]
        assert cos(r["w13_grad"], torch.cat([w1, w3])) > 0.98
        assert cos(r["wo_grad"], grads["layers.0.attn.output_proj.weight"][:, rank * 16 : (rank + 1) * 16]) > 0.98
        assert cos(r["emb_grad"], grads["tok_embeddings.weight"]) > 0.98

    from torchtune_b200.training.quantization import convert_to_float8_training

    rowwise = convert_to_float8_training(llama3_1(**ARCH), "rowwise")
    with pytest.raises(ValueError, match="tensorwise"):
        tensor_parallelize(rowwise, TensorParallelContext(torch.device("cpu"), max_rows_per_rank=8, max_width=48))


# ----------------------------------------------------------------------------- tensor-parallel generation of an early-fusion model
def _fusion_reference():
    from helpers import tiny_early_fusion_llama4

    torch.manual_seed(5)
    model = tiny_early_fusion_llama4()
    fixed_init_(model, std=0.1)
    return model.eval()


def _fusion_inputs():
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, 64, (2, 12), generator=g)
    tokens[0, 2:6] = 70
    tokens[1, 4:8] = 70
    return tokens, torch.randn(2, 3, 16, 16, generator=g)


def _fusion_worker(rank, world, port, results, state_dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torchtune_b200.config import OmegaConf
        from torchtune_b200.engine.inference import SingleTurnGenerator

        gen = SingleTurnGenerator.__new__(SingleTurnGenerator)  # the part of the generator that builds the model, without a recipe around it
        gen._device, gen._dtype, gen._tp = torch.device("cpu"), torch.float32, None
        model = gen._build_tensor_parallel(OmegaConf.create({"model": {"_component_": "helpers.tiny_early_fusion_llama4"}}), state_dict)
        tokens, images = _fusion_inputs()
        with torch.no_grad():
            logits = model(tokens, encoder_input={"vision": {"images": images}})
        local = model.decoder.tp_decoder.layers[0].mlp.experts.gate_proj
        results[rank] = dict(logits=logits, expert_cols=local.shape[-1], meta_left=[n for n, p in model.named_parameters() if p.is_meta])
    finally:
        dist.destroy_process_group()


def test_tp_generation_model_of_an_early_fusion_model_is_built_layer_by_layer():
    world = 2
    reference = _fusion_reference()
    state = {k: v.clone() for k, v in reference.state_dict().items()}
    results = mp.Manager().dict()
    mp.spawn(_fusion_worker, args=(world, 29651, results, state), nprocs=world, join=True)
    tokens, images = _fusion_inputs()
    with torch.no_grad():
        want = reference(tokens, encoder_input={"vision": {"images": images}})
    for rank in range(world):
        r = results[rank]
        assert not r["meta_left"]
        assert r["expert_cols"] == 48 // world  # the experts' columns are split, the vision tower is whole
        torch.testing.assert_close(r["logits"].float(), want.float(), rtol=1e-4, atol=1e-4)

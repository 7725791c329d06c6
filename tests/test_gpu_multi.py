"""Multi-GPU checks (run as child processes, one per GPU; skipped with fewer than two GPUs)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _torchrun(script: str, nproc: int, port: int, timeout: int = 600):
    # the tiny checkpoints have head dims the attention kernel does not cover (16, 32), so the children may take PyTorch statements
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{ROOT / 'tests'}", MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", TTB_STRICT="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    res = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    return res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_decoder_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_tp_worker.py"), 2, 29571)
    assert "TP_OK" in out


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_ep_worker.py"), 2, 29573)
    assert "EP_OK" in out


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_parameters_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_zero3_worker.py"), 2, 29575)
    assert "ZERO3_OK" in out


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_context_parallel_exchange_over_peer_memory_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_cp_worker.py"), 2, 29577)
    assert "CP_OK" in out


def _tiny_ckpt(tmp_path):
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import write_tiny_hf_checkpoint

    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    return ckpt


def _tune(args, port, timeout=600, nproc=2):
    # the tiny checkpoints have head dims the attention kernel does not cover (16, 32), so the children may take PyTorch statements
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{ROOT / 'tests'}", MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", TTB_STRICT="0")
    cmd = [sys.executable, str(ROOT / "tune"), "run", "--nnodes=1", f"--nproc_per_node={nproc}", "--master-addr=127.0.0.1", f"--master-port={port}"] + args
    res = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


def _losses(path):
    import re

    return [float(m.group(1)) for m in re.finditer(r"loss:([0-9.eE+-]+)", path.read_text())]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("name,port,extra", [("dp", 29581, []), ("tp", 29583, ["tensor_parallel_dim=2"]), ("cp", 29585, ["context_parallel_dim=2"]),
                                             ("z3", 29587, ["shard_parameters=True", "shard_parameters_min_numel=1"])])
def test_distributed_recipe_on_two_gpus(tmp_path, name, port, extra):
    """The distributed full fine-tune recipe end to end in bf16 on two GPUs for every parallel mode; losses must be finite, fall
    within the band of a randomly initialised 1024-token vocabulary and a checkpoint must be written."""
    ckpt = _tiny_ckpt(tmp_path)
    out = tmp_path / name
    _tune(["full_finetune_distributed", "--config", "tiny/llama_full_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
           "device=cuda", "dtype=bf16", "max_steps_per_epoch=4", "dataset.num_samples=32", "optimizer.lr=1e-3"] + extra, port)
    losses = _losses(out / "logs" / "log.txt")
    assert len(losses) == 4 and all(l == l and 4.0 < l < 9.0 for l in losses), losses
    assert (out / "epoch_0" / "model-00001-of-00001.safetensors").exists()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_recipe_on_two_gpus(tmp_path):
    """Tiny Llama-4 style MoE decoder through the distributed recipe with the experts split over two GPUs (peer-memory push / pull,
    grouped GEMMs) against the same run with all experts on both ranks."""
    from torchtune_b200.models.llama4 import llama4_decoder

    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    torch.manual_seed(0)
    model = llama4_decoder(vocab_size=1024, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=128, hidden_dim=256, max_seq_len=256, num_experts=4, experts_per_token=2, rope_base=500000)
    with torch.no_grad():
        for prm in model.parameters():
            prm.copy_(torch.randn_like(prm) * 0.05)
    torch.save(model.state_dict(), ckpt / "model.pt")
    runs = {}
    for name, port, extra in (("dp", 29589, []), ("ep", 29591, ["expert_parallel_dim=2"])):
        out = tmp_path / name
        _tune(["full_finetune_distributed", "--config", "tiny/llama4_moe_full_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
               "device=cuda", "dtype=bf16", "max_steps_per_epoch=4", "dataset.num_samples=32", "optimizer.lr=1e-3"] + extra, port)
        runs[name] = _losses(out / "logs" / "log.txt")
    assert len(runs["ep"]) == 4 and all(l == l for l in runs["ep"])
    # bf16 routing can flip near-ties between the two runs; the curves stay close
    for a, b in zip(runs["ep"], runs["dp"]):
        assert abs(a - b) < 0.05 * abs(b), (runs["ep"], runs["dp"])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fp8_tensor_parallel_recipe_on_two_gpus(tmp_path):
    """enable_fp8_training with tensor_parallel_dim=2: the sharded projections run on the fp8 tensor cores between the row gather
    and the reduce-scatter; losses stay in the band of the bf16 run."""
    ckpt = _tiny_ckpt(tmp_path)
    out = tmp_path / "fp8tp"
    _tune(["full_finetune_distributed", "--config", "tiny/llama_full_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
           "device=cuda", "dtype=bf16", "max_steps_per_epoch=4", "dataset.num_samples=32", "optimizer.lr=1e-3", "tensor_parallel_dim=2", "enable_fp8_training=True"], 29597)
    losses = _losses(out / "logs" / "log.txt")
    assert len(losses) == 4 and all(l == l and 4.0 < l < 9.0 for l in losses), losses


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_lora_over_sharded_base_weights_on_two_gpus(tmp_path):
    """LoRA with shard_parameters=True (frozen base rows split over the GPUs, gathered inside the forward GEMM) follows the loss
    curve of LoRA on the resident data-parallel engine."""
    ckpt = _tiny_ckpt(tmp_path)
    res = {}
    for name, port, extra in (("dp", 29593, []), ("z3", 29595, ["shard_parameters=True", "shard_parameters_min_numel=1"])):
        out = tmp_path / name
        _tune(["lora_finetune_distributed", "--config", "tiny/llama_lora_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
               "device=cuda", "dtype=bf16", "max_steps_per_epoch=4", "dataset.num_samples=32", "optimizer.lr=1e-2"] + extra, port)
        res[name] = _losses(out / "logs" / "log.txt")
    assert len(res["z3"]) == 4
    for a, b in zip(res["dp"], res["z3"]):
        assert abs(a - b) < 0.02 * abs(a), res
    assert (tmp_path / "z3" / "epoch_0" / "adapter_model.safetensors").exists()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_qlora_over_sharded_nf4_base_on_two_gpus(tmp_path):
    """QLoRA with shard_parameters=True (each GPU keeps half of every 4-bit base weight's codes and scales; a weight is gathered and
    expanded right before its GEMM; the model is built without storage first) follows QLoRA with a resident 4-bit base."""
    ckpt = _tiny_ckpt(tmp_path)
    res = {}
    for name, port, extra in (("dp", 29647, []), ("z3", 29649, ["shard_parameters=True", "shard_parameters_min_numel=1"])):
        out = tmp_path / name
        _tune(["lora_finetune_distributed", "--config", "tiny/llama_lora_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
               "device=cuda", "dtype=bf16", "max_steps_per_epoch=4", "dataset.num_samples=32", "optimizer.lr=1e-2", "model.quantize_base=True", "save_adapter_weights_only=True"] + extra, port)
        res[name] = _losses(out / "logs" / "log.txt")
    assert len(res["z3"]) == 4
    for a, b in zip(res["dp"], res["z3"]):
        assert abs(a - b) < 0.02 * abs(a), res
    assert (tmp_path / "z3" / "epoch_0" / "adapter_model.safetensors").exists()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_dp_times_tp_mesh_on_four_gpus(tmp_path):
    """tensor_parallel_dim=2 on four GPUs (two tensor-parallel groups of consecutive ranks, two model replicas) follows the loss
    curve of plain data parallelism on the same global batch."""
    ckpt = _tiny_ckpt(tmp_path)
    res = {}
    for name, port, extra in (("dp", 29601, ["batch_size=2"]), ("mesh", 29603, ["batch_size=4", "tensor_parallel_dim=2"])):
        out = tmp_path / name
        _tune(["full_finetune_distributed", "--config", "tiny/llama_full_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
               "device=cuda", "dtype=bf16", "max_steps_per_epoch=4", "dataset.num_samples=64", "optimizer.lr=1e-3"] + extra, port, nproc=4)
        res[name] = _losses(out / "logs" / "log.txt")
    assert len(res["mesh"]) == 4
    for a, b in zip(res["dp"], res["mesh"]):
        assert abs(a - b) < 0.02 * abs(a), res


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_dp_times_ep_mesh_on_four_gpus(tmp_path):
    """expert_parallel_dim=2 on four GPUs (two expert-parallel groups side by side) follows plain data parallelism."""
    from torchtune_b200.models.llama4 import llama4_decoder

    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    torch.manual_seed(0)
    model = llama4_decoder(vocab_size=1024, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=128, hidden_dim=256, max_seq_len=256, num_experts=4, experts_per_token=2, rope_base=500000)
    with torch.no_grad():
        for prm in model.parameters():
            prm.copy_(torch.randn_like(prm) * 0.05)
    torch.save(model.state_dict(), ckpt / "model.pt")
    res = {}
    for name, port, extra in (("dp", 29605, []), ("mesh", 29607, ["expert_parallel_dim=2"])):
        out = tmp_path / name
        _tune(["full_finetune_distributed", "--config", "tiny/llama4_moe_full_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={out}", "metric_logger.filename=log.txt",
               "device=cuda", "dtype=bf16", "max_steps_per_epoch=3", "dataset.num_samples=32", "optimizer.lr=1e-3"] + extra, port, nproc=4)
        res[name] = _losses(out / "logs" / "log.txt")
    assert len(res["mesh"]) == 3
    for a, b in zip(res["dp"], res["mesh"]):
        assert abs(a - b) < 0.02 * abs(a), res

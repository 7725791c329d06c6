"""QAT: fake-quantised forward equals the converted int4 model; the warm-up switch keeps the
first steps identical to plain fine-tuning; the recipes run end to end."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import TINY, fixed_init_, read_losses, run_tune, write_tiny_hf_checkpoint
from torchtune_b200.models.llama3_1 import llama3_1, lora_llama3_1
from torchtune_b200.modules.peft import QATLoRALinear
from torchtune_b200.training import quantization as Q

ROOT = Path(__file__).resolve().parent.parent


def test_qat_prepare_convert_equivalence_and_packing():
    torch.manual_seed(0)
    model = llama3_1(**TINY)
    fixed_init_(model)
    x = torch.randint(0, 1024, (2, 16))
    ref = model(x)
    quantizer = Q.Int8DynActInt4WeightQATQuantizer(groupsize=64)
    assert Q.get_quantizer_mode(quantizer) == "8da4w-qat"
    model = quantizer.prepare(model)
    fq = model(x)
    assert 0 < (fq - ref).abs().max() < 0.5
    model.apply(Q.disable_fake_quant)
    torch.testing.assert_close(model(x), ref)
    model.apply(Q.enable_fake_quant)
    fq.sum().backward()
    assert all(p.grad is not None for p in model.parameters())
    model = quantizer.convert(model)
    torch.testing.assert_close(model(x), fq, rtol=1e-5, atol=1e-5)
    lin = next(m for m in model.modules() if isinstance(m, Q.Int4WeightLinear))
    assert lin.weight_packed.dtype == torch.uint8 and lin.weight_packed.shape[1] * 2 == lin.in_features


@pytest.mark.parametrize("cls,symmetric", [(Q.Int8DynActInt4WeightQuantizer, True), (Q.Int4WeightOnlyQuantizer, False)])
def test_ptq_int4_roundtrip_error_bound(cls, symmetric):
    torch.manual_seed(1)
    w = torch.randn(32, 128)
    packed, scale, zero = Q._quantize_int4_groupwise(w, 32, symmetric)
    back = Q._dequantize_int4_groupwise(packed, scale, zero, 32, symmetric, torch.float32)
    step = scale.repeat_interleave(32, dim=1)
    assert ((back - w).abs() <= step * (1.0 if symmetric else 0.5) + 1e-6).all()
    model = torch.nn.Sequential()
    model.add_module("proj", __import__("torchtune_b200").modules.Linear(128, 32, bias=False))
    cls(groupsize=32).quantize(model)
    assert isinstance(model.proj, Q.Int4WeightLinear)


def test_swap_lora_linear_with_qat():
    model = lora_llama3_1(["q_proj", "v_proj"], **TINY, lora_rank=4, lora_alpha=8)
    Q.swap_lora_linear_with_qat(model, Q.FakeQuantizeConfig(bits=8, is_symmetric=False), Q.FakeQuantizeConfig(bits=4, group_size=64))
    n = sum(isinstance(m, QATLoRALinear) for m in model.modules())
    assert n == 2 * TINY["num_layers"]
    model(torch.randint(0, 1024, (1, 8))).sum().backward()


def test_qat_single_device_recipe_with_warmup(tmp_path, tune_path, monkeypatch):
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    common = f"checkpointer.checkpoint_dir={ckpt} metric_logger.filename=log.txt max_steps_per_epoch=4"
    run_tune(tune_path, f"run full_finetune_single_device --config tiny/llama_full_single_device {common} output_dir={tmp_path / 'plain'}", monkeypatch)
    run_tune(tune_path, f"run qat_single_device --config tiny/llama_qat_single_device {common} output_dir={tmp_path / 'qat'} fake_quant_after_n_steps=2", monkeypatch)
    plain = read_losses(tmp_path / "plain" / "logs" / "log.txt")
    qat = read_losses(tmp_path / "qat" / "logs" / "log.txt")
    assert len(qat) == 4
    assert qat[:2] == pytest.approx(plain[:2], abs=1e-6)  # fake quant still off
    assert abs(qat[2] - plain[2]) > 1e-6  # switched on at step 2
    assert (tmp_path / "qat" / "epoch_0" / "model-00001-of-00001.safetensors").exists()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("recipe,cfg,port", [("qat_distributed", "tiny/llama_qat_distributed", 29551), ("qat_lora_finetune_distributed", "tiny/llama_qat_lora_distributed", 29552)])
def test_qat_distributed_recipes(tmp_path, recipe, cfg, port):
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    env = dict(os.environ, PYTHONPATH=str(ROOT), MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    args = ["run", "--nnodes=1", "--nproc_per_node=2", "--master-addr=127.0.0.1", f"--master-port={port}", recipe, "--config", cfg,
            f"checkpointer.checkpoint_dir={ckpt}", "metric_logger.filename=log.txt", "max_steps_per_epoch=3", f"output_dir={tmp_path / 'out'}"]
    res = subprocess.run([sys.executable, str(ROOT / "tune")] + args, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=800)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert len(read_losses(tmp_path / "out" / "logs" / "log.txt")) == 3

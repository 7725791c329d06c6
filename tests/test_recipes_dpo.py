"""DPO recipes on CPU: the first logged step must equal the closed-form loss ln 2 (policy ==
reference before any update), later steps separate chosen from rejected; the fused sequence
log-prob path agrees with the materialised-logits path."""
import math
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import TINY, fixed_init_, run_tune, write_tiny_hf_checkpoint
from torchtune_b200 import rlhf
from torchtune_b200.engine.preference import sequence_logprobs
from torchtune_b200.models.llama3_1 import llama3_1

ROOT = Path(__file__).resolve().parent.parent


def _metric(log_file, name):
    return [float(x) for x in re.findall(rf"{re.escape(name)}:(\S+)", Path(log_file).read_text())]


def test_fused_sequence_logprobs_match_logits_path():
    model = llama3_1(**TINY)
    fixed_init_(model)
    tokens = torch.randint(0, 1024, (4, 24))
    labels = tokens.clone()
    labels[:, :7] = -100
    labels[2, 20:] = -100
    got, mean_logit = sequence_logprobs(model, tokens, labels)
    logits = model(tokens)
    want = rlhf.get_batch_log_probs(logits, labels)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(mean_logit, logits.mean(dim=(1, 2)), rtol=1e-3, atol=1e-5)
    assert model.skip_output_layer is False


def test_lora_dpo_single_device(tmp_path, tune_path, monkeypatch):
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    out = tmp_path / "out"
    run_tune(
        tune_path,
        f"run lora_dpo_single_device --config tiny/llama_lora_dpo_single_device checkpointer.checkpoint_dir={ckpt} output_dir={out} "
        "metric_logger.filename=log.txt dataset.num_samples=2 epochs=8 max_steps_per_epoch=1 optimizer.lr=2e-2",
        monkeypatch,
    )
    log = out / "logs" / "log.txt"
    losses = _metric(log, "loss")
    assert len(losses) == 8
    assert losses[0] == pytest.approx(math.log(2.0), abs=1e-5)  # LoRA B = 0 → policy == reference
    assert losses[-1] < losses[0]
    assert _metric(log, "rewards/accuracies")[-1] == 1.0
    assert _metric(log, "rewards/margins")[-1] > 0
    assert (out / "epoch_7" / "adapter_model.safetensors").exists()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("recipe,cfg,port", [("lora_dpo_distributed", "tiny/llama_lora_dpo_distributed", 29541), ("full_dpo_distributed", "tiny/llama_full_dpo_distributed", 29542)])
def test_dpo_distributed_two_ranks(tmp_path, recipe, cfg, port):
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    env = dict(os.environ, PYTHONPATH=str(ROOT), MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    lr = "5e-3" if "lora" in recipe else "1e-4"
    args = ["run", "--nnodes=1", "--nproc_per_node=2", "--master-addr=127.0.0.1", f"--master-port={port}", recipe, "--config", cfg,
            f"checkpointer.checkpoint_dir={ckpt}", "metric_logger.filename=log.txt", "dataset.num_samples=4", "epochs=6", "max_steps_per_epoch=1", f"optimizer.lr={lr}", f"output_dir={tmp_path / 'out'}"]
    res = subprocess.run([sys.executable, str(ROOT / "tune")] + args, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=800)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    log = tmp_path / "out" / "logs" / "log.txt"
    losses = _metric(log, "loss")
    assert len(losses) == 6
    assert losses[0] == pytest.approx(math.log(2.0), abs=1e-5)
    assert min(losses[1:]) < losses[0]

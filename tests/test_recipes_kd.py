"""Knowledge-distillation recipe on CPU: with a teacher equal to the student's base weights and
LoRA B = 0 the first step's losses have closed forms — ``kd_loss`` equals the teacher's mean
token entropy and ``loss = ½·class_loss + ½·kd_loss``."""
import re
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from helpers import TINY, fixed_init_, run_tune, write_tiny_hf_checkpoint
from torchtune_b200.datasets import synthetic_sft_dataset
from torchtune_b200.models.llama3_1 import llama3_1


def _metric(log_file, name):
    return [float(x) for x in re.findall(rf"\b{re.escape(name)}:(\S+)", Path(log_file).read_text())]


def test_kd_single_device(tmp_path, tune_path, monkeypatch):
    ckpt = tmp_path / "ckpt"
    sd = write_tiny_hf_checkpoint(ckpt)
    out = tmp_path / "out"
    run_tune(
        tune_path,
        f"run knowledge_distillation_single_device --config tiny/llama_kd_single_device checkpointer.checkpoint_dir={ckpt} output_dir={out} metric_logger.filename=log.txt max_steps_per_epoch=3",
        monkeypatch,
    )
    log = out / "logs" / "log.txt"
    loss, ce, kd = _metric(log, "loss"), _metric(log, "class_loss"), _metric(log, "kd_loss")
    assert len(loss) == len(ce) == len(kd) == 3
    model = llama3_1(**TINY)
    model.load_state_dict(sd)
    ds = synthetic_sft_dataset(vocab_size=1024, seq_len=128, num_samples=20, prompt_len=16, seed=0)
    tokens = torch.stack([ds[0]["tokens"], ds[1]["tokens"]])
    labels = torch.stack([ds[0]["labels"], ds[1]["labels"]])
    with torch.no_grad():
        logits = model(tokens).reshape(-1, 1024)
    y = labels.reshape(-1)
    want_ce = F.cross_entropy(logits, y, ignore_index=-100).item()
    logp = F.log_softmax(logits, -1)
    ent = -(logp.exp() * logp).sum(-1)
    want_kd = (ent * (y != -100)).sum().item() / (y != -100).sum().item()
    assert ce[0] == pytest.approx(want_ce, rel=1e-4)
    assert kd[0] == pytest.approx(want_kd, rel=1e-4)
    assert loss[0] == pytest.approx(0.5 * want_ce + 0.5 * want_kd, rel=1e-4)

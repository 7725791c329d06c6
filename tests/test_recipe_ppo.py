"""PPO recipe end to end on CPU with tiny models: two optimisation rounds, finite metrics,
policy and value checkpoints written and the policy actually updated."""
import json
import re
from pathlib import Path

import torch
from safetensors.torch import load_file, save_file

from helpers import fixed_init_, run_tune, write_tiny_hf_checkpoint
from torchtune_b200.models.llama2 import llama2, llama2_classifier
from torchtune_b200.rlhf.utils import reward_tune_to_hf

ARCH = dict(vocab_size=1024, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=256, max_seq_len=256, intermediate_dim=768, norm_eps=1e-5)


def _write_reward_checkpoint(path: Path):
    path.mkdir(parents=True)
    model = llama2_classifier(num_classes=1, **ARCH)
    fixed_init_(model, seed=3)
    hf = reward_tune_to_hf(model.state_dict(), num_heads=4, num_kv_heads=2, dim=256)
    save_file({k: v.contiguous() for k, v in hf.items()}, str(path / "model-00001-of-00001.safetensors"))
    (path / "config.json").write_text(json.dumps({"hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 1024}))


def test_ppo_single_device(tmp_path, tune_path, monkeypatch):
    policy_dir, reward_dir, out = tmp_path / "policy", tmp_path / "reward", tmp_path / "out"
    write_tiny_hf_checkpoint(policy_dir, arch=ARCH, builder=llama2)
    _write_reward_checkpoint(reward_dir)
    run_tune(
        tune_path,
        f"run ppo_full_finetune_single_device --config tiny/llama2_ppo_single_device checkpointer.checkpoint_dir={policy_dir} "
        f"reward_checkpointer.checkpoint_dir={reward_dir} output_dir={out} metric_logger.filename=log.txt",
        monkeypatch,
    )
    text = (out / "logs" / "log.txt").read_text()
    steps = re.findall(r"Step (\d+)", text)
    assert len(steps) == 2  # num_steps 8 / batch_size 4
    for name in ("loss", "policy_loss", "value_loss", "kl", "rlhf_reward", "ratios", "clipfrac", "approx_policy_kl", "scores", "response_lengths"):
        vals = [float(x) for x in re.findall(rf"\b{name}:(\S+)", text)]
        assert len(vals) == 2 and all(v == v and abs(v) < 1e6 for v in vals), (name, vals)
    before = load_file(str(policy_dir / "model-00001-of-00001.safetensors"))
    after = load_file(str(out / "policy" / "epoch_0" / "model-00001-of-00001.safetensors"))
    assert any(not torch.equal(before[k], after[k]) for k in before)
    value = load_file(str(out / "value" / "epoch_0" / "model-00001-of-00001.safetensors"))
    assert "score.weight" in value and value["score.weight"].shape == (1, 256)

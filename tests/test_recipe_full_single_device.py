"""End-to-end CPU oracle: tiny Llama, fp32, 10 AdamW steps through the real CLI, chunked
linear-CE, HF-safetensors save and reload with identical logits; then resume equivalence."""
from pathlib import Path

import pytest
import torch

from helpers import TINY, read_losses, run_tune, write_tiny_hf_checkpoint
from torchtune_b200 import config
from torchtune_b200.datasets import synthetic_sft_dataset
from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.modules.loss import LinearCrossEntropyLoss
from torchtune_b200.training import FullModelHFCheckpointer


def _plain_torch_reference(sd, steps=10):
    """The same training run written directly against torch (AdamW, full logits CE)."""
    model = llama3_1(**TINY)
    model.load_state_dict(sd)
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5)
    ds = synthetic_sft_dataset(vocab_size=1024, seq_len=128, num_samples=20, prompt_len=16, seed=0)
    losses = []
    for step in range(steps):
        batch = [ds[2 * step], ds[2 * step + 1]]
        tokens = torch.stack([b["tokens"] for b in batch])
        labels = torch.stack([b["labels"] for b in batch])
        logits = model(tokens)
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 1024).float(), labels.reshape(-1), ignore_index=-100)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    return losses, model


def test_tiny_llama_cpu_10_steps_and_hf_round_trip(tmp_path, tune_path, monkeypatch):
    ckpt = tmp_path / "ckpt"
    out = tmp_path / "out"
    sd = write_tiny_hf_checkpoint(ckpt)
    run_tune(
        tune_path,
        f"run full_finetune_single_device --config tiny/llama_full_single_device checkpointer.checkpoint_dir={ckpt} "
        f"output_dir={out} metric_logger.filename=log.txt",
        monkeypatch,
    )
    losses = read_losses(out / "logs" / "log.txt")
    assert len(losses) == 10
    ref_losses, ref_model = _plain_torch_reference(sd)
    torch.testing.assert_close(torch.tensor(losses), torch.tensor(ref_losses), rtol=1e-4, atol=1e-4)
    assert abs(losses[0] - 6.93) < 0.1  # ln(1024)

    # reload what the recipe saved (HF layout) and compare logits with the reference run
    saved = out / "epoch_0"
    assert (saved / "model-00001-of-00001.safetensors").exists()
    assert (saved / "config.json").exists()
    reader = FullModelHFCheckpointer(str(saved), ["model-00001-of-00001.safetensors"], "LLAMA3", output_dir=str(tmp_path / "o2"))
    reloaded = llama3_1(**TINY)
    reloaded.load_state_dict(reader.load_checkpoint()["model"])
    tokens = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        torch.testing.assert_close(reloaded(tokens), ref_model(tokens), rtol=1e-4, atol=1e-4)

    # saving and reloading again is bit-exact (q/k permutations are exact inverses)
    reader.save_checkpoint({"model": reloaded.state_dict()}, epoch=0)
    again = FullModelHFCheckpointer(str(tmp_path / "o2" / "epoch_0"), ["model-00001-of-00001.safetensors"], "LLAMA3", output_dir=str(tmp_path / "o3"))
    sd2 = again.load_checkpoint()["model"]
    for k, v in reloaded.state_dict().items():
        assert torch.equal(v, sd2[k]), k


def test_config_naming_an_8bit_optimizer_of_an_absent_package_trains_and_resumes(tmp_path, tune_path, monkeypatch):
    """A config written for the reference's low-memory recipe names `bitsandbytes.optim.PagedAdamW8bit`; without that package the
    built-in 8-bit AdamW takes its place, trains, and its coded state survives a checkpoint."""
    try:
        import bitsandbytes  # noqa: F401

        pytest.skip("bitsandbytes is installed here")
    except ImportError:
        pass
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    base = (f"run full_finetune_single_device --config tiny/llama_full_single_device checkpointer.checkpoint_dir={ckpt} metric_logger.filename=log.txt "
            "optimizer._component_=bitsandbytes.optim.PagedAdamW8bit optimizer.lr=1e-3 max_steps_per_epoch=3 epochs=2 dataset.num_samples=12 ")
    run_tune(tune_path, base + f"output_dir={tmp_path / 'run'}", monkeypatch)
    losses = read_losses(tmp_path / "run" / "logs" / "log.txt")
    assert len(losses) == 6 and losses[-1] < losses[0]
    state = torch.load(tmp_path / "run" / "epoch_0" / "recipe_state.pt", weights_only=False)
    kinds = {v.dtype for st in state["optimizer"]["state"].values() for k, v in st.items() if isinstance(v, torch.Tensor) and k.endswith("_q")}
    assert kinds == {torch.int8, torch.uint8}
    # the second epoch again, from the checkpoint of the first: the same losses
    import shutil

    shutil.rmtree(tmp_path / "run" / "epoch_1")
    (tmp_path / "run" / "logs" / "log.txt").unlink()
    run_tune(tune_path, base + f"output_dir={tmp_path / 'run'} resume_from_checkpoint=True", monkeypatch)
    resumed = read_losses(tmp_path / "run" / "logs" / "log.txt")
    torch.testing.assert_close(torch.tensor(resumed), torch.tensor(losses[3:]), rtol=1e-5, atol=1e-5)


def test_resume_matches_uninterrupted(tmp_path, tune_path, monkeypatch):
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    base = f"run full_finetune_single_device --config tiny/llama_full_single_device checkpointer.checkpoint_dir={ckpt} metric_logger.filename=log.txt max_steps_per_epoch=3 epochs=2 dataset.num_samples=12 "
    run_tune(tune_path, base + f"output_dir={tmp_path / 'full'}", monkeypatch)
    full = read_losses(tmp_path / "full" / "logs" / "log.txt")
    assert len(full) == 6
    # interrupted run: one epoch only, then resume for the second
    run_tune(tune_path, base + f"output_dir={tmp_path / 'part'} epochs=2 save_every_n_steps=3 max_steps_per_epoch=3", monkeypatch) if False else None
    run_tune(tune_path, base.replace("epochs=2", "epochs=2") + f"output_dir={tmp_path / 'part'}", monkeypatch)
    # delete the final checkpoint, keep epoch_0 (intermediate, has recipe state), then resume
    import shutil

    shutil.rmtree(tmp_path / "part" / "epoch_1")
    (tmp_path / "part" / "logs" / "log.txt").unlink()
    run_tune(tune_path, base + f"output_dir={tmp_path / 'part'} resume_from_checkpoint=True", monkeypatch)
    resumed = read_losses(tmp_path / "part" / "logs" / "log.txt")
    torch.testing.assert_close(torch.tensor(resumed), torch.tensor(full[3:]), rtol=1e-5, atol=1e-5)


def test_async_sharded_checkpoint_resume_matches_uninterrupted(tmp_path, tune_path, monkeypatch):
    """enable_async_checkpointing: intermediate checkpoints are per-rank shard files written by a background thread;
    resuming from one continues the loss curve of the uninterrupted run."""
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    base = (f"run full_finetune_single_device --config tiny/llama_full_single_device checkpointer.checkpoint_dir={ckpt} metric_logger.filename=log.txt "
            "max_steps_per_epoch=3 dataset.num_samples=12 enable_async_checkpointing=True ")
    run_tune(tune_path, base + f"epochs=2 output_dir={tmp_path / 'full'}", monkeypatch)
    full = read_losses(tmp_path / "full" / "logs" / "log.txt")
    assert len(full) == 6
    assert (tmp_path / "full" / "epoch_0" / "rank_0.pt").exists() and (tmp_path / "full" / "epoch_0" / "metadata.json").exists()
    assert (tmp_path / "full" / "epoch_1" / "model-00001-of-00001.safetensors").exists()  # the final checkpoint is a full one
    # interrupted run: stop after the first epoch by asking for a single epoch of two, then resume
    run_tune(tune_path, base + f"epochs=2 output_dir={tmp_path / 'part'}", monkeypatch)
    import shutil

    shutil.rmtree(tmp_path / "part" / "epoch_1")
    (tmp_path / "part" / "logs" / "log.txt").unlink()
    run_tune(tune_path, base + f"epochs=2 output_dir={tmp_path / 'part'} resume_from_checkpoint=True", monkeypatch)
    resumed = read_losses(tmp_path / "part" / "logs" / "log.txt")
    assert len(resumed) == 3
    torch.testing.assert_close(torch.tensor(resumed), torch.tensor(full[3:]), rtol=1e-5, atol=1e-6)


def test_distributed_checkpointer_roundtrip_sync_and_async(tmp_path):
    from torchtune_b200.training import DistributedCheckpointer

    ck = DistributedCheckpointer(checkpoint_dir=str(tmp_path), output_dir=str(tmp_path / "out"))
    state = {"model": {"w": torch.arange(6.0).view(2, 3)}, "optimizer": {"step": 3, "m": torch.ones(4)}, "seed": 7}
    ck.save_checkpoint(state, epoch=0)
    ck.save_checkpoint({**state, "seed": 8}, epoch=1, save_async=True)
    ck.wait()
    assert not list((tmp_path / "out").glob("*.partial"))
    target = {"model": {"w": torch.zeros(2, 3)}, "optimizer": {"step": 0, "m": torch.zeros(4)}, "seed": 0}
    out = ck.load_checkpoint(target)
    assert out["seed"] == 8 and out["optimizer"]["step"] == 3
    assert torch.equal(target["model"]["w"], state["model"]["w"]) and torch.equal(target["optimizer"]["m"], torch.ones(4))
    with __import__("pytest").raises(ValueError):
        ck.load_checkpoint({"model": {"w": torch.zeros(3, 3)}})

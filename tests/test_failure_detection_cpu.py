"""Failure detection and recovery, exercised on the host only (gloo ranks on CPU, files on disk): a rank that never joins a
collective ends the others' wait with an error after ``process_group_timeout_s``; an exception on one rank ends the whole
``tune run`` job with a non-zero exit code; a checkpoint directory whose writers did not finish is never resumed from."""
import os
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _absent_rank_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from torchtune_b200.parallel.strategy import ParallelStrategy

    strategy = ParallelStrategy({"process_group_timeout_s": 3}, torch.device("cpu"))
    t = torch.ones(())
    strategy.all_reduce_sum_(t)  # everyone is here: works
    assert t.item() == world
    if rank == 1:
        time.sleep(12)  # this rank is stuck on the host and never reaches the next collective
        results[rank] = "absent"
        return
    t0 = time.perf_counter()
    try:
        strategy.all_reduce_sum_(t)
        results[rank] = "no error"
    except Exception as exc:  # noqa: BLE001 - the backend's error type is not part of the contract
        results[rank] = f"error after {time.perf_counter() - t0:.1f}s: {type(exc).__name__}"


@pytest.mark.timeout(120)
def test_rank_that_never_joins_ends_the_collective_with_an_error():
    results = mp.Manager().dict()
    mp.spawn(_absent_rank_worker, args=(2, 29613, results), nprocs=2, join=True)
    assert results[1] == "absent"
    assert results[0].startswith("error after"), results[0]
    assert float(results[0].split()[2].rstrip("s:")) < 11.0, results[0]


@pytest.mark.timeout(300)
def test_exception_on_one_rank_fails_the_job(tmp_path):
    """``tune run`` on two ranks where rank 1's data loading raises: the launcher must come back with a failure instead of
    leaving rank 0 waiting."""
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import write_tiny_hf_checkpoint

    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    plugin = tmp_path / "failing_dataset.py"
    plugin.write_text(
        "import os\n"
        "from torchtune_b200.datasets import synthetic_sft_dataset\n"
        "def build(*args, **kw):\n"
        "    if os.environ.get('RANK') == '1':\n"
        "        raise RuntimeError('injected host-side failure on rank 1')\n"
        "    return synthetic_sft_dataset(*args, **kw)\n"
    )
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{tmp_path}", MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, str(ROOT / "tune"), "run", "--nnodes=1", "--nproc_per_node=2", "--master-addr=127.0.0.1", "--master-port=29572", "--max-restarts=0",
           "full_finetune_distributed", "--config", "tiny/llama_full_distributed", f"checkpointer.checkpoint_dir={ckpt}", f"output_dir={tmp_path / 'out'}",
           "dataset._component_=failing_dataset.build", "process_group_timeout_s=5", "max_steps_per_epoch=1"]
    t0 = time.perf_counter()
    res = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode != 0
    assert "injected host-side failure on rank 1" in (res.stdout + res.stderr)
    assert time.perf_counter() - t0 < 200


def test_unfinished_checkpoint_directory_is_never_resumed_from(tmp_path):
    from torchtune_b200.training.checkpointing._utils import get_all_checkpoints_in_dir, get_most_recent_checkpoint

    (tmp_path / "step_2").mkdir()
    (tmp_path / "step_2" / "rank_0.pt").write_bytes(b"x")
    (tmp_path / "step_4.partial").mkdir()  # writers were interrupted before the rename
    (tmp_path / "step_4.partial" / "rank_0.pt").write_bytes(b"x")
    (tmp_path / "step_6").mkdir()  # created but empty
    assert get_most_recent_checkpoint(tmp_path) == tmp_path / "step_2"
    assert sorted(p.name for p in get_all_checkpoints_in_dir(tmp_path)) == ["step_2", "step_6"]


def test_stale_partial_directory_and_markers_of_a_dead_attempt_are_discarded(tmp_path):
    """A job that died in mid-save leaves ``step_4.partial`` with the rank files and ``.done`` markers of that attempt.  The next
    process clears it before its first save, and its own markers carry a per-save nonce, so the old ones could never stand in
    for a rank that has not written yet."""
    from torchtune_b200.training.checkpointing._sharded import DistributedCheckpointer

    out = tmp_path / "out"
    stale = out / "step_4.partial"
    stale.mkdir(parents=True)
    (stale / "rank_0.pt").write_bytes(b"torn")
    (stale / "rank_0.done").write_text("ok")
    (stale / "rank_1.done").write_text("ok")
    nested = out / "epoch_0" / "adapter_model.partial"
    nested.mkdir(parents=True)
    (nested / "rank_0.done").write_text("ok")
    ckpt = DistributedCheckpointer(str(tmp_path), str(out))
    ckpt.save_checkpoint({"w": torch.arange(4.0)}, epoch=0, step=4, dir_prefix="step")
    ckpt.wait()
    assert not stale.exists() and not nested.exists()
    done = out / "step_4"
    assert sorted(p.name for p in done.iterdir()) == ["metadata.json", "rank_0.pt"]  # no marker survives the publish
    assert torch.equal(torch.load(done / "rank_0.pt")["w"], torch.arange(4.0))


def test_sharded_checkpoint_of_another_world_size_is_refused(tmp_path):
    from torchtune_b200.training.checkpointing._sharded import DistributedCheckpointer

    ckpt = DistributedCheckpointer(str(tmp_path), str(tmp_path / "out"))
    ckpt.save_checkpoint({"w": torch.arange(4.0)}, epoch=0, step=2, dir_prefix="step")
    ckpt.wait()
    meta = tmp_path / "out" / "step_2" / "metadata.json"
    meta.write_text(meta.read_text().replace('"world_size": 1', '"world_size": 4'))
    with pytest.raises(ValueError, match="was written by 4 ranks"):
        ckpt.load_checkpoint()


def test_restarted_job_resumes_from_the_newest_complete_checkpoint(tmp_path, tune_path, monkeypatch):
    """What ``torchrun --max-restarts`` does after a worker failure is to run the same command again with
    ``TORCHELASTIC_RESTART_COUNT`` raised: the recipe must then pick up the newest complete checkpoint by itself."""
    import shutil

    from helpers import read_losses, run_tune, write_tiny_hf_checkpoint

    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt)
    base = f"run full_finetune_single_device --config tiny/llama_full_single_device checkpointer.checkpoint_dir={ckpt} metric_logger.filename=log.txt max_steps_per_epoch=3 epochs=2 dataset.num_samples=12 "
    run_tune(tune_path, base + f"output_dir={tmp_path / 'full'}", monkeypatch)
    full = read_losses(tmp_path / "full" / "logs" / "log.txt")
    run_tune(tune_path, base + f"output_dir={tmp_path / 'part'}", monkeypatch)
    shutil.rmtree(tmp_path / "part" / "epoch_1")  # as if the job had died during the second epoch
    (tmp_path / "part" / "epoch_2.partial").mkdir()
    (tmp_path / "part" / "logs" / "log.txt").unlink()
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "1")
    run_tune(tune_path, base + f"output_dir={tmp_path / 'part'}", monkeypatch)  # same command line, no resume flag
    resumed = read_losses(tmp_path / "part" / "logs" / "log.txt")
    torch.testing.assert_close(torch.tensor(resumed), torch.tensor(full[3:]), rtol=1e-5, atol=1e-5)
    # a first start (restart count 0) with the same leftovers starts from the beginning
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "0")
    shutil.rmtree(tmp_path / "part" / "epoch_1")
    (tmp_path / "part" / "logs" / "log.txt").unlink()
    run_tune(tune_path, base + f"output_dir={tmp_path / 'part'}", monkeypatch)
    assert len(read_losses(tmp_path / "part" / "logs" / "log.txt")) == 6

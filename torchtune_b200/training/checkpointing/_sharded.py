"""Per-rank sharded checkpoints with optional asynchronous writes
(role of torchtune/training/checkpointing/_checkpointer.py:1305-1478, ``DistributedCheckpointer``).

The reference delegates to ``torch.distributed.checkpoint`` (a planner negotiates which rank writes which
DTensor chunk).  In this package sharded state is already a contiguous per-rank slice of flat buffers (optimizer
moments, tensor-parallel weight shards), so every rank simply writes *its own* state to ``rank_<r>.pt`` and rank 0
adds ``metadata.json`` (world size, keys, step).  An asynchronous save first snapshots all tensors into host
memory — the only part that blocks training — and hands the file write to a worker thread; a second save waits
for the previous one.  Checkpoints are written to a temporary directory and renamed when every rank is done, so a
directory that exists is always complete.
"""
from __future__ import annotations

import json
import os
import shutil
import threading
import time
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ...utils import get_logger, get_world_size_and_rank
from ._utils import get_most_recent_checkpoint

logger = get_logger("DEBUG")


def _to_host(obj: Any) -> Any:
    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_host(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_host(v) for v in obj)
    return obj


def _copy_into(dst: Any, src: Any, path: str = "") -> Any:
    """Fill ``dst`` (the caller's pre-allocated state) from ``src``; tensors are copied in place so sharded /
    device placement is kept, other values are replaced.  Keys missing from ``src`` are left untouched."""
    if isinstance(dst, dict) and isinstance(src, dict):
        for k in dst:
            if k in src:
                dst[k] = _copy_into(dst[k], src[k], f"{path}.{k}")
        for k in src:
            if k not in dst:
                dst[k] = src[k]
        return dst
    if isinstance(dst, torch.Tensor) and isinstance(src, torch.Tensor):
        if dst.shape != src.shape:
            raise ValueError(f"checkpoint entry {path} has shape {tuple(src.shape)}, expected {tuple(dst.shape)} (was it written with a different world size?)")
        dst.copy_(src)
        return dst
    return src


class DistributedCheckpointer:
    def __init__(self, checkpoint_dir: str, output_dir: str, process_group: Optional[dist.ProcessGroup] = None) -> None:
        self._checkpoint_dir = Path(checkpoint_dir)
        self._output_dir = Path(output_dir)
        self._process_group = process_group
        self._world, self._rank = get_world_size_and_rank()
        self._adapter_dir = "adapter_model"
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="ckpt-writer")
        self._checkpoint_future: Optional[Future] = None
        self._save_seq = 0  # saves issued by this process; identical on every rank because saves are collective
        self._stale_cleared = False

    @property
    def output_dir(self) -> Path:
        return self._output_dir

    def _barrier(self) -> None:
        if dist.is_available() and dist.is_initialized() and self._world > 1:
            dist.barrier(group=self._process_group)

    def wait(self) -> None:
        """Block until a pending asynchronous save has been written."""
        if self._checkpoint_future is not None:
            self._checkpoint_future.result()
            self._checkpoint_future = None

    # ------------------------------------------------------------------ save
    def _clear_stale_partials(self) -> None:
        """Once per process, before the first writer runs: rank 0 removes ``*.partial`` directories that an interrupted job left
        behind (their ``rank_r.pt`` files and markers belong to a dead attempt), then every rank passes a barrier."""
        if self._stale_cleared:
            return
        self._stale_cleared = True
        if self._rank == 0 and self._output_dir.is_dir():
            for pattern in ("*.partial", "*/*.partial"):
                for stale in self._output_dir.glob(pattern):
                    if stale.is_dir():
                        shutil.rmtree(stale, ignore_errors=True)
        self._barrier()

    def _write(self, host_state: Dict[str, Any], final: Path, step_info: Dict[str, Any], nonce: str) -> None:
        tmp = final.with_name(final.name + ".partial")
        tmp.mkdir(parents=True, exist_ok=True)
        torch.save(host_state, tmp / f"rank_{self._rank}.pt")
        # the marker name carries this save's nonce (step, restart count, save counter), so a marker left by an earlier attempt
        # at the same step can never count as "rank r has finished writing"
        (tmp / f"rank_{self._rank}.{nonce}.done").write_text("ok")
        if self._rank == 0:
            # rank 0 publishes the directory once every rank's marker is present (file-system rendezvous:
            # the writer thread must not issue collectives that could interleave with training collectives)
            deadline = time.time() + 3600
            while any(not (tmp / f"rank_{r}.{nonce}.done").exists() for r in range(self._world)):
                if time.time() > deadline:
                    raise TimeoutError(f"not all ranks finished writing {tmp}")
                time.sleep(0.05)
            (tmp / "metadata.json").write_text(json.dumps({"world_size": self._world, "keys": sorted(host_state.keys()), **step_info}))
            for marker in tmp.glob("rank_*.done"):
                marker.unlink()
            if final.exists():
                shutil.rmtree(final)
            os.replace(tmp, final)

    def save_checkpoint(self, state_dict: Dict[str, Any], epoch: int, save_async: bool = False, adapter_only: bool = False, *, step: Optional[int] = None, dir_prefix: str = "epoch") -> None:
        if dir_prefix == "epoch":
            name = f"epoch_{epoch}"
        elif dir_prefix == "step":
            if step is None:
                raise ValueError("Step number is required when dir_prefix is 'step'.")
            name = f"step_{step}"
        else:
            raise ValueError(f"Invalid dir_prefix: {dir_prefix}. Must be one of 'epoch' or 'step'.")
        final = self._output_dir / name
        if adapter_only:
            final = final / self._adapter_dir
        if self._checkpoint_future is not None and not self._checkpoint_future.done():
            t0 = time.perf_counter()
            logger.info(f"Rank {self._rank}: previous checkpoint has not finished. Checkpointing frequency is too high. Waiting...")
            self._checkpoint_future.result()
            logger.info(f"Rank {self._rank}: waited {time.perf_counter() - t0:.2f} seconds for previous checkpoint to finish")
        self._checkpoint_future = None
        self._clear_stale_partials()
        self._save_seq += 1
        nonce = f"e{epoch}-s{step}-r{os.environ.get('TORCHELASTIC_RESTART_COUNT', '0')}-n{self._save_seq}"
        t0 = time.perf_counter()
        host_state = _to_host(state_dict)  # the only step that must finish before training continues
        info = {"epoch": epoch, "step": step}
        if save_async:
            self._checkpoint_future = self._pool.submit(self._write, host_state, final, info, nonce)

            def _report(f: Future) -> None:
                if f.exception() is None:
                    logger.info(f"Rank {self._rank}: Checkpoint is saved asynchronously to {final} successfully.")
                else:
                    logger.error(f"Rank {self._rank}: Checkpoint failed to save asynchronously to {final} with the exception {f.exception()}")

            self._checkpoint_future.add_done_callback(_report)
            logger.info(f"Rank {self._rank}: Trainer was blocked for {time.perf_counter() - t0:.2f} seconds for checkpointing to finish...")
        else:
            self._write(host_state, final, info, nonce)
            if self._rank != 0:  # wait for rank 0 to publish the directory
                deadline = time.time() + 3600
                while not (final / "metadata.json").exists():
                    if time.time() > deadline:
                        raise TimeoutError(f"checkpoint {final} was not published")
                    time.sleep(0.05)
            self._barrier()

    # ------------------------------------------------------------------ load
    def load_checkpoint(self, state_dict: Optional[Dict[str, Any]] = None, adapter_only: bool = False) -> Dict[str, Any]:
        """Load this rank's shard of the most recent checkpoint under ``output_dir`` into ``state_dict`` (in place when
        given, so the caller's sharded tensors keep their placement)."""
        self.wait()
        path = get_most_recent_checkpoint(self._output_dir)
        if path is None:
            raise ValueError("No intermediate checkpoint was found in the output directory.Please ensure that a checkpoint exists to load.")
        path = Path(path)
        if adapter_only:
            path = path / self._adapter_dir
        meta = json.loads((path / "metadata.json").read_text())
        if meta["world_size"] != self._world:
            raise ValueError(f"checkpoint {path} was written by {meta['world_size']} ranks, this job has {self._world}")
        loaded = torch.load(path / f"rank_{self._rank}.pt", map_location="cpu", weights_only=False)
        if state_dict is None:
            return loaded
        return _copy_into(state_dict, loaded)

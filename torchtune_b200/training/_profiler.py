"""torch.profiler set-up and trace export (parity: torchtune/training/_profiler.py:33-387)."""
from __future__ import annotations

import os
import time
from functools import partial
from pathlib import Path
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..config import DictConfig
from ..utils import get_logger, get_world_size_and_rank

log = get_logger("INFO")

PROFILER_KEY = "profiler"
DEFAULT_PROFILER_ACTIVITIES = {torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA}
DEFAULT_SCHEDULE: dict = {"wait_steps": 5, "warmup_steps": 5, "active_steps": 2, "num_cycles": 1}
DEFAULT_TRACE_OPTS: dict = {"profile_memory": False, "with_stack": False, "record_shapes": True, "with_flops": False}
DEFAULT_PROFILE_DIR: str = "profiler_output"


def _warn(msg: str) -> None:
    if get_world_size_and_rank()[1] == 0:
        log.warning(msg)


def trace_handler(prof: torch.profiler.profile, output_dir: str, metric: str = "self_cuda_time_total", row_limit: int = 25) -> None:
    """Per profiling cycle write, under ``output_dir/iteration_<step>/``: a gzipped Chrome
    trace per rank, rank-0 memory snapshot (if memory profiling), stack files and the
    key-averages table; then barrier so ranks leave together."""
    _, rank = get_world_size_and_rank()
    out = Path(output_dir) / f"iteration_{prof.step_num}"
    out.mkdir(parents=True, exist_ok=True)
    t0 = time.monotonic()
    prof.export_chrome_trace(str(out / f"rank{rank}_trace.json.gz"))
    if rank == 0:
        log.info(f"Finished dumping traces in {time.monotonic() - t0:.2f} seconds")
    if prof.profile_memory and torch.cuda.is_available() and rank == 0:
        try:
            torch.cuda.memory._dump_snapshot(str(out / "rank0_memory_snapshot.pickle"))
        except Exception as exc:
            log.warning(f" Failed to export memory snapshot: {exc}")
    if prof.with_stack:
        try:
            prof.export_stacks(str(out / f"rank{rank}_stacks.txt"), metric=metric)
        except Exception as exc:
            log.warning(f" Failed to export stacks: {exc}")
    (out / f"rank{rank}_key_averages.txt").write_text(prof.key_averages(group_by_input_shape=prof.record_shapes).table(sort_by=metric, row_limit=row_limit))
    if rank == 0:
        log.info(f"Finished dumping traces in {time.monotonic() - t0:.2f} seconds")
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


class DummyProfiler:
    """No-op stand-in so recipes can call ``start/step/stop`` unconditionally."""

    def __enter__(self):
        return self

    def __exit__(self, *args):
        pass

    def start(self):
        pass

    def stop(self):
        pass

    def step(self):
        pass


def setup_torch_profiler(
    enabled: bool = False,
    cpu: bool = True,
    cuda: bool = True,
    xpu: bool = False,
    hpu: bool = False,
    profile_memory: bool = DEFAULT_TRACE_OPTS["profile_memory"],
    with_stack: bool = DEFAULT_TRACE_OPTS["with_stack"],
    record_shapes: bool = DEFAULT_TRACE_OPTS["record_shapes"],
    with_flops: bool = DEFAULT_TRACE_OPTS["with_flops"],
    wait_steps: Optional[int] = None,
    warmup_steps: Optional[int] = None,
    active_steps: Optional[int] = None,
    num_cycles: Optional[int] = None,
    output_dir: Optional[str] = None,
) -> Tuple[object, DictConfig]:
    """Build ``(profiler, resolved config)``.  Missing schedule fields take the defaults
    (wait 5 / warmup 5 / active 2 / 1 cycle); memory profiling forces stacks and shapes."""
    if not enabled:
        _warn(" Profiling disabled.")
        return DummyProfiler(), DictConfig({"enabled": False})
    activities = []
    if cpu:
        activities.append(torch.profiler.ProfilerActivity.CPU)
    if cuda and torch.cuda.is_available():
        activities.append(torch.profiler.ProfilerActivity.CUDA)
    if not activities:
        _warn("No activities specified, defaulting to CPU + CUDA")
        activities = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        cpu = cuda = True
    sched = {"wait_steps": wait_steps, "warmup_steps": warmup_steps, "active_steps": active_steps, "num_cycles": num_cycles}
    if all(v is None for v in sched.values()):
        _warn(" No schedule found in config, defaulting to {}".format(", ".join(f"{k} = {v}" for k, v in DEFAULT_SCHEDULE.items())))
        sched = dict(DEFAULT_SCHEDULE)
    else:
        for k, v in sched.items():
            if v is None:
                _warn(f" Missing key {k} in torch profiler schedule, defaulting to {k} = {DEFAULT_SCHEDULE[k]}")
                sched[k] = DEFAULT_SCHEDULE[k]
    schedule = torch.profiler.schedule(wait=sched["wait_steps"], warmup=sched["warmup_steps"], active=sched["active_steps"], repeat=sched["num_cycles"])
    if profile_memory:
        _warn("`profile_memory` requires `with_stack` and `record_shapes`, these will be enabled since `profile_memory` is True")
    with_stack = with_stack or profile_memory
    record_shapes = record_shapes or profile_memory
    output_dir = Path(output_dir) if output_dir is not None else Path(DEFAULT_PROFILE_DIR)
    output_dir.mkdir(parents=True, exist_ok=True)
    profiler = torch.profiler.profile(
        activities=activities,
        profile_memory=profile_memory,
        with_stack=with_stack,
        record_shapes=record_shapes,
        with_flops=with_flops,
        schedule=schedule,
        experimental_config=torch._C._profiler._ExperimentalConfig(verbose=True) if with_stack else None,
        on_trace_ready=partial(trace_handler, output_dir=str(output_dir)),
    )
    cfg = DictConfig(
        {
            "enabled": enabled,
            "output_dir": str(output_dir),
            "cpu": cpu,
            "cuda": cuda,
            "xpu": xpu,
            "hpu": hpu,
            "profile_memory": profile_memory,
            "with_stack": with_stack,
            "record_shapes": record_shapes,
            "with_flops": with_flops,
            **sched,
        }
    )
    return profiler, cfg

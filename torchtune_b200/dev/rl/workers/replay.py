"""Bounded first-in-first-out buffer of prompt groups between post-processing and training (the reference uses a
``RayReplayBuffer`` whose size equals the inference batch, recipes/configs/dev/qwen3B_async_grpo.yaml:42 — effectively a queue)."""
from __future__ import annotations

import queue
from typing import Callable, List, Optional

from ..datatypes import Trajectory


class ReplayBuffer:
    def __init__(self, max_size: int, backing_queue=None):
        self._q = backing_queue if backing_queue is not None else queue.Queue(maxsize=max(1, int(max_size)))

    def extend(self, traj: Trajectory, should_stop: Optional[Callable[[], bool]] = None) -> bool:
        while True:
            try:
                self._q.put(traj, timeout=0.2)
                return True
            except queue.Full:
                if should_stop is not None and should_stop():
                    return False

    def sample(self, groups: int, should_stop: Optional[Callable[[], bool]] = None, pad_id: int = 0) -> Optional[Trajectory]:
        got: List[Trajectory] = []
        while len(got) < groups:
            try:
                got.append(self._q.get(timeout=0.2))
            except queue.Empty:
                if should_stop is not None and should_stop():
                    return None
        return Trajectory.stack(got, pad_id=pad_id)

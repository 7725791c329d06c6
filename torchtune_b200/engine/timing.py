"""Device-side step timing: CUDA events on the launching stream, host clock on CPU."""
from __future__ import annotations

import time
from typing import Optional

import torch


class StepTimer:
    """``start()`` / ``stop()`` bracket a region; ``elapsed_s`` is device time on CUDA
    (event pair, synchronised on read) and wall time on CPU."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self._t0: Optional[float] = None
        self._e0 = self._e1 = None
        self._elapsed = 0.0

    def start(self) -> None:
        if self.cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self.cuda:
            self._e1.record()
        else:
            self._elapsed = time.perf_counter() - self._t0

    @property
    def elapsed_s(self) -> float:
        if self.cuda:
            self._e1.synchronize()
            return self._e0.elapsed_time(self._e1) / 1e3
        return self._elapsed

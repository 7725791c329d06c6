"""Latest published policy weights and their version (parity: torchtune/dev/rl/workers/parameter_servers/vllm.py:19-111).

The reference keeps a sharded copy of the weights in a Ray actor and pushes them to the vLLM workers over a dedicated NCCL
group.  Here the server owns one host copy of every tensor (in shared memory when the roles are processes): the trainer
overwrites it under a lock and bumps the version, inference workers poll the version between batches and copy what changed —
a pull protocol, so a slow inference worker never blocks the trainer."""
from __future__ import annotations

import threading
from typing import Dict, Optional, Tuple

import torch


class ParameterServer:
    def __init__(self, template: Dict[str, torch.Tensor], shared: bool = False, lock=None, version=None):
        self._weights = {k: v.detach().to("cpu", copy=True).contiguous() for k, v in template.items()}
        if shared:
            import torch.multiprocessing as mp

            for t in self._weights.values():
                t.share_memory_()
            self._lock = lock if lock is not None else mp.Lock()
            self._version = version if version is not None else mp.Value("i", 0)
        else:
            self._lock = lock if lock is not None else threading.Lock()
            self._version = version

        self._local_version = 0

    @property
    def version(self) -> int:
        return self._version.value if self._version is not None else self._local_version

    def publish(self, state_dict: Dict[str, torch.Tensor], version: Optional[int] = None) -> int:
        """Store ``state_dict`` (any device) as the newest weights; returns the new version."""
        with self._lock:
            for k, dst in self._weights.items():
                dst.copy_(state_dict[k].detach(), non_blocking=False)
            new = (self.version + 1) if version is None else int(version)
            if self._version is not None:
                self._version.value = new
            else:
                self._local_version = new
            return new

    def fetch(self, newer_than: int) -> Optional[Tuple[int, Dict[str, torch.Tensor]]]:
        """``(version, weights)`` when something newer than ``newer_than`` was published, else ``None``.  The returned tensors are
        private copies (the trainer may publish again at once)."""
        if self.version <= newer_than:
            return None
        with self._lock:
            return self.version, {k: v.clone() for k, v in self._weights.items()}

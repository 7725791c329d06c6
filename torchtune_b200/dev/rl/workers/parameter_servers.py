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


class BroadcastParameterServer(ParameterServer):
    """Push protocol for inference workers that live in another job (parity: torchtune/dev/rl/workers/parameter_servers/vllm.py:67-111).

    The pull protocol above needs the roles to share host memory.  When the inference workers are separate processes on other GPUs
    (or other hosts), the server takes rank 0 of a :class:`~torchtune_b200.dev.rl.utils.StatelessGroup`, the workers take ranks
    ``1..``, and :meth:`push` broadcasts the version and then every tensor in sorted-name order;
    :class:`~torchtune_b200.dev.rl.workers.datacollectors.GeneratorWeightWorker` receives in the same order.  Tensors are staged on the
    group's device one at a time, so the transfer never holds a second copy of the model."""

    def __init__(self, template: Dict[str, torch.Tensor], shared: bool = False, lock=None, version=None):
        super().__init__(template, shared=shared, lock=lock, version=version)
        self._group = None

    def init_update_group(self, master_address: str, master_port: int, world_size: int, device: Optional[torch.device] = None,
                          timeout_s: float = 600.0) -> None:
        from ..utils import stateless_init_process_group

        self._group = stateless_init_process_group(master_address, master_port, 0, world_size, device, timeout_s)

    def manifest(self):
        """``[(name, dtype, shape)]`` in the order :meth:`push` sends them."""
        return [(k, self._weights[k].dtype, tuple(self._weights[k].shape)) for k in sorted(self._weights)]

    def push(self) -> int:
        """Broadcast the current version and weights to every worker of the update group; returns the version sent."""
        if self._group is None:
            raise RuntimeError("init_update_group() has not been called")
        dev = self._group.device
        with self._lock:
            version = self.version
            self._group.broadcast(torch.tensor([version], dtype=torch.int64, device=dev), src=0)
            for k in sorted(self._weights):
                self._group.broadcast(self._weights[k].to(dev, copy=True), src=0)
        return version

    def close(self) -> None:
        if self._group is not None:
            self._group.close()
            self._group = None


# the reference's name for the server that feeds its inference engine
VLLMParameterServer = BroadcastParameterServer

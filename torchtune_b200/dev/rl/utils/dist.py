"""A process group that lives beside the default one (parity: torchtune/dev/rl/utils/dist.py:10-32).

The trainer ranks and the inference workers of asynchronous RL are separate jobs: each already has (or has no) default process
group of its own, and the weights still have to cross from one to the other.  The reference builds that bridge from vLLM's
stateless group and its NCCL wrapper.  Here it is a ``TCPStore`` rendezvous plus a backend object constructed directly —
``ProcessGroupNCCL`` for CUDA tensors, ``ProcessGroupGloo`` for host tensors — which never touches
``torch.distributed``'s global state, so both sides keep whatever default group they had."""
from __future__ import annotations

from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist


class StatelessGroup:
    """Broadcast / send / recv / barrier between ``world_size`` processes that share nothing but an address and a port.

    Rank 0 hosts the store.  ``device`` picks the backend: a CUDA device gives NCCL (tensors must live on that device), anything
    else gives gloo."""

    def __init__(self, master_address: str, master_port: int, rank: int, world_size: int,
                 device: Optional[torch.device] = None, timeout_s: float = 600.0):
        if not 0 <= rank < world_size:
            raise ValueError(f"rank {rank} outside a group of {world_size}")
        self.rank, self.world_size = int(rank), int(world_size)
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        timeout = timedelta(seconds=timeout_s)
        self._store = dist.TCPStore(master_address, int(master_port), self.world_size, is_master=(rank == 0),
                                    timeout=timeout, wait_for_workers=True)
        # a prefix keeps this group's keys apart from anything else that shares the port
        store = dist.PrefixStore("ttb_stateless", self._store)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            self._pg = dist.ProcessGroupNCCL(store, self.rank, self.world_size, timeout)
        else:
            self._pg = dist.ProcessGroupGloo(store, self.rank, self.world_size, timeout)

    def _check(self, tensor: torch.Tensor) -> None:
        if tensor.device.type != self.device.type:
            raise ValueError(f"group on {self.device.type} was given a {tensor.device.type} tensor")

    def broadcast(self, tensor: torch.Tensor, src: int = 0, stream=None) -> torch.Tensor:
        """In-place broadcast from ``src``.  ``stream`` is accepted for call compatibility with the reference's communicator; the
        NCCL backend orders the collective after the current stream on its own."""
        self._check(tensor)
        opts = dist.BroadcastOptions()
        opts.rootRank, opts.rootTensor = int(src), 0
        self._pg.broadcast([tensor], opts).wait()
        return tensor

    def send(self, tensor: torch.Tensor, dst: int) -> None:
        self._check(tensor)
        self._pg.send([tensor], int(dst), 0).wait()

    def recv(self, tensor: torch.Tensor, src: int) -> torch.Tensor:
        self._check(tensor)
        self._pg.recv([tensor], int(src), 0).wait()
        return tensor

    def barrier(self) -> None:
        self._pg.barrier().wait()

    def close(self) -> None:
        """Drop the backend before the store (the store's host must outlive the others' last key access, hence the barrier)."""
        if self._pg is not None:
            try:
                self._pg.barrier().wait()
                if hasattr(self._pg, "shutdown"):
                    self._pg.shutdown()  # releases the communicator now instead of at interpreter exit
            finally:
                self._pg = None
                self._store = None


def stateless_init_process_group(master_address: str, master_port: int, rank: int, world_size: int,
                                 device: Optional[torch.device] = None, timeout_s: float = 600.0) -> StatelessGroup:
    """Same call as the reference's helper; returns a :class:`StatelessGroup`."""
    return StatelessGroup(master_address, master_port, rank, world_size, device, timeout_s)

"""Device selection and batch movement (parity: torchtune/utils/_device.py:24-289)."""
from __future__ import annotations

import os
from enum import Enum
from typing import Any, Optional, Tuple

import torch


def get_world_size_and_rank() -> Tuple[int, int]:
    """``(world_size, rank)`` of the default process group, ``(1, 0)`` outside one."""
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.distributed.get_world_size(), torch.distributed.get_rank()
    return 1, 0


def is_torch_npu_available() -> bool:
    return False


def _local_rank() -> Optional[int]:
    value = os.environ.get("LOCAL_RANK")
    return int(value) if value is not None else None


def _default_device_type() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def _setup_device(device: torch.device) -> torch.device:
    """Pin an index-less CUDA device to ``LOCAL_RANK`` and make it current."""
    if device.type != "cuda":
        return device
    local = _local_rank() or 0
    if device.index is None:
        device = torch.device("cuda", local)
    if device.index >= torch.cuda.device_count():
        raise RuntimeError("The local rank is larger than the number of available GPUs.")
    torch.cuda.set_device(device)
    return device


def _validate_device_from_env(device: torch.device) -> None:
    local = _local_rank()
    if device.type == "cuda" and local is not None and device.index is not None and device.index != local:
        raise RuntimeError(
            f"You can't specify a device index when using distributed training. "
            f"Device specified is {device} but local rank is:{local}"
        )
    try:
        torch.empty(0, device=device)
    except RuntimeError as exc:
        raise RuntimeError(f"The device {device} is not available on this machine.") from exc


def get_device(device: Optional[str] = None) -> torch.device:
    """Resolve ``"cuda"``/``"cpu"``/``None`` to a concrete, validated ``torch.device``."""
    dev = torch.device(device if device is not None else _default_device_type())
    dev = _setup_device(dev)
    _validate_device_from_env(dev)
    return dev


def batch_to_device(batch: dict, device: torch.device) -> None:
    """Move every tensor of a (nested) batch dict in place; objects exposing ``.to`` follow."""
    for key, value in batch.items():
        if isinstance(value, dict):
            batch_to_device(value, device)
        elif isinstance(value, torch.Tensor):
            batch[key] = value.to(device, non_blocking=value.is_pinned() if value.device.type == "cpu" else False)
        elif hasattr(value, "to") and callable(value.to):
            batch[key] = value.to(device)
        elif isinstance(value, (list, tuple)) and all(isinstance(v, torch.Tensor) for v in value):
            batch[key] = type(value)(v.to(device) for v in value)
        elif isinstance(value, (int, float, str, bool, type(None), list, tuple)):
            continue
        else:
            raise ValueError(
                f"To use batch_to_device, all elements in the batch must be a dict or Tensor. Got key '{key}' with value of type {type(value)}"
            )


class DeviceSupport(Enum):
    """Device families with their display name and communication backend."""

    CPU = ("cpu", "CPU", "gloo")
    CUDA = ("cuda", "GPU", "nccl")

    def __init__(self, device_type: str, device_name: str, communication_backend: str):
        self.device_type = device_type
        self.device_name = device_name
        self.communication_backend = communication_backend

    @staticmethod
    def from_type(device_type: str) -> "DeviceSupport":
        for member in DeviceSupport:
            if member.device_type == device_type:
                return member
        raise ValueError(f"Unknown device type: {device_type}.")


def get_device_support() -> DeviceSupport:
    return DeviceSupport.from_type(_default_device_type())


def get_torch_device_namespace() -> Any:
    return torch.cuda if torch.cuda.is_available() else torch.cpu


def has_cuda_capability(major: int, minor: int) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (major, minor)


def is_sm100(device: Optional[torch.device] = None) -> bool:
    """True on Blackwell datacentre parts (compute capability 10.x)."""
    if not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability(device)[0] == 10


def is_torch_hpu_available() -> bool:
    """This build targets NVIDIA B200 only: there is no Habana path."""
    return False

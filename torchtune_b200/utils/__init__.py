from ._device import (
    DeviceSupport,
    batch_to_device,
    get_device,
    get_device_support,
    get_torch_device_namespace,
    get_world_size_and_rank,
    has_cuda_capability,
    is_sm100,
)
from ._logging import deprecated, get_logger, log_once, log_rank_zero
from ._version import torch_version_ge

__all__ = [
    "batch_to_device",
    "get_device",
    "get_logger",
    "torch_version_ge",
    "get_world_size_and_rank",
    "DeviceSupport",
    "get_device_support",
    "get_torch_device_namespace",
    "has_cuda_capability",
    "is_sm100",
    "deprecated",
    "log_once",
    "log_rank_zero",
]

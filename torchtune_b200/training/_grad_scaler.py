"""In-place gradient scaling (parity: torchtune/training/_grad_scaler.py:42-109)."""
from __future__ import annotations

from collections import defaultdict
from typing import Iterable, Optional, Union

import torch
from torch import Tensor, nn


def scale_grads_(parameters: Union[Tensor, Iterable[Tensor]], scaler: Union[Tensor, float], foreach: Optional[bool] = None) -> None:
    """Multiply every existing ``.grad`` by ``scaler`` (a float or 0-d tensor), grouped per
    device/dtype so each group is one multi-tensor launch."""
    if isinstance(parameters, Tensor):
        parameters = [parameters]
    groups = defaultdict(list)
    for p in parameters:
        if p.grad is not None:
            groups[(p.grad.device, p.grad.dtype)].append(p.grad)
    for (device, _), grads in groups.items():
        s = scaler.to(device) if isinstance(scaler, Tensor) else scaler
        if foreach is False:
            for g in grads:
                g.mul_(s)
        else:
            torch._foreach_mul_(grads, s)


def scale_grads(model: nn.Module, scaler: Tensor) -> None:
    """Deprecated spelling of :func:`scale_grads_` taking a module."""
    scale_grads_(model.parameters(), scaler)

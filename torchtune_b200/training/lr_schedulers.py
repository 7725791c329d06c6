"""Learning-rate schedules (parity: torchtune/training/lr_schedulers.py:41-122)."""
from __future__ import annotations

import math
from typing import Union

import torch
from torch.optim.lr_scheduler import LambdaLR


def get_cosine_schedule_with_warmup(
    optimizer: torch.optim.Optimizer, num_warmup_steps: int, num_training_steps: int, num_cycles: float = 0.5, last_epoch: int = -1
) -> LambdaLR:
    """Linear ramp 0→lr over ``num_warmup_steps`` then ``max(0, ½(1+cos(2π·cycles·progress)))``."""

    def factor(step: int) -> float:
        if step < num_warmup_steps:
            return step / max(1, num_warmup_steps)
        progress = (step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps)
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * progress)))

    return LambdaLR(optimizer, factor, last_epoch)


def get_lr(optimizer) -> float:
    """The single learning rate shared by all param groups (or by all in-backward optimizers)."""
    groups = []
    if hasattr(optimizer, "optim_map"):
        for opt in optimizer.optim_map.values():
            groups.extend(opt.param_groups)
    else:
        groups = optimizer.param_groups
    if not groups:
        raise RuntimeError(f"Invalid optimizer param groups with len of: {len(groups)}")
    lrs = {g["lr"] for g in groups}
    if len(lrs) != 1:
        raise RuntimeError(f"LR Scheduler doesn't support different lr values in different param groups. Found {len(lrs)} different values.")
    return groups[0]["lr"]

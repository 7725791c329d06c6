"""Loss base classes (parity: torchtune/modules/loss/loss_types.py:14-86)."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch
from torch import nn


class SFTLoss(ABC):
    """Losses that consume ``(model outputs, integer targets)``."""

    def apply_compile_strategy(self, *args, **kwargs):
        """No tracing compiler is used; kept so recipes can call it unconditionally."""
        return self

    @abstractmethod
    def set_model_output(self, model: nn.Module) -> None:
        """Give the loss access to the model's output projection."""

    def patch_tp_plan(self, tp_plan) -> dict:
        return tp_plan

    @property
    def tp_requires_loss_parallel_ctx_manager(self) -> bool:
        return False

    @abstractmethod
    def forward(self, outputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        ...


class RLLoss(ABC):
    """Losses over policy / reference log-probabilities."""

    def apply_compile_strategy(self, *args, **kwargs):
        return self

    @abstractmethod
    def forward(self, *args, **kwargs):
        ...

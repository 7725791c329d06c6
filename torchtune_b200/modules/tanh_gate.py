"""Learnable tanh gate (parity: torchtune/modules/tanh_gate.py:12-27)."""
import torch
from torch import nn


class TanhGate(nn.Module):
    """``x * tanh(scale)`` with a single scalar parameter initialised at zero."""

    def __init__(self) -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.zeros(1))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * self.scale.tanh()

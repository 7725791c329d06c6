"""RMS normalisation (parity: torchtune/modules/rms_norm.py:11-60)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * scale`` with fp32 statistics; the learnable
    parameter is called ``scale``."""

    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.normalized_shape = (dim,)
        self.eps = eps
        self.scale = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.scale, self.eps)

    def extra_repr(self) -> str:
        return f"dim={self.normalized_shape[0]}, eps={self.eps}"


def rms_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Weight-less RMS norm over the last dimension (Llama-4 q/k normalisation)."""
    return ops.rms_norm(x, None, eps)

"""Linear layer routed through :func:`torchtune_b200.ops.linear`."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


class Linear(nn.Linear):
    """Drop-in ``nn.Linear`` (same parameters / state-dict keys) whose forward, dgrad
    and wgrad run the tcgen05 GEMM for bf16 CUDA tensors."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)

"""Output projection sharing the token-embedding matrix (parity: torchtune/modules/tied_linear.py:12-64)."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


class _TiedMatmul(nn.Module):
    """Parameter-free module so that module hooks (sharding, checkpointing) have something to attach to."""

    def forward(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, weight)


class TiedLinear:
    """Callable (deliberately *not* an ``nn.Module``, so the shared weight appears once
    in the state dict) computing ``x @ tied_module.weight.T``."""

    def __init__(self, tied_module: nn.Module):
        if not hasattr(tied_module, "weight"):
            raise AttributeError("Provided module does not have attribute 'weight'. Please check your tied_module.")
        self.tied_module = tied_module
        self.linear = _TiedMatmul()

    @property
    def weight(self) -> torch.Tensor:
        return self.tied_module.weight

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear(x, self.tied_module.weight)

"""Frozen linear layer with an NF4 weight (parity: torchtune/modules/low_precision/nf4_linear.py:16-70)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .nf4 import NF4Weight, linear_nf4


class FrozenNF4Linear(nn.Module):
    """``y = x @ W.T (+ b)`` where ``W`` is stored in NF4 and never trained.  The state
    dict carries a dense ``weight`` (see :mod:`.nf4`)."""

    def __init__(
        self, in_dim: int, out_dim: int, bias: bool = False, device=None, dtype: Optional[torch.dtype] = None, **quantization_kwargs
    ):
        super().__init__()
        self.in_features, self.out_features = in_dim, out_dim
        dtype = dtype or torch.bfloat16
        self.nf4 = NF4Weight(out_dim, in_dim, dtype=dtype, device=device, **quantization_kwargs)
        init = torch.empty(out_dim, in_dim, dtype=torch.float32, device=device)
        nn.init.kaiming_uniform_(init, a=5**0.5)
        if init.device.type != "meta":
            self.nf4.quantize_(init)
        self.bias = nn.Parameter(torch.zeros(out_dim, dtype=dtype, device=device), requires_grad=False) if bias else None

    @property
    def weight(self) -> torch.Tensor:
        return self.nf4.dequantize()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_nf4(x, self.nf4, self.bias)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        destination[prefix + "weight"] = self.nf4.dequantize()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        key = prefix + "weight"
        if key in state_dict:
            self.nf4.quantize_(state_dict.pop(key))
        elif strict:
            missing_keys.append(key)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

"""LayerNorm evaluated in fp32 (parity: torchtune/modules/layer_norm.py:14-37)."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


class Fp32LayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = None if self.weight is None else self.weight.float()
        b = None if self.bias is None else self.bias.float()
        return F.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).type_as(x)

"""Gated feed-forward block (parity: torchtune/modules/feed_forward.py:14-54)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops


class FeedForward(nn.Module):
    """``down(act(gate(x)) * up(x))``; attribute names are ``w1`` (gate), ``w2``
    (down) and ``w3`` (up).  With SiLU and an up projection the activation and
    product run as one fused SwiGLU kernel."""

    def __init__(
        self,
        *,
        gate_proj: nn.Module,
        down_proj: nn.Module,
        up_proj: Optional[nn.Module] = None,
        activation: nn.Module = nn.SiLU(),
    ):
        super().__init__()
        self.w1 = gate_proj
        self.w2 = down_proj
        self.w3 = up_proj
        self.activation = activation
        self._silu = isinstance(activation, nn.SiLU)

    def _fusable(self) -> bool:
        """Plain bias-free bf16 linears on both sides of a SiLU gate: the gate / up projections and the activation run as one GEMM."""
        lin = (type(self.w1), type(self.w3))
        return self._silu and all(t.__name__ == "Linear" and issubclass(t, nn.Linear) for t in lin) and self.w1.bias is None and self.w3.bias is None

    def _down(self, h: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        """Down projection; with ``residual`` the block's input stream is added in the projection's GEMM epilogue."""
        if residual is None:
            return self.w2(h)
        if type(self.w2) is nn.Linear:
            return ops.linear_residual(h, self.w2.weight, self.w2.bias, residual)
        return self.w2(h) + residual

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual``: a tensor of the output's shape that is added to the result (a decoder layer passes its residual stream)."""
        if self.w3 is not None and ops.cuda_ops_enabled(x) and x.dtype == torch.bfloat16 and self._fusable():
            from ..ops._cuda import gate_up_swiglu

            h = gate_up_swiglu(x, self.w1.weight, self.w3.weight)
            if h is not None:
                return self._down(h, residual)
        g = self.w1(x)
        if self.w3 is None:
            return self._down(self.activation(g), residual)
        u = self.w3(x)
        h = ops.swiglu(g, u) if self._silu else self.activation(g) * u
        return self._down(h, residual)

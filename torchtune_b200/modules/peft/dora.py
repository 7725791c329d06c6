"""Weight-decomposed LoRA (parity: torchtune/modules/peft/dora.py:21-206)."""
from __future__ import annotations

import math
from typing import List

import torch
from torch import nn

from ... import ops
from ..low_precision.nf4 import NF4Weight, linear_nf4
from .lora import _lora_a_init_params, _lora_b_init_params


class DoRALinear(nn.Module):
    """``y = m · (W + s·BA) x / ||W + s·BA||_row`` with a learnable per-output magnitude
    ``m``; the norm is treated as a constant in backward."""

    def __init__(
        self,
        in_dim: int,
        out_dim: int,
        rank: int,
        alpha: float,
        dropout: float = 0.0,
        use_bias: bool = False,
        quantize_base: bool = False,
        **quantization_kwargs,
    ):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.scaling = alpha / rank
        self.rank, self.alpha = rank, alpha
        self.use_bias = use_bias
        self._quantize_base = quantize_base
        if not quantize_base and quantization_kwargs:
            raise ValueError(f"``quantize_base`` is False, but received the following quantization arguments: {quantization_kwargs}")
        base = nn.Linear(in_dim, out_dim, bias=use_bias)
        if quantize_base:
            self.nf4 = NF4Weight(out_dim, in_dim, dtype=base.weight.dtype, device=base.weight.device, **quantization_kwargs)
            if base.weight.device.type != "meta":
                self.nf4.quantize_(base.weight.detach())
            self.register_parameter("weight", None)
        else:
            self.register_parameter("weight", nn.Parameter(base.weight.detach()))
        self.register_parameter("bias", nn.Parameter(base.bias.detach()) if use_bias else None)
        self.dropout = nn.Dropout(p=dropout) if dropout > 0.0 else nn.Identity()
        self.lora_a = nn.Linear(in_dim, rank, bias=False)
        self.lora_b = nn.Linear(rank, out_dim, bias=False)
        self.magnitude = nn.Parameter(torch.empty(out_dim))
        self.disabled = False
        self.initialize_parameters()

    def to_empty(self, *, device=None, recurse: bool = True):
        self.lora_a.to_empty(device=device, recurse=recurse)
        self.lora_b.to_empty(device=device, recurse=recurse)
        self.magnitude = nn.Parameter(torch.empty_like(self.magnitude, device=device), requires_grad=self.magnitude.requires_grad)
        return self

    def initialize_parameters(self) -> None:
        _lora_a_init_params(self.lora_a)
        _lora_b_init_params(self.lora_b)

    def base_weight(self, dtype=None) -> torch.Tensor:
        return self.nf4.dequantize(dtype) if self._quantize_base else self.weight

    @torch.no_grad()
    def initialize_dora_magnitude(self) -> None:
        """Set ``m`` to the row norms of the current merged weight; call after loading."""
        if any(t.is_meta for t in (self.lora_a.weight, self.lora_b.weight, self.magnitude)):
            raise RuntimeError("Cannot initialize DoRA magnitude if base or LoRA parameters are still on meta device.")
        w = self.base_weight(self.lora_a.weight.dtype)
        self.magnitude.copy_(self._weight_norm(w, self.lora_b.weight @ self.lora_a.weight))

    def _weight_norm(self, weight: torch.Tensor, lora_weight: torch.Tensor) -> torch.Tensor:
        return torch.linalg.norm(weight + self.scaling * lora_weight, dim=1).to(weight.dtype)

    def adapter_params(self) -> List[str]:
        return ["lora_a.weight", "lora_b.weight", "magnitude"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._quantize_base:
            base_out = linear_nf4(x, self.nf4, self.bias)
        else:
            base_out = ops.linear(x, self.weight, self.bias)
        if self.disabled:
            return base_out
        xd = self.dropout(x)
        lora_out = ops.linear(ops.linear(xd, self.lora_a.weight), self.lora_b.weight)
        w = self.base_weight(x.dtype)
        norm = self._weight_norm(w, (self.lora_b.weight @ self.lora_a.weight)).detach()
        mag_scale = (self.magnitude / norm).view(1, -1)
        # bias is not rescaled: it is excluded from the weight decomposition
        no_bias = base_out if self.bias is None else base_out - self.bias
        dora = (mag_scale - 1) * no_bias + mag_scale * lora_out * self.scaling
        return dora + base_out

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        if self._quantize_base:
            destination[prefix + "weight"] = self.nf4.dequantize()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        if self._quantize_base:
            key = prefix + "weight"
            if key in state_dict:
                self.nf4.quantize_(state_dict.pop(key))
            elif strict:
                missing_keys.append(key)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

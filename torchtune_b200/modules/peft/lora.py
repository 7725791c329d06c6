"""LoRA linear layers (parity: torchtune/modules/peft/lora.py:27-320)."""
from __future__ import annotations

from enum import Enum

import math
from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ..low_precision.nf4 import NF4Weight, linear_nf4


class TrainableParams(Enum):
    """How a model part is trained by the LoRA builders: every weight, adapters only, or nothing."""

    FULL = "full"
    LORA = "lora"
    FROZEN = "frozen"


class LoRALinear(nn.Module):
    """``y = x W^T (+ b) + (alpha / rank) · B(A(dropout(x)))``.

    Parameters: ``weight`` ``[out, in]`` (frozen; NF4 when ``quantize_base``), optional
    ``bias``, ``lora_a.weight`` ``[rank, in]`` (Kaiming-uniform, a=√5) and
    ``lora_b.weight`` ``[out, rank]`` (zeros, so the initial output equals the base).
    ``disabled=True`` skips the adapter branch (reference pass of DPO).
    """

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
        self.rank = rank
        self.alpha = alpha
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.use_bias = use_bias
        self._quantize_base = quantize_base
        if not quantize_base and quantization_kwargs:
            raise ValueError(f"``quantize_base`` is False, but received the following quantization arguments: {quantization_kwargs}")
        base = nn.Linear(in_dim, out_dim, bias=use_bias)
        if quantize_base:
            if use_bias:
                raise NotImplementedError("quantized base weights do not support a bias")
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
        self.merged = False
        self.disabled = False
        self.initialize_parameters()

    def to_empty(self, *, device=None, recurse: bool = True):
        self.lora_a.to_empty(device=device, recurse=recurse)
        self.lora_b.to_empty(device=device, recurse=recurse)
        return self

    def initialize_parameters(self) -> None:
        _lora_a_init_params(self.lora_a)
        _lora_b_init_params(self.lora_b)

    def adapter_params(self) -> List[str]:
        return ["lora_a.weight", "lora_b.weight"]

    def base_weight(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if self._quantize_base:
            return self.nf4.dequantize(dtype)
        return self.weight

    def _base_forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._quantize_base:
            return linear_nf4(x, self.nf4, self.bias)
        return ops.linear(x, self.weight, self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.disabled:
            return self._base_forward(x)
        if not self._quantize_base and type(self)._base_forward is LoRALinear._base_forward:
            # dense base: one fused call (adapter product accumulated by the GEMM epilogue on CUDA)
            return ops.lora_linear(x, self.dropout(x), self.weight, self.bias, self.lora_a.weight, self.lora_b.weight, self.alpha / self.rank)
        if self._quantize_base and type(self)._base_forward is LoRALinear._base_forward:
            fused = ops.lora_linear_nf4(x, self.dropout(x), self.nf4, self.bias, self.lora_a.weight, self.lora_b.weight, self.alpha / self.rank)
            if fused is not None:
                return fused
        out = self._base_forward(x)
        a = ops.linear(self.dropout(x), self.lora_a.weight)
        return out + (self.alpha / self.rank) * ops.linear(a, self.lora_b.weight)

    # dense-weight state-dict view for the NF4 case
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


def _lora_a_init_params(x: nn.Linear) -> None:
    if x.weight.device.type != "meta":
        nn.init.kaiming_uniform_(x.weight, a=math.sqrt(5))


def _lora_b_init_params(x: nn.Linear) -> None:
    if x.weight.device.type != "meta":
        nn.init.zeros_(x.weight)


class _FakeQuant(nn.Module):
    """Symmetric/asymmetric per-group or per-token fake quantiser with a straight-through
    gradient; the owned counterpart of the external QAT fake quantiser used at
    torchtune/modules/peft/lora.py:150-306."""

    def __init__(self, bits: int, group_size: Optional[int], symmetric: bool, per_token: bool = False):
        super().__init__()
        self.bits, self.group_size, self.symmetric, self.per_token = bits, group_size, symmetric, per_token
        self.enabled = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.enabled:
            return x
        shape = x.shape
        g = x.shape[-1] if (self.per_token or not self.group_size) else self.group_size
        xf = x.float().reshape(-1, g)
        if self.symmetric:
            qmax = 2 ** (self.bits - 1) - 1
            scale = xf.abs().amax(-1, keepdim=True).clamp_min(1e-9) / qmax
            q = torch.clamp(torch.round(xf / scale), -qmax - 1, qmax) * scale
        else:
            qmax = 2**self.bits - 1
            lo, hi = xf.amin(-1, keepdim=True).clamp_max(0), xf.amax(-1, keepdim=True).clamp_min(0)
            scale = ((hi - lo) / qmax).clamp_min(1e-9)
            zp = torch.round(-lo / scale)
            q = (torch.clamp(torch.round(xf / scale) + zp, 0, qmax) - zp) * scale
        q = q.reshape(shape).to(x.dtype)
        return x + (q - x).detach()


class QATLoRALinear(LoRALinear):
    """LoRA layer whose base matmul sees fake-quantised activations and weights
    (e.g. int8 per-token activations + int4 grouped weights), adapters in full precision."""

    def __init__(
        self,
        in_dim: int,
        out_dim: int,
        rank: int,
        alpha: float,
        dropout: float = 0.0,
        activation_qat_config=None,
        weight_qat_config=None,
    ):
        super().__init__(in_dim, out_dim, rank, alpha, dropout, use_bias=False, quantize_base=False)
        self.activation_fake_quantizer = _make_fq(activation_qat_config, activation=True)
        self.weight_fake_quantizer = _make_fq(weight_qat_config, activation=False)

    @classmethod
    def from_lora_linear(cls, lora_linear: LoRALinear, activation_qat_config=None, weight_qat_config=None) -> "QATLoRALinear":
        if lora_linear.bias is not None:
            raise ValueError("Bias is not supported in QAT + LoRA yet")
        if lora_linear._quantize_base:
            raise ValueError("quantize_base is not compatible with QAT + LoRA")
        p = lora_linear.dropout.p if isinstance(lora_linear.dropout, nn.Dropout) else 0.0
        with torch.device(lora_linear.weight.device if lora_linear.weight.device.type == "meta" else "cpu"):
            new = cls(lora_linear.in_dim, lora_linear.out_dim, lora_linear.rank, lora_linear.alpha, p, activation_qat_config, weight_qat_config)
        new.weight = lora_linear.weight
        new.lora_a.weight = lora_linear.lora_a.weight
        new.lora_b.weight = lora_linear.lora_b.weight
        return new

    def _base_forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(self.activation_fake_quantizer(x), self.weight_fake_quantizer(self.weight))


def _make_fq(cfg, activation: bool) -> nn.Module:
    if cfg is None:
        return nn.Identity()
    bits = int(getattr(cfg, "bits", None) or (8 if activation else 4))
    group = getattr(cfg, "group_size", None)
    symmetric = bool(getattr(cfg, "is_symmetric", not activation))
    return _FakeQuant(bits, group, symmetric, per_token=activation and group is None)

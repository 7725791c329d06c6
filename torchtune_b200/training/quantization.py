"""Post-training quantisation, quantisation-aware training and fp8 training switches
(parity: torchtune/training/quantization.py:51-320; the reference delegates the quantisers
to an external library, here they are implemented in the package).

Schemes:

``8da4w``  int8 per-token dynamic (asymmetric) activations × int4 per-group symmetric weights
``4w``     int4 per-group weights, activations untouched

Each scheme has a post-training quantiser (``quantize(model)``) and a QAT quantiser
(``prepare(model)`` inserts fake quantisation with straight-through gradients, ``convert(model)``
replaces it by the real quantised layer).  Quantised weights are stored two nibbles per byte
with one fp scale (and zero point for ``4w``) per group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..modules.peft.lora import LoRALinear, QATLoRALinear, _FakeQuant


@dataclass
class FakeQuantizeConfig:
    """``bits`` wide integers; one scale per ``group_size`` input features, or per token when
    ``group_size`` is ``None``; symmetric (signed, no zero point) or asymmetric."""

    bits: int = 4
    group_size: Optional[int] = None
    is_symmetric: bool = True
    dtype: Optional[torch.dtype] = None

    def __post_init__(self):
        if self.dtype in (torch.int4, getattr(torch, "int4", None)):
            self.bits = 4
        elif self.dtype == torch.int8:
            self.bits = 8


# ------------------------------------------------------------------------------ packing
def _quantize_int4_groupwise(w: torch.Tensor, group_size: int, symmetric: bool):
    out_f, in_f = w.shape
    if in_f % group_size:
        raise ValueError(f"in_features ({in_f}) must be divisible by the group size ({group_size})")
    g = w.float().reshape(out_f, in_f // group_size, group_size)
    if symmetric:
        scale = g.abs().amax(-1, keepdim=True).clamp_min(1e-9) / 7.0
        q = torch.clamp(torch.round(g / scale), -8, 7)
        zero = torch.zeros_like(scale)
        stored = (q + 8).to(torch.uint8)
    else:
        lo, hi = g.amin(-1, keepdim=True).clamp_max(0), g.amax(-1, keepdim=True).clamp_min(0)
        scale = ((hi - lo) / 15.0).clamp_min(1e-9)
        zero = torch.round(-lo / scale)
        stored = torch.clamp(torch.round(g / scale) + zero, 0, 15).to(torch.uint8)
    stored = stored.reshape(out_f, in_f)
    packed = (stored[:, 0::2] << 4) | stored[:, 1::2]
    return packed.contiguous(), scale.squeeze(-1).contiguous(), zero.squeeze(-1).contiguous()


def _dequantize_int4_groupwise(packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, group_size: int, symmetric: bool, dtype: torch.dtype) -> torch.Tensor:
    out_f = packed.shape[0]
    stored = torch.stack([(packed >> 4) & 0xF, packed & 0xF], dim=-1).reshape(out_f, -1).float()
    g = stored.reshape(out_f, -1, group_size)
    off = 8.0 if symmetric else zero.unsqueeze(-1)
    return ((g - off) * scale.unsqueeze(-1)).reshape(out_f, -1).to(dtype)


class Int4WeightLinear(nn.Module):
    """Linear layer with packed int4 weights; ``dynamic_int8_activations`` adds per-token
    asymmetric int8 activation quantisation (the ``8da4w`` scheme)."""

    def __init__(self, in_features: int, out_features: int, group_size: int, symmetric: bool, dynamic_int8_activations: bool, dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        self.in_features, self.out_features, self.group_size = in_features, out_features, group_size
        self.symmetric, self.dynamic_int8_activations, self.compute_dtype = symmetric, dynamic_int8_activations, dtype
        n_groups = in_features // group_size
        self.register_buffer("weight_packed", torch.zeros(out_features, in_features // 2, dtype=torch.uint8, device=device))
        self.register_buffer("scales", torch.zeros(out_features, n_groups, dtype=torch.float32, device=device))
        self.register_buffer("zeros", torch.zeros(out_features, n_groups, dtype=torch.float32, device=device))

    @classmethod
    def from_float(cls, weight: torch.Tensor, group_size: int, symmetric: bool, dynamic_int8_activations: bool) -> "Int4WeightLinear":
        mod = cls(weight.shape[1], weight.shape[0], group_size, symmetric, dynamic_int8_activations, dtype=weight.dtype, device=weight.device)
        packed, scale, zero = _quantize_int4_groupwise(weight.detach(), group_size, symmetric)
        mod.weight_packed.copy_(packed)
        mod.scales.copy_(scale)
        mod.zeros.copy_(zero)
        return mod

    def dequantized_weight(self) -> torch.Tensor:
        return _dequantize_int4_groupwise(self.weight_packed, self.scales, self.zeros, self.group_size, self.symmetric, self.compute_dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.dynamic_int8_activations:
            x = _int8_per_token(x)
        return F.linear(x, self.dequantized_weight().to(x.dtype))


_ACT_FQ = _FakeQuant(8, None, symmetric=False, per_token=True)


def _int8_per_token(x: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return _ACT_FQ(x)


class FakeQuantizedLinear(nn.Linear):
    """``nn.Linear`` whose forward sees fake-quantised activations and/or weights (QAT)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, activation_config: Optional[FakeQuantizeConfig] = None, weight_config: Optional[FakeQuantizeConfig] = None, **kw):
        super().__init__(in_features, out_features, bias, **kw)
        self.activation_fake_quantizer = _build_fq(activation_config, activation=True)
        self.weight_fake_quantizer = _build_fq(weight_config, activation=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.activation_fake_quantizer is not None:
            x = self.activation_fake_quantizer(x)
        w = self.weight if self.weight_fake_quantizer is None else self.weight_fake_quantizer(self.weight)
        from .. import ops

        return ops.linear(x, w, self.bias)

    @classmethod
    def from_linear(cls, lin: nn.Module, activation_config, weight_config) -> "FakeQuantizedLinear":
        has_bias = getattr(lin, "bias", None) is not None
        with torch.device("meta"):
            new = cls(lin.in_features, lin.out_features, has_bias, activation_config, weight_config)
        new.weight = lin.weight
        if has_bias:
            new.bias = lin.bias
        return new

    def to_linear(self) -> nn.Linear:
        from ..modules import Linear

        with torch.device("meta"):
            new = Linear(self.in_features, self.out_features, self.bias is not None)
        new.weight = self.weight
        if self.bias is not None:
            new.bias = self.bias
        return new


def _build_fq(cfg: Optional[FakeQuantizeConfig], activation: bool) -> Optional[_FakeQuant]:
    if cfg is None:
        return None
    return _FakeQuant(cfg.bits, cfg.group_size, cfg.is_symmetric, per_token=cfg.group_size is None)


def _is_plain_linear(m: nn.Module) -> bool:
    return isinstance(m, nn.Linear) and not isinstance(m, FakeQuantizedLinear) and type(m).__name__ in ("Linear",)


def _swap(model: nn.Module, predicate: Callable[[nn.Module, str], bool], factory: Callable[[nn.Module], nn.Module], prefix: str = "") -> nn.Module:
    for name, child in list(model.named_children()):
        fqn = f"{prefix}.{name}" if prefix else name
        if predicate(child, fqn):
            setattr(model, name, factory(child))
        else:
            _swap(child, predicate, factory, fqn)
    return model


# ------------------------------------------------------------------------------ quantisers
class _PTQ:
    mode = ""
    symmetric = True
    dynamic_act = False

    def __init__(self, groupsize: int = 256, **_: object):
        self.groupsize = groupsize

    def _eligible(self, m: nn.Module, fqn: str) -> bool:
        return _is_plain_linear(m) and m.bias is None and m.in_features % self.groupsize == 0

    def quantize(self, model: nn.Module) -> nn.Module:
        return _swap(model, self._eligible, lambda lin: Int4WeightLinear.from_float(lin.weight, self.groupsize, self.symmetric, self.dynamic_act))


class Int8DynActInt4WeightQuantizer(_PTQ):
    """Post-training ``8da4w``."""

    mode, symmetric, dynamic_act = "8da4w", True, True


class Int4WeightOnlyQuantizer(_PTQ):
    """Post-training ``4w`` (asymmetric int4 groups, activations in bf16)."""

    mode, symmetric, dynamic_act = "4w", False, False

    def __init__(self, groupsize: int = 128, inner_k_tiles: int = 8, **kw: object):
        super().__init__(groupsize)
        self.inner_k_tiles = inner_k_tiles


class _QAT(_PTQ):
    def _configs(self):
        act = FakeQuantizeConfig(bits=8, group_size=None, is_symmetric=False) if self.dynamic_act else None
        return act, FakeQuantizeConfig(bits=4, group_size=self.groupsize, is_symmetric=self.symmetric)

    def prepare(self, model: nn.Module) -> nn.Module:
        act, wt = self._configs()
        return _swap(model, self._eligible, lambda lin: FakeQuantizedLinear.from_linear(lin, act, wt))

    def convert(self, model: nn.Module) -> nn.Module:
        return _swap(
            model,
            lambda m, fqn: isinstance(m, FakeQuantizedLinear),
            lambda fq: Int4WeightLinear.from_float(fq.weight, self.groupsize, self.symmetric, self.dynamic_act),
        )


class Int8DynActInt4WeightQATQuantizer(_QAT):
    mode, symmetric, dynamic_act = "8da4w-qat", True, True


class Int4WeightOnlyQATQuantizer(_QAT):
    mode, symmetric, dynamic_act = "4w-qat", False, False

    def __init__(self, groupsize: int = 128, inner_k_tiles: int = 8, **kw: object):
        super().__init__(groupsize)
        self.inner_k_tiles = inner_k_tiles


class Int8DynActInt4WeightQATQuantizerModuleSwap(Int8DynActInt4WeightQATQuantizer):
    mode = "8da4w-qat-module-swap"


class Int4WeightOnlyQATQuantizerModuleSwap(Int4WeightOnlyQATQuantizer):
    mode = "4w-qat-module-swap"


def _set_fake_quant(mod: nn.Module, enabled: bool) -> None:
    if isinstance(mod, (FakeQuantizedLinear, QATLoRALinear)):
        for fq in (getattr(mod, "activation_fake_quantizer", None), getattr(mod, "weight_fake_quantizer", None)):
            if isinstance(fq, _FakeQuant):
                fq.enabled = enabled


def enable_fake_quant(mod: nn.Module) -> None:
    """For ``model.apply``: switch fake quantisation on in every QAT layer."""
    _set_fake_quant(mod, True)


def disable_fake_quant(mod: nn.Module) -> None:
    """For ``model.apply``: switch fake quantisation off (used for the first
    ``fake_quant_after_n_steps`` steps of QAT)."""
    _set_fake_quant(mod, False)


_QUANTIZERS = (
    Int8DynActInt4WeightQuantizer,
    Int4WeightOnlyQuantizer,
    Int8DynActInt4WeightQATQuantizer,
    Int4WeightOnlyQATQuantizer,
    Int8DynActInt4WeightQATQuantizerModuleSwap,
    Int4WeightOnlyQATQuantizerModuleSwap,
)
_quantizer_to_mode: Dict[type, str] = {q: q.mode for q in _QUANTIZERS}
_quantizer_mode_to_disable_fake_quant = {m: disable_fake_quant for m in _quantizer_to_mode.values() if "qat" in m}
_quantizer_mode_to_enable_fake_quant = {m: enable_fake_quant for m in _quantizer_to_mode.values() if "qat" in m}


def get_quantizer_mode(quantizer: Optional[object]) -> Optional[str]:
    """``'8da4w'``, ``'4w'``, ``'8da4w-qat'`` … or ``None`` for an unknown object."""
    return _quantizer_to_mode.get(type(quantizer))


def _get_disable_fake_quant(quantizer_mode: str) -> Optional[Callable]:
    return _quantizer_mode_to_disable_fake_quant.get(quantizer_mode)


def _get_enable_fake_quant(quantizer_mode: str) -> Optional[Callable]:
    return _quantizer_mode_to_enable_fake_quant.get(quantizer_mode)


def swap_lora_linear_with_qat(module: nn.Module, activation_qat_config: Optional[FakeQuantizeConfig] = None, weight_qat_config: Optional[FakeQuantizeConfig] = None) -> None:
    """Replace every :class:`LoRALinear` below ``module`` by a :class:`QATLoRALinear` sharing its parameters."""
    _swap(module, lambda m, fqn: type(m) is LoRALinear, lambda m: QATLoRALinear.from_lora_linear(m, activation_qat_config, weight_qat_config))


# ------------------------------------------------------------------------------ fp8 training
def is_fp8_tensorwise_scaling(fp8_recipe_name: Optional[str]) -> bool:
    return fp8_recipe_name is None or fp8_recipe_name == "tensorwise"


class Float8Linear(nn.Linear):
    """Linear with dynamically scaled fp8 operands: one scale per tensor (``tensorwise``), per row (``rowwise``), or per block of 32
    values along each contraction dimension (``blockwise``: the MX format, scales applied inside the tensor core by
    ``tcgen05.mma.kind::mxf8f6f4.block_scale``).

    bf16 CUDA inputs run on the fp8 tensor cores (``ops.fp8_linear``: cast+transpose kernel, tcgen05 ``kind::f8f6f4`` GEMM for
    forward, input gradient and weight gradient; e5m2 output gradients with tensorwise scaling).  Elsewhere the forward
    quantise→dequantise round trip is emulated around the ordinary matmul with straight-through gradients."""

    recipe = "tensorwise"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops

        if self.recipe == "blockwise":
            y = ops.mxfp8_linear(x, self.weight, self.bias)
            if y is not None:
                return y
            from ..ops import reference

            if x.shape[-1] % reference.MX_BLOCK:
                return ops.linear(x, self.weight, self.bias)
            x2 = x.reshape(-1, x.shape[-1])
            xq = x + (reference.mx_roundtrip(x2).view_as(x).to(x.dtype) - x).detach()
            wq = self.weight + (reference.mx_roundtrip(self.weight).to(self.weight.dtype) - self.weight).detach()
            return ops.linear(xq, wq, self.bias)
        y = ops.fp8_linear(x, self.weight, self.bias, rowwise=self.recipe != "tensorwise")
        if y is not None:
            return y
        dims = None if self.recipe == "tensorwise" else -1
        xq = _fp8_roundtrip(x, dims)
        wq = _fp8_roundtrip(self.weight, dims)
        from .. import ops

        return ops.linear(xq, wq, self.bias)


def _fp8_roundtrip(t: torch.Tensor, dim: Optional[int]) -> torch.Tensor:
    fmax = torch.finfo(torch.float8_e4m3fn).max
    amax = t.detach().abs().amax() if dim is None else t.detach().abs().amax(dim=dim, keepdim=True)
    scale = fmax / amax.float().clamp_min(1e-12)
    q = (t.detach().float() * scale).clamp(-fmax, fmax).to(torch.float8_e4m3fn).float() / scale
    return t + (q.to(t.dtype) - t).detach()


def convert_to_float8_training(model: nn.Module, fp8_recipe_name: Optional[str] = None) -> nn.Module:
    """Swap every linear layer except the final vocabulary projection (and layers whose
    dimensions are not multiples of 16) for :class:`Float8Linear`."""
    recipe = fp8_recipe_name or "tensorwise"
    if recipe in ("mxfp8", "mx"):
        recipe = "blockwise"
    if recipe not in ("tensorwise", "rowwise", "rowwise_with_gw_hp", "blockwise"):
        raise ValueError(f"unknown fp8 recipe {recipe!r}")

    def eligible(m: nn.Module, fqn: str) -> bool:
        mult = 32 if recipe == "blockwise" else 16
        return _is_plain_linear(m) and fqn != "output" and not fqn.endswith(".output") and m.in_features % mult == 0 and m.out_features % mult == 0

    def make(lin: nn.Linear) -> Float8Linear:
        with torch.device("meta"):
            new = Float8Linear(lin.in_features, lin.out_features, lin.bias is not None)
        new.weight = lin.weight
        if lin.bias is not None:
            new.bias = lin.bias
        new.recipe = recipe if recipe in ("tensorwise", "blockwise") else "rowwise"
        return new

    return _swap(model, eligible, make)


def _validate_float8_tp_plan(tp_plan: Optional[dict], fp8_recipe_name: Optional[str] = None) -> None:
    if tp_plan is None or is_fp8_tensorwise_scaling(fp8_recipe_name):
        return
    raise ValueError("fp8 training with tensor parallelism supports only tensorwise scaling")


__all__ = [
    "FakeQuantizeConfig",
    "FakeQuantizedLinear",
    "Float8Linear",
    "Int4WeightLinear",
    "Int4WeightOnlyQATQuantizer",
    "Int4WeightOnlyQATQuantizerModuleSwap",
    "Int4WeightOnlyQuantizer",
    "Int8DynActInt4WeightQATQuantizer",
    "Int8DynActInt4WeightQATQuantizerModuleSwap",
    "Int8DynActInt4WeightQuantizer",
    "convert_to_float8_training",
    "disable_fake_quant",
    "enable_fake_quant",
    "get_quantizer_mode",
    "is_fp8_tensorwise_scaling",
    "swap_lora_linear_with_qat",
]

"""Stochastic depth over batch rows (parity: torchtune/modules/layer_dropout.py:16-300;
arXiv 1603.09382, LayerSkip arXiv 2404.16710).

:class:`LayerDropout` runs a function only on the rows of the batch that survive a Bernoulli draw and
passes the other rows through unchanged; :func:`prepare_layer_dropout` wraps the layers of a model with
probabilities that grow with depth according to a :class:`ScaleType`."""
from __future__ import annotations

import math
from enum import Enum
from typing import Any, Callable, Iterable, Optional, Union

import torch
from torch import nn

from .common_utils import slice_str_to_array


class LayerDropout(nn.Module):
    def __init__(self, prob: float = 0.0, dim: Optional[int] = 0, disable_on_eval: Optional[bool] = True, seed: Optional[int] = None):
        super().__init__()
        self.prob, self.dim, self.disable_on_eval = prob, dim, disable_on_eval
        self.generator = torch.Generator(device="cpu")
        self.inferred: Optional[float] = None  # fraction of rows that went through the function last time
        if seed is not None:
            self.generator.manual_seed(seed)

    def forward(self, function: Union[Callable, nn.Module], input: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        if self.prob == 0 or (self.disable_on_eval and not self.training):
            self.inferred = 1.0
            return function(input, *args, **kwargs)
        assert self.dim == 0, "Currently only supporting dropping elements along the 0th dimension"
        n = input.shape[0]
        skip = torch.bernoulli(torch.full((n,), float(self.prob)), generator=self.generator).bool()
        self.inferred = 1.0 - skip.float().mean().item()
        keep = (~skip).nonzero().flatten().to(input.device)
        out = input.clone()
        if keep.numel() > 0:
            out[keep] = function(input.index_select(0, keep), *args, **kwargs).to(out.dtype)
        return out


class ModuleLayerDropoutWrapper(nn.Module):
    """Applies :class:`LayerDropout` around ``module`` while staying transparent: the wrapper shares the wrapped
    module's parameter / buffer / sub-module tables, so state-dict keys, attribute access and indexing are those of the
    wrapped module (no ``module.`` prefix appears in checkpoints)."""

    def __init__(self, module: nn.Module, dropout: LayerDropout):
        super().__init__()
        self.__dict__["module"] = module
        self.__dict__["dropout"] = dropout
        self._modules = module._modules
        self._parameters = module._parameters
        self._buffers = module._buffers

    def train(self, mode: bool = True):
        self.__dict__["dropout"].train(mode)
        self.__dict__["module"].train(mode)
        return super().train(mode)

    def forward(self, input: torch.Tensor, *args: Any, **kwargs: Any):
        return self.__dict__["dropout"](self.__dict__["module"], input, *args, **kwargs)

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.__dict__["module"], name)

    def __getitem__(self, key: int) -> Any:
        return self.__dict__["module"][key]


class ScaleType(str, Enum):
    UNIFORM = "uniform"
    EXP = "exp"
    LINEAR = "linear"
    LOG = "log"
    SIN = "sin"
    SIGMOID = "sigmoid"
    STEP = "step"


def get_scale(scale_type: ScaleType, scale_period: int, val: int) -> float:
    """Value in ``[0, 1]`` that rises from 0 at ``val = 0`` to 1 at ``val >= scale_period`` along the chosen curve."""
    if scale_period == 0 or val >= scale_period:
        return 1.0
    t = val / scale_period
    curves = {
        ScaleType.UNIFORM: lambda: 1.0,
        ScaleType.EXP: lambda: math.pow(2, t) - 1,
        ScaleType.LINEAR: lambda: t,
        ScaleType.LOG: lambda: math.log(val + 1, scale_period + 1),
        ScaleType.SIN: lambda: math.sin(0.5 * math.pi * t),
        ScaleType.SIGMOID: lambda: 1 / (1 + math.exp(-10 * (t - 0.5))),
    }
    return max(min(curves[ScaleType(scale_type)](), 1.0), 0.0)


def prepare_layer_dropout(layers: Union[nn.ModuleList, Iterable[nn.Module]], prob_max: float = 0.0, prob_layer_scale: Optional[ScaleType] = ScaleType.UNIFORM, layers_str: Optional[str] = None, disable_on_eval: Optional[bool] = True) -> None:
    """Wrap ``layers[i]`` in place with dropout probability ``prob_max · scale(i)``; ``layers_str`` (slice syntax, e.g.
    ``"0:8:2,10"``) restricts which layers get any dropout."""
    n = len(layers)
    selected = slice_str_to_array(layers_str, n) if layers_str else [True] * n
    for i in range(n):
        prob = prob_max * get_scale(prob_layer_scale, n - 1, i) if selected[i] else 0.0
        assert 0.0 <= prob <= prob_max, f"prob={prob} should be between 0 and {prob_max}"
        layers[i] = ModuleLayerDropoutWrapper(layers[i], LayerDropout(prob, disable_on_eval=disable_on_eval, seed=i))

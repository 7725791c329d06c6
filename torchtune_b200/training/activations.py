"""Selective activation checkpointing under the module path the reference uses (torchtune/training/activations.py:19-88); the
implementation lives in :mod:`torchtune_b200.training.memory`."""
from __future__ import annotations

from typing import Union

from torch import nn

from .memory import CheckpointedLayer, apply_selective_activation_checkpointing

__all__ = ["apply_selective_activation_checkpointing", "checkpoint_wrapper"]


def checkpoint_wrapper(module: nn.Module, ac_mode: str, ac_style: Union[int, str]) -> nn.Module:
    """Wrap one module for recomputation in backward.  ``ac_mode='full'`` always wraps; ``'selective'`` with an integer
    ``ac_style=k`` wraps every k-th module this function is called on (a counter kept on the function, as callers walk the
    layers in order); an operator-level ``ac_style='op'`` policy has no counterpart here — the fused kernels leave no
    cheap-to-keep intermediate results to select — and falls back to wrapping the module."""
    if ac_mode not in ("full", "selective"):
        raise ValueError(f"Invalid AC mode: {ac_mode}. Valid modes: full, selective")
    if ac_mode == "full" or ac_style == "op":
        return CheckpointedLayer(module)
    every = int(ac_style)
    if every <= 0:
        raise ValueError(f"Selective layer AC expects a positive int as selective_ac_option but got {every}")
    checkpoint_wrapper._count = getattr(checkpoint_wrapper, "_count", 0) + 1
    return CheckpointedLayer(module) if every == 1 or checkpoint_wrapper._count % every == 0 else module

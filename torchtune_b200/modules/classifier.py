"""Sequence-classifier head swap (parity: torchtune/modules/classifier.py:15-53)."""
from __future__ import annotations

from typing import Any, Callable, Union

from torch import nn

from .linear import Linear
from .transformer import TransformerDecoder


def classifier_model(num_classes: int, base_model_path: Union[str, Callable], **base_model_kwargs: Any) -> TransformerDecoder:
    """Build ``base_model_path(**kwargs)`` and replace ``output`` by ``Linear(dim, num_classes)``
    (reward / value models)."""
    from ..config._resolve import get_component_from_path

    builder = get_component_from_path(base_model_path) if isinstance(base_model_path, str) else base_model_path
    model = builder(**base_model_kwargs)
    if hasattr(model, "output"):
        dim = model.output.weight.shape[1]
        model.output = Linear(dim, num_classes, bias=False)
    elif hasattr(model, "decoder") and hasattr(model.decoder, "output"):
        dim = model.decoder.output.weight.shape[1]
        model.decoder.output = Linear(dim, num_classes, bias=False)
    else:
        raise ValueError("Could not find an output layer to adapt.")
    return model

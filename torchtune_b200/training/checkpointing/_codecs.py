"""Registry mapping a :class:`ModelType` to its HF ↔ native weight converters.

The reference selects converters with an if/elif ladder inside the checkpointer
(torchtune/training/checkpointing/_checkpointer.py:609-717, :792-876); here each family
registers a pair of callables taking ``(state_dict, hf_config)``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Tuple

import torch

from ...models import convert_weights
from ._utils import ModelType

Converter = Callable[[Dict[str, torch.Tensor], Dict[str, Any]], Dict[str, torch.Tensor]]
_HF_CODECS: Dict[ModelType, Tuple[Converter, Converter]] = {}


def register_hf_codec(model_type: ModelType, to_native: Converter, from_native: Converter) -> None:
    _HF_CODECS[model_type] = (to_native, from_native)


def _text_cfg(cfg: Dict[str, Any]) -> Dict[str, Any]:
    return cfg.get("text_config", cfg)


def _llama_args(cfg: Dict[str, Any]) -> Dict[str, Any]:
    c = _text_cfg(cfg)
    return dict(
        num_heads=c["num_attention_heads"],
        num_kv_heads=c.get("num_key_value_heads", c["num_attention_heads"]),
        dim=c["hidden_size"],
        head_dim=c.get("head_dim", None),
    )


def _generic_to_native(sd, cfg):
    return convert_weights.hf_to_tune(sd, **_llama_args(cfg))


def _generic_from_native(sd, cfg):
    return convert_weights.tune_to_hf(sd, **_llama_args(cfg))


def hf_codec(model_type: ModelType) -> Tuple[Converter, Converter]:
    if model_type not in _HF_CODECS:
        _load_family_codecs()
    return _HF_CODECS.get(model_type, (_generic_to_native, _generic_from_native))


def _load_family_codecs() -> None:
    """Import family converter modules that exist; each registers itself on import."""
    import importlib

    for mod in (
        "phi3._convert_weights",
        "qwen2._convert_weights",
        "qwen3._convert_weights",
        "gemma2._convert_weights",
        "llama4._convert_weights",
        "llama3_2_vision._convert_weights",
        "clip._convert_weights",
        "t5._convert_weights",
    ):
        try:
            importlib.import_module(f"torchtune_b200.models.{mod}")
        except ImportError:
            pass
    try:
        importlib.import_module("torchtune_b200.rlhf.utils._convert_weights")
    except ImportError:
        pass

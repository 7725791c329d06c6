"""Helpers that turn a table of size presets into the public builder functions of a
model family (``<name>()``, ``lora_<name>(...)``, ``qlora_<name>(...)``).

The reference writes each of these by hand (e.g.
torchtune/models/llama3_1/_model_builders.py:20-330); generating them from a table keeps
the public names and signatures while holding every preset in one place.
"""
from __future__ import annotations

import functools
from typing import Any, Callable, Dict, List, Optional

from ..modules import TransformerDecoder


def preset(component: Callable[..., TransformerDecoder], name: str, doc: str, exposed: Optional[Dict[str, Any]] = None, **fixed: Any):
    """Full-model builder ``name(**exposed)`` calling ``component(**fixed, **exposed)``."""
    exposed = dict(exposed or {})

    def builder(**kwargs: Any) -> TransformerDecoder:
        unknown = set(kwargs) - set(exposed)
        if unknown:
            raise TypeError(f"{name}() got unexpected keyword arguments {sorted(unknown)}")
        return component(**{**fixed, **exposed, **kwargs})

    builder.__name__ = builder.__qualname__ = name
    builder.__doc__ = doc
    _set_signature(builder, exposed)
    return builder


def lora_preset(lora_component: Callable[..., TransformerDecoder], name: str, doc: str, exposed: Optional[Dict[str, Any]] = None, **fixed: Any):
    """LoRA builder with the standard adapter keyword arguments."""
    exposed = dict(exposed or {})

    def builder(
        lora_attn_modules: List[str],
        apply_lora_to_mlp: bool = False,
        apply_lora_to_output: bool = False,
        lora_rank: int = 8,
        lora_alpha: float = 16,
        lora_dropout: float = 0.0,
        use_dora: bool = False,
        quantize_base: bool = False,
        **kwargs: Any,
    ) -> TransformerDecoder:
        unknown = set(kwargs) - set(exposed)
        if unknown:
            raise TypeError(f"{name}() got unexpected keyword arguments {sorted(unknown)}")
        return lora_component(
            lora_attn_modules=lora_attn_modules,
            apply_lora_to_mlp=apply_lora_to_mlp,
            apply_lora_to_output=apply_lora_to_output,
            lora_rank=lora_rank,
            lora_alpha=lora_alpha,
            lora_dropout=lora_dropout,
            use_dora=use_dora,
            quantize_base=quantize_base,
            **{**fixed, **exposed, **kwargs},
        )

    builder.__name__ = builder.__qualname__ = name
    builder.__doc__ = doc
    return builder


def qlora_preset(lora_builder: Callable[..., TransformerDecoder], name: str) -> Callable[..., TransformerDecoder]:
    fn = functools.partial(lora_builder, quantize_base=True)
    fn.__name__ = name  # type: ignore[attr-defined]
    fn.__doc__ = f"``{lora_builder.__name__}`` with the frozen base weights stored in NF4 (QLoRA, arXiv 2305.14314)."
    return fn


def _set_signature(fn: Callable, exposed: Dict[str, Any]) -> None:
    import inspect

    params = [inspect.Parameter(k, inspect.Parameter.KEYWORD_ONLY if False else inspect.Parameter.POSITIONAL_OR_KEYWORD, default=v) for k, v in exposed.items()]
    fn.__signature__ = inspect.Signature(params)  # type: ignore[attr-defined]

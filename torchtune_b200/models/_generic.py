"""Generator for the ``<family>(...)`` / ``lora_<family>(...)`` component-builder pair of a
decoder family from one function that maps keyword arguments to a :class:`DecoderArch`.

The reference spells both out per family (e.g. torchtune/models/llama2/_component_builders.py:43-330,
torchtune/models/mistral/_component_builders.py, torchtune/models/qwen2/_component_builders.py);
the public names and keyword arguments are kept.
"""
from __future__ import annotations

import inspect
from typing import Any, Callable, List, Tuple

from ..modules import TransformerDecoder
from ._factory import DecoderArch, adapter_from_kwargs, build_decoder

_LORA_KEYS = ("lora_rank", "lora_alpha", "lora_dropout", "use_dora", "quantize_base")


def component_builders(name: str, arch_fn: Callable[..., DecoderArch], doc: str) -> Tuple[Callable, Callable]:
    """Returns ``(builder, lora_builder)``; ``arch_fn(**kwargs)`` describes the architecture."""

    def builder(*args: Any, **kwargs: Any) -> TransformerDecoder:
        bound = inspect.signature(arch_fn).bind(*args, **kwargs)
        return build_decoder(arch_fn(*bound.args, **bound.kwargs))

    def lora_builder(
        lora_attn_modules: List[str],
        apply_lora_to_mlp: bool = False,
        apply_lora_to_output: bool = False,
        **kwargs: Any,
    ) -> TransformerDecoder:
        if "lora_rank" not in kwargs or "lora_alpha" not in kwargs:
            raise TypeError(f"lora_{name}() missing required keyword arguments 'lora_rank' and 'lora_alpha'")
        lora = {k: kwargs.pop(k) for k in _LORA_KEYS if k in kwargs}
        ad = adapter_from_kwargs(lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, **lora)
        return build_decoder(arch_fn(**kwargs), ad)

    builder.__name__ = builder.__qualname__ = name
    builder.__doc__ = doc
    builder.__signature__ = inspect.signature(arch_fn).replace(return_annotation=TransformerDecoder)  # type: ignore[attr-defined]
    lora_builder.__name__ = lora_builder.__qualname__ = f"lora_{name}"
    lora_builder.__doc__ = doc + "  LoRA / DoRA adapters (optionally over an NF4 base) on the listed projections."
    return builder, lora_builder


def classifier_builders(name: str, arch_fn: Callable[..., DecoderArch], doc: str) -> Tuple[Callable, Callable]:
    """Same, with the output projection replaced by ``Linear(dim, num_classes)`` (reward / value models)."""
    from ..modules import Linear

    base, lora_base = component_builders(name, arch_fn, doc)

    def _swap(model: TransformerDecoder, num_classes: int) -> TransformerDecoder:
        dim = model.tok_embeddings.embedding_dim
        model.output = Linear(dim, num_classes, bias=False)
        return model

    def builder(num_classes: int, **kwargs: Any) -> TransformerDecoder:
        return _swap(base(**kwargs), num_classes)

    def lora_builder(lora_attn_modules: List[str], apply_lora_to_mlp: bool = False, apply_lora_to_output: bool = False, *, num_classes: int, **kwargs: Any) -> TransformerDecoder:
        # adapters on a freshly initialised classification head make no sense: it is trained fully
        return _swap(lora_base(lora_attn_modules, apply_lora_to_mlp, False, **kwargs), num_classes)

    builder.__name__ = f"{name}_classifier"
    lora_builder.__name__ = f"lora_{name}_classifier"
    builder.__doc__ = lora_builder.__doc__ = doc + "  Classification head instead of the vocabulary projection."
    return builder, lora_builder

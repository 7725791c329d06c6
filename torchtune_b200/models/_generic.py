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


def layer_builders(arch_fn: Callable[..., DecoderArch]) -> Tuple[Callable, Callable, Callable]:
    """``(mlp, lora_self_attention, lora_mlp)`` for one family: single-layer pieces with the family's activation, biases, head
    width, rotary embedding and per-head norms, for callers who assemble their own decoder (the reference writes these out per
    family, e.g. torchtune/models/llama3/_component_builders.py:129-147, 300-380, 467-510).

    The pieces come from the same :class:`DecoderArch` the whole-model builder uses, so a layer built here matches a layer of the
    full model weight for weight."""
    from ._factory import AdapterSpec, build_attention, build_mlp

    params = inspect.signature(arch_fn).parameters

    def _arch(embed_dim: int, hidden: int, num_heads: int = 1, num_kv_heads: int = 1, max_seq_len: int = 1, **extra: Any) -> DecoderArch:
        kw = dict(vocab_size=1, num_layers=1, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len)
        if "intermediate_dim" in params:
            kw["intermediate_dim"] = hidden
        if "head_dim" in params and params["head_dim"].default is inspect.Parameter.empty and "head_dim" not in extra:
            kw["head_dim"] = embed_dim // num_heads
        unknown = set(extra) - set(params)
        if unknown:
            raise TypeError(f"unexpected keyword arguments {sorted(unknown)}")
        kw.update(extra)
        return arch_fn(**kw)

    def mlp(dim: int, hidden_dim: int, quantize_base: bool = False):
        arch = _arch(dim, hidden_dim)
        return build_mlp(dim, hidden_dim, AdapterSpec(quantize_base=quantize_base), arch.activation(), arch.mlp_bias)

    def lora_mlp(*, dim: int, hidden_dim: int, lora_rank: int, lora_alpha: float, lora_dropout: float = 0.0, quantize_base: bool = False, use_dora: bool = False):
        arch = _arch(dim, hidden_dim)
        ad = AdapterSpec(apply_to_mlp=True, rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base)
        return build_mlp(dim, hidden_dim, ad, arch.activation(), arch.mlp_bias)

    def lora_self_attention(lora_modules: List[str], *, embed_dim: int, num_heads: int, num_kv_heads: int, max_seq_len: int, lora_rank: int, lora_alpha: float,
                            lora_dropout: float = 0.0, quantize_base: bool = False, use_dora: bool = False, **arch_kwargs: Any):
        if not lora_modules:
            raise ValueError("lora_modules is empty: name at least one of q_proj, k_proj, v_proj, output_proj")
        arch = _arch(embed_dim, embed_dim, num_heads, num_kv_heads, max_seq_len, **arch_kwargs)
        ad = AdapterSpec(attn_modules=tuple(lora_modules), rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base)
        rope = arch.rope(arch.resolved_head_dim(), arch.max_seq_len) if arch.rope else None
        return build_attention(arch, ad, rope)

    return mlp, lora_self_attention, lora_mlp

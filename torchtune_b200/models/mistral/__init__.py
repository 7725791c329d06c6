"""Mistral 7B and its reward/classifier variants (parity: torchtune/models/mistral/*)."""
from typing import Optional

from ...modules import RotaryPositionalEmbeddings
from .._factory import DecoderArch
from .._family import lora_preset, preset, qlora_preset
from .._generic import classifier_builders, component_builders, layer_builders


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int, attn_dropout: float = 0.0, norm_eps: float = 1e-5, rope_base: int = 10_000) -> DecoderArch:
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, rope=lambda hd, msl: RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base))


mistral, lora_mistral = component_builders("mistral", _arch, "Mistral decoder: GQA, SwiGLU, RMSNorm, interleaved RoPE (the sliding window of the original is not applied).")
mistral_mlp, lora_mistral_self_attention, lora_mistral_mlp = layer_builders(_arch)
mistral_classifier, lora_mistral_classifier = classifier_builders("mistral", _arch, "Mistral decoder.")

_C = dict(vocab_size=32_000, num_layers=32, num_heads=32, num_kv_heads=8, embed_dim=4096, intermediate_dim=14336, max_seq_len=32768, attn_dropout=0.0, norm_eps=1e-5)
mistral_7b = preset(mistral, "mistral_7b", "Mistral 7B.", **_C)
lora_mistral_7b = lora_preset(lora_mistral, "lora_mistral_7b", "Mistral 7B with adapters.", **_C)
qlora_mistral_7b = qlora_preset(lora_mistral_7b, "qlora_mistral_7b")
mistral_reward_7b = preset(mistral_classifier, "mistral_reward_7b", "Mistral 7B with a scalar reward head.", num_classes=1, **_C)
lora_mistral_reward_7b = lora_preset(lora_mistral_classifier, "lora_mistral_reward_7b", "Mistral 7B reward model with adapters.", num_classes=1, **_C)
qlora_mistral_reward_7b = qlora_preset(lora_mistral_reward_7b, "qlora_mistral_reward_7b")


def mistral_tokenizer(path: str, max_seq_len: Optional[int] = None, prompt_template="torchtune_b200.models.mistral.MistralChatTemplate", truncation_type: str = "right"):
    from ...data._prompt_templates import _get_prompt_template
    from ._tokenizer import MistralTokenizer

    return MistralTokenizer(path=path, max_seq_len=max_seq_len, prompt_template=_get_prompt_template(prompt_template) if prompt_template is not None else None, truncation_type=truncation_type)


def __getattr__(name):
    if name == "MistralTokenizer":
        from ._tokenizer import MistralTokenizer

        return MistralTokenizer
    if name == "MistralChatTemplate":
        from ._prompt_template import MistralChatTemplate

        return MistralChatTemplate
    raise AttributeError(name)

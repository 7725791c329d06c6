"""Llama 2 (parity: torchtune/models/llama2/_component_builders.py:43-600, _model_builders.py:25-380)."""
from typing import Optional

from ...modules import RotaryPositionalEmbeddings
from .._factory import DecoderArch
from .._family import lora_preset, preset, qlora_preset
from .._generic import classifier_builders, component_builders, layer_builders


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int, attn_dropout: float = 0.0, intermediate_dim: Optional[int] = None, norm_eps: float = 1e-5, rope_base: int = 10_000) -> DecoderArch:
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, rope=lambda hd, msl: RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base))


llama2, lora_llama2 = component_builders("llama2", _arch, "Llama-2 decoder: MHA/GQA, SwiGLU, RMSNorm, interleaved RoPE, untied output.")
llama2_mlp, lora_llama2_self_attention, lora_llama2_mlp = layer_builders(_arch)
llama2_classifier, lora_llama2_classifier = classifier_builders("llama2", _arch, "Llama-2 decoder.")

_C = dict(vocab_size=32_000, max_seq_len=4096, attn_dropout=0.0, norm_eps=1e-5)
_S = {
    "7b": dict(num_layers=32, num_heads=32, num_kv_heads=32, embed_dim=4096),
    "13b": dict(num_layers=40, num_heads=40, num_kv_heads=40, embed_dim=5120, intermediate_dim=13824),
    "70b": dict(num_layers=80, num_heads=64, num_kv_heads=8, embed_dim=8192, intermediate_dim=28672),
}
llama2_7b = preset(llama2, "llama2_7b", "Llama-2 7B.", **_C, **_S["7b"])
llama2_13b = preset(llama2, "llama2_13b", "Llama-2 13B.", **_C, **_S["13b"])
llama2_70b = preset(llama2, "llama2_70b", "Llama-2 70B.", **_C, **_S["70b"])
lora_llama2_7b = lora_preset(lora_llama2, "lora_llama2_7b", "Llama-2 7B with adapters.", **_C, **_S["7b"])
lora_llama2_13b = lora_preset(lora_llama2, "lora_llama2_13b", "Llama-2 13B with adapters.", **_C, **_S["13b"])
lora_llama2_70b = lora_preset(lora_llama2, "lora_llama2_70b", "Llama-2 70B with adapters.", **_C, **_S["70b"])
qlora_llama2_7b = qlora_preset(lora_llama2_7b, "qlora_llama2_7b")
qlora_llama2_13b = qlora_preset(lora_llama2_13b, "qlora_llama2_13b")
qlora_llama2_70b = qlora_preset(lora_llama2_70b, "qlora_llama2_70b")
llama2_reward_7b = preset(llama2_classifier, "llama2_reward_7b", "Llama-2 7B with a scalar reward head.", num_classes=1, **_C, **_S["7b"])
lora_llama2_reward_7b = lora_preset(lora_llama2_classifier, "lora_llama2_reward_7b", "Llama-2 7B reward model with adapters.", num_classes=1, **_C, **_S["7b"])
qlora_llama2_reward_7b = qlora_preset(lora_llama2_reward_7b, "qlora_llama2_reward_7b")


def llama2_tokenizer(path: str, max_seq_len: Optional[int] = None, prompt_template="torchtune_b200.models.llama2.Llama2ChatTemplate", truncation_type: str = "right"):
    from ...data._prompt_templates import _get_prompt_template
    from ._tokenizer import Llama2Tokenizer

    return Llama2Tokenizer(path=path, max_seq_len=max_seq_len, prompt_template=_get_prompt_template(prompt_template) if prompt_template is not None else None, truncation_type=truncation_type)


def __getattr__(name):
    if name == "Llama2Tokenizer":
        from ._tokenizer import Llama2Tokenizer

        return Llama2Tokenizer
    if name == "Llama2ChatTemplate":
        from ._prompt_template import Llama2ChatTemplate

        return Llama2ChatTemplate
    raise AttributeError(name)

from .._factory import scale_hidden_dim_for_mlp  # noqa: E402,F401

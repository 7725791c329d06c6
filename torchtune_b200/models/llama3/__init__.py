"""Llama 3 (parity: torchtune/models/llama3/_component_builders.py, _model_builders.py:26-260)."""
from typing import Optional

from ...modules import RotaryPositionalEmbeddings
from .._factory import DecoderArch, scale_hidden_dim_for_mlp  # noqa: F401
from .._family import lora_preset, preset, qlora_preset
from .._generic import component_builders, layer_builders


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int, attn_dropout: float = 0.0, rope_base: int = 500_000, intermediate_dim: Optional[int] = None, norm_eps: float = 1e-5) -> DecoderArch:
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, rope=lambda hd, msl: RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base))


llama3, lora_llama3 = component_builders("llama3", _arch, "Llama-3 decoder: GQA, SwiGLU, RMSNorm, interleaved RoPE (base 500k), 128k vocabulary.")
llama3_mlp, lora_llama3_self_attention, lora_llama3_mlp = layer_builders(_arch)

_C = dict(vocab_size=128_256, max_seq_len=8192, attn_dropout=0.0, norm_eps=1e-5, rope_base=500_000)
_S = {
    "8b": dict(num_layers=32, num_heads=32, num_kv_heads=8, embed_dim=4096, intermediate_dim=14336),
    "70b": dict(num_layers=80, num_heads=64, num_kv_heads=8, embed_dim=8192, intermediate_dim=28672),
}
llama3_8b = preset(llama3, "llama3_8b", "Llama-3 8B.", **_C, **_S["8b"])
llama3_70b = preset(llama3, "llama3_70b", "Llama-3 70B.", **_C, **_S["70b"])
lora_llama3_8b = lora_preset(lora_llama3, "lora_llama3_8b", "Llama-3 8B with adapters.", **_C, **_S["8b"])
lora_llama3_70b = lora_preset(lora_llama3, "lora_llama3_70b", "Llama-3 70B with adapters.", **_C, **_S["70b"])
qlora_llama3_8b = qlora_preset(lora_llama3_8b, "qlora_llama3_8b")
qlora_llama3_70b = qlora_preset(lora_llama3_70b, "qlora_llama3_70b")


def llama3_tokenizer(path: str, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
    from ...data._prompt_templates import _get_prompt_template
    from ...modules.transforms.tokenizers import parse_hf_tokenizer_json
    from ._tokenizer import Llama3Tokenizer

    special = parse_hf_tokenizer_json(special_tokens_path) if special_tokens_path is not None else None
    template = _get_prompt_template(prompt_template) if prompt_template is not None else None
    return Llama3Tokenizer(path=path, special_tokens=special, max_seq_len=max_seq_len, prompt_template=template, truncation_type=truncation_type)


def __getattr__(name):
    if name == "Llama3Tokenizer":
        from ._tokenizer import Llama3Tokenizer

        return Llama3Tokenizer
    if name in ("base_llama_tp_plan", "decoder_only_tp_plan", "_fp8_llama_tp_plan"):
        from . import _parallelism

        return getattr(_parallelism, name)
    raise AttributeError(name)

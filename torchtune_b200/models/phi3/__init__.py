"""Phi-3 mini (parity: torchtune/models/phi3/*): Llama-like decoder with half-split RoPE."""
from typing import Optional

from ...modules import Phi3RotaryPositionalEmbeddings
from .._factory import DecoderArch
from .._family import lora_preset, preset, qlora_preset
from .._generic import component_builders, layer_builders
from ._convert_weights import phi3_hf_to_tune, phi3_tune_to_hf  # noqa: F401


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int, attn_dropout: float = 0.0, norm_eps: float = 1e-5, rope_base: int = 10_000) -> DecoderArch:
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, rope=lambda hd, msl: Phi3RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base))


phi3, lora_phi3 = component_builders("phi3", _arch, "Phi-3 decoder.")
phi3_mlp, lora_phi3_self_attention, lora_phi3_mlp = layer_builders(_arch)
_C = dict(vocab_size=32_064, num_layers=32, num_heads=32, num_kv_heads=32, embed_dim=3072, intermediate_dim=8192, max_seq_len=4096, attn_dropout=0.0, norm_eps=1e-5)
phi3_mini = preset(phi3, "phi3_mini", "Phi-3 mini 4k instruct (3.8B).", **_C)
lora_phi3_mini = lora_preset(lora_phi3, "lora_phi3_mini", "Phi-3 mini with adapters.", **_C)
qlora_phi3_mini = qlora_preset(lora_phi3_mini, "qlora_phi3_mini")


def phi3_mini_tokenizer(path: str, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
    from ...data._prompt_templates import _get_prompt_template
    from ...modules.transforms.tokenizers import parse_hf_tokenizer_json
    from ._tokenizer import Phi3MiniTokenizer

    special = parse_hf_tokenizer_json(special_tokens_path) if special_tokens_path is not None else None
    template = _get_prompt_template(prompt_template) if prompt_template is not None else None
    return Phi3MiniTokenizer(path=path, special_tokens=special, max_seq_len=max_seq_len, prompt_template=template, truncation_type=truncation_type)


def __getattr__(name):
    # tokenizer classes are imported on first use (they pull in sentencepiece / regex tables)
    if name == "Phi3MiniTokenizer":
        from ._tokenizer import Phi3MiniTokenizer

        return Phi3MiniTokenizer
    raise AttributeError(name)

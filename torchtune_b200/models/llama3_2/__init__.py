"""Llama 3.2 text models, tied embeddings by default (parity: torchtune/models/llama3_2/*)."""
from typing import Optional

from ...modules import Llama3ScaledRoPE
from .._factory import DecoderArch
from .._family import lora_preset, preset, qlora_preset
from .._generic import component_builders, layer_builders


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int, attn_dropout: float = 0.0, rope_base: int = 500_000, intermediate_dim: Optional[int] = None, norm_eps: float = 1e-5, scale_factor: int = 32, tie_word_embeddings: bool = True) -> DecoderArch:
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, tie_embeddings=tie_word_embeddings, rope=lambda hd, msl: Llama3ScaledRoPE(dim=hd, max_seq_len=msl, base=rope_base, scale_factor=scale_factor))


llama3_2, lora_llama3_2 = component_builders("llama3_2", _arch, "Llama-3.2 decoder: Llama-3.1 architecture with scale factor 32 and (by default) the output projection tied to the token embeddings.")
llama3_mlp, lora_llama3_2_self_attention, lora_llama3_mlp = layer_builders(_arch)

_C = dict(vocab_size=128_256, max_seq_len=131072, attn_dropout=0.0, norm_eps=1e-5, rope_base=500_000, scale_factor=32)
_S = {
    "1b": dict(num_layers=16, num_heads=32, num_kv_heads=8, embed_dim=2048, intermediate_dim=8192),
    "3b": dict(num_layers=28, num_heads=24, num_kv_heads=8, embed_dim=3072, intermediate_dim=8192),
}
_T = {"tie_word_embeddings": True}
llama3_2_1b = preset(llama3_2, "llama3_2_1b", "Llama-3.2 1B.", exposed=_T, **_C, **_S["1b"])
llama3_2_3b = preset(llama3_2, "llama3_2_3b", "Llama-3.2 3B.", exposed=_T, **_C, **_S["3b"])
lora_llama3_2_1b = lora_preset(lora_llama3_2, "lora_llama3_2_1b", "Llama-3.2 1B with adapters.", exposed=_T, **_C, **_S["1b"])
lora_llama3_2_3b = lora_preset(lora_llama3_2, "lora_llama3_2_3b", "Llama-3.2 3B with adapters.", exposed=_T, **_C, **_S["3b"])
qlora_llama3_2_1b = qlora_preset(lora_llama3_2_1b, "qlora_llama3_2_1b")
qlora_llama3_2_3b = qlora_preset(lora_llama3_2_3b, "qlora_llama3_2_3b")

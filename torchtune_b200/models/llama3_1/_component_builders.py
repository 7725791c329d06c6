"""Llama 3.1 architecture (parity: torchtune/models/llama3_1/_component_builders.py:41-330)."""
from __future__ import annotations

from typing import List, Optional

from ...modules import Llama3ScaledRoPE, TransformerDecoder
from .._factory import AdapterSpec, DecoderArch, adapter_from_kwargs, build_decoder


def _arch(vocab_size, num_layers, num_heads, num_kv_heads, embed_dim, max_seq_len, attn_dropout, rope_base, intermediate_dim, norm_eps, scale_factor, tie=False) -> DecoderArch:
    return DecoderArch(
        vocab_size=vocab_size,
        num_layers=num_layers,
        num_heads=num_heads,
        num_kv_heads=num_kv_heads,
        embed_dim=embed_dim,
        max_seq_len=max_seq_len,
        intermediate_dim=intermediate_dim,
        attn_dropout=attn_dropout,
        norm_eps=norm_eps,
        rope=lambda hd, msl: Llama3ScaledRoPE(dim=hd, max_seq_len=msl, base=rope_base, scale_factor=scale_factor),
        tie_embeddings=tie,
    )


def llama3_1(
    vocab_size: int,
    num_layers: int,
    num_heads: int,
    num_kv_heads: int,
    embed_dim: int,
    max_seq_len: int,
    attn_dropout: float = 0.0,
    rope_base: int = 500_000,
    intermediate_dim: Optional[int] = None,
    norm_eps: float = 1e-5,
    scale_factor: int = 8,
) -> TransformerDecoder:
    """Decoder with GQA, SwiGLU, RMSNorm and frequency-scaled interleaved RoPE; untied output."""
    return build_decoder(_arch(vocab_size, num_layers, num_heads, num_kv_heads, embed_dim, max_seq_len, attn_dropout, rope_base, intermediate_dim, norm_eps, scale_factor))


def lora_llama3_1(
    lora_attn_modules: List[str],
    apply_lora_to_mlp: bool = False,
    apply_lora_to_output: bool = False,
    *,
    vocab_size: int,
    num_layers: int,
    num_heads: int,
    num_kv_heads: int,
    embed_dim: int,
    max_seq_len: int,
    intermediate_dim: Optional[int] = None,
    attn_dropout: float = 0.0,
    norm_eps: float = 1e-5,
    rope_base: int = 500_000,
    scale_factor: int = 8,
    lora_rank: int,
    lora_alpha: float,
    lora_dropout: float = 0.0,
    use_dora: bool = False,
    quantize_base: bool = False,
) -> TransformerDecoder:
    arch = _arch(vocab_size, num_layers, num_heads, num_kv_heads, embed_dim, max_seq_len, attn_dropout, rope_base, intermediate_dim, norm_eps, scale_factor)
    ad = adapter_from_kwargs(lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base)
    return build_decoder(arch, ad)


def _layer_arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int, attn_dropout: float = 0.0,
                rope_base: int = 500_000, intermediate_dim: Optional[int] = None, norm_eps: float = 1e-5, scale_factor: int = 8) -> DecoderArch:
    return _arch(vocab_size, num_layers, num_heads, num_kv_heads, embed_dim, max_seq_len, attn_dropout, rope_base, intermediate_dim, norm_eps, scale_factor)


def _layer_builders():
    from .._generic import layer_builders

    return layer_builders(_layer_arch)


# single-layer pieces under the reference's names (torchtune/models/llama3_1/_component_builders.py:127-145, 296-376, 379-420)
llama3_mlp, lora_llama3_attention, lora_llama3_mlp = _layer_builders()

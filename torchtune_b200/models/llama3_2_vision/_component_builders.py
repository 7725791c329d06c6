"""Llama 3.2 Vision components (parity: torchtune/models/llama3_2_vision/_component_builders.py:59-800).

One set of builders serves the full and the LoRA variants: an :class:`AdapterSpec` per part
(decoder layers, fusion layers, CLIP trunk, projection head) says where adapters go.
"""
from __future__ import annotations

from enum import Enum
from typing import List, Optional

from torch import nn

from ...modules import Fp32LayerNorm, Linear, Llama3ScaledRoPE, MultiHeadAttention, RMSNorm, TanhGate, TransformerCrossAttentionLayer, TransformerDecoder, TransformerSelfAttentionLayer
from ...modules.common_utils import _register_reparametrize_state_dict_hooks
from ...modules.model_fusion import FusionEmbedding, FusionLayer
from ...modules.peft import DoRALinear, LoRALinear
from .._factory import AdapterSpec, DecoderArch, build_attention, build_mlp, scale_hidden_dim_for_mlp
from ..clip._component_builders import _vision_encoder, clip_mlp
from ._encoder import Llama3VisionEncoder, Llama3VisionProjectionHead


class LoRATrainable(Enum):
    FULL = "full"
    LORA = "lora"
    FROZEN = "frozen"


_NONE = AdapterSpec()


def _decoder(*, vocab_size: int, num_layers: int, fusion_interval: int, num_special_tokens: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int,
             encoder_max_seq_len: int, rope_base: float, intermediate_dim: Optional[int], layer_ad: AdapterSpec, fusion_ad: AdapterSpec) -> TransformerDecoder:
    head_dim = embed_dim // num_heads
    hidden = intermediate_dim or scale_hidden_dim_for_mlp(embed_dim)
    arch = DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads or num_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=hidden)
    rope = Llama3ScaledRoPE(dim=head_dim, max_seq_len=max_seq_len, base=rope_base)
    xarch = DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads or num_heads, embed_dim=embed_dim, max_seq_len=encoder_max_seq_len,
                        intermediate_dim=hidden, qk_norm=lambda d, eps: RMSNorm(d, eps=1e-5))
    layers: List[nn.Module] = []
    for idx in range(1, num_layers + 1):
        layer = TransformerSelfAttentionLayer(attn=build_attention(arch, layer_ad, rope), mlp=build_mlp(embed_dim, hidden, layer_ad), sa_norm=RMSNorm(embed_dim, eps=1e-5), mlp_norm=RMSNorm(embed_dim, eps=1e-5))
        if idx % fusion_interval == 0:
            xattn = build_attention(xarch, fusion_ad, None)
            xattn.is_causal = False
            cross = TransformerCrossAttentionLayer(attn=xattn, mlp=build_mlp(embed_dim, hidden, fusion_ad), ca_norm=RMSNorm(embed_dim), mlp_norm=RMSNorm(embed_dim), ca_scale=TanhGate(), mlp_scale=TanhGate())
            layers.append(FusionLayer(layer=layer, fusion_layer=cross))
        else:
            layers.append(layer)
    if layer_ad.apply_to_output:
        cls = DoRALinear if layer_ad.use_dora else LoRALinear
        output = cls(embed_dim, vocab_size, rank=layer_ad.rank, alpha=layer_ad.alpha, dropout=layer_ad.dropout)
    else:
        output = Linear(embed_dim, vocab_size, bias=False)
    model = TransformerDecoder(tok_embeddings=FusionEmbedding(vocab_size, num_special_tokens, embed_dim), layers=layers, max_seq_len=max_seq_len, num_heads=num_heads, head_dim=head_dim,
                               norm=RMSNorm(embed_dim, eps=1e-5), output=output)
    if layer_ad.quantize_base or fusion_ad.quantize_base:
        _register_reparametrize_state_dict_hooks(model, dtype=model.tok_embeddings.embedding.weight.dtype)
    return model


def llama3_2_vision_decoder(*, vocab_size: int, num_layers: int, fusion_interval: int, num_special_tokens: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int,
                            encoder_max_seq_len: int, rope_base: float = 500000.0, intermediate_dim: Optional[int] = None) -> TransformerDecoder:
    """Llama-3.1 text decoder with a gated cross-attention layer in front of every ``fusion_interval``-th
    layer and ``num_special_tokens`` extra (trainable) embedding rows."""
    return _decoder(vocab_size=vocab_size, num_layers=num_layers, fusion_interval=fusion_interval, num_special_tokens=num_special_tokens, num_heads=num_heads, num_kv_heads=num_kv_heads,
                    embed_dim=embed_dim, max_seq_len=max_seq_len, encoder_max_seq_len=encoder_max_seq_len, rope_base=rope_base, intermediate_dim=intermediate_dim, layer_ad=_NONE, fusion_ad=_NONE)


def _spec(on: bool, lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base) -> AdapterSpec:
    if not on:
        return AdapterSpec(quantize_base=quantize_base)
    return AdapterSpec(attn_modules=tuple(lora_attn_modules), apply_to_mlp=apply_lora_to_mlp, apply_to_output=apply_lora_to_output, rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base)


def lora_llama3_2_vision_decoder(decoder_lora: bool, fusion_lora: bool, lora_attn_modules: List[str], apply_lora_to_mlp: bool = False, apply_lora_to_output: bool = False, *, vocab_size: int,
                                 num_layers: int, fusion_interval: int, num_special_tokens: int, num_heads: int, num_kv_heads: int, embed_dim: int, max_seq_len: int, encoder_max_seq_len: int,
                                 rope_base: float = 500000.0, intermediate_dim: Optional[int] = None, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False,
                                 quantize_base: bool = False) -> TransformerDecoder:
    args = (lora_attn_modules, apply_lora_to_mlp)
    tail = (lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base)
    return _decoder(vocab_size=vocab_size, num_layers=num_layers, fusion_interval=fusion_interval, num_special_tokens=num_special_tokens, num_heads=num_heads, num_kv_heads=num_kv_heads,
                    embed_dim=embed_dim, max_seq_len=max_seq_len, encoder_max_seq_len=encoder_max_seq_len, rope_base=rope_base, intermediate_dim=intermediate_dim,
                    layer_ad=_spec(decoder_lora, *args, apply_lora_to_output and decoder_lora, *tail), fusion_ad=_spec(fusion_lora, *args, False, *tail))


def _projection_head(*, num_layers: int, num_heads: int, decoder_embed_dim: int, clip_embed_dim: int, num_hidden_inputs: int, ad: AdapterSpec) -> Llama3VisionProjectionHead:
    head_dim = clip_embed_dim // num_heads
    mods = set(ad.attn_modules)
    lora = dict(rank=ad.rank, alpha=ad.alpha, dropout=ad.dropout, use_dora=ad.use_dora) if (mods or ad.apply_to_mlp) else None
    layers = []
    for _ in range(num_layers):
        attn = MultiHeadAttention(
            embed_dim=clip_embed_dim, num_heads=num_heads, num_kv_heads=num_heads, head_dim=head_dim,
            q_proj=ad.make(clip_embed_dim, clip_embed_dim, "q_proj" in mods), k_proj=ad.make(clip_embed_dim, clip_embed_dim, "k_proj" in mods),
            v_proj=ad.make(clip_embed_dim, clip_embed_dim, "v_proj" in mods), output_proj=ad.make(clip_embed_dim, clip_embed_dim, "output_proj" in mods),
            pos_embeddings=None, attn_dropout=0.0, is_causal=False,
        )
        mlp = clip_mlp(clip_embed_dim, clip_embed_dim, 4 * clip_embed_dim, nn.GELU(), quantize_base=ad.quantize_base, _lora=lora if ad.apply_to_mlp else None)
        layers.append(TransformerSelfAttentionLayer(attn=attn, mlp=mlp, sa_norm=Fp32LayerNorm(clip_embed_dim, eps=1e-5), mlp_norm=Fp32LayerNorm(clip_embed_dim, eps=1e-5), sa_scale=TanhGate(), mlp_scale=TanhGate()))
    proj_in = clip_embed_dim * (num_hidden_inputs + 1)
    if ad.apply_to_output:
        cls = DoRALinear if ad.use_dora else LoRALinear
        output = cls(proj_in, decoder_embed_dim, rank=ad.rank, alpha=ad.alpha, dropout=ad.dropout, use_bias=True, quantize_base=False)
    else:
        output = Linear(proj_in, decoder_embed_dim)
    return Llama3VisionProjectionHead(layers=layers, output=output, num_hidden_inputs=num_hidden_inputs)


def llama3_2_vision_projection_head(*, num_layers: int, num_heads: int, decoder_embed_dim: int, clip_embed_dim: int, num_hidden_inputs: int) -> Llama3VisionProjectionHead:
    return _projection_head(num_layers=num_layers, num_heads=num_heads, decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, num_hidden_inputs=num_hidden_inputs, ad=_NONE)


def lora_llama3_2_vision_projection_head(lora_modules: List[str], *, num_layers: int, num_heads: int, decoder_embed_dim: int, clip_embed_dim: int, num_hidden_inputs: int, apply_lora_to_mlp: bool = False,
                                         apply_lora_to_output: bool = False, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, **_) -> Llama3VisionProjectionHead:
    ad = _spec(True, lora_modules, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base)
    return _projection_head(num_layers=num_layers, num_heads=num_heads, decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, num_hidden_inputs=num_hidden_inputs, ad=ad)


def _encoder(*, patch_size: int, num_heads: int, clip_embed_dim: int, clip_num_layers: int, clip_hidden_states: Optional[List[int]], num_layers_projection: int, decoder_embed_dim: int,
             tile_size: int, max_num_tiles: int, in_channels: int, clip_ad: AdapterSpec, head_ad: AdapterSpec) -> Llama3VisionEncoder:
    lora = dict(rank=clip_ad.rank, alpha=clip_ad.alpha, dropout=clip_ad.dropout, use_dora=clip_ad.use_dora) if (clip_ad.attn_modules or clip_ad.apply_to_mlp) else None
    clip = _vision_encoder(
        tile_size=tile_size, patch_size=patch_size, embed_dim=clip_embed_dim, num_layers=clip_num_layers, num_heads=num_heads, activation=nn.GELU, cls_output_dim=512, attn_bias=False,
        use_rope=False, out_indices=clip_hidden_states, output_cls_projection=False, max_num_tiles=max_num_tiles, in_channels=in_channels, append_cls_token=False, use_tile_pos_embed=True,
        lora_modules=tuple(clip_ad.attn_modules), lora=lora, apply_lora_to_mlp=clip_ad.apply_to_mlp, quantize_base=clip_ad.quantize_base,
    )
    head = _projection_head(num_layers=num_layers_projection, num_heads=num_heads, decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, num_hidden_inputs=len(clip_hidden_states or []), ad=head_ad)
    enc = Llama3VisionEncoder(clip=clip, projection_head=head)
    if clip_ad.quantize_base or head_ad.quantize_base:
        _register_reparametrize_state_dict_hooks(enc, dtype=clip.conv.weight.dtype)
    return enc


def llama3_2_vision_encoder(*, patch_size: int, num_heads: int, clip_embed_dim: int, clip_num_layers: int, clip_hidden_states: Optional[List[int]], num_layers_projection: int,
                            decoder_embed_dim: int, tile_size: int, max_num_tiles: int = 4, in_channels: int = 3) -> Llama3VisionEncoder:
    return _encoder(patch_size=patch_size, num_heads=num_heads, clip_embed_dim=clip_embed_dim, clip_num_layers=clip_num_layers, clip_hidden_states=clip_hidden_states,
                    num_layers_projection=num_layers_projection, decoder_embed_dim=decoder_embed_dim, tile_size=tile_size, max_num_tiles=max_num_tiles, in_channels=in_channels, clip_ad=_NONE, head_ad=_NONE)


def lora_llama3_2_vision_encoder(encoder_lora: bool, fusion_lora: bool, lora_attn_modules: List[str], apply_lora_to_mlp: bool = False, apply_lora_to_output: bool = False, *, patch_size: int,
                                 num_heads: int, clip_embed_dim: int, clip_num_layers: int, clip_hidden_states: Optional[List[int]], num_layers_projection: int, decoder_embed_dim: int,
                                 tile_size: int, max_num_tiles: int = 4, in_channels: int = 3, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False,
                                 quantize_base: bool = False, **_) -> Llama3VisionEncoder:
    tail = (lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base)
    return _encoder(patch_size=patch_size, num_heads=num_heads, clip_embed_dim=clip_embed_dim, clip_num_layers=clip_num_layers, clip_hidden_states=clip_hidden_states,
                    num_layers_projection=num_layers_projection, decoder_embed_dim=decoder_embed_dim, tile_size=tile_size, max_num_tiles=max_num_tiles, in_channels=in_channels,
                    clip_ad=_spec(encoder_lora, lora_attn_modules, apply_lora_to_mlp, False, *tail), head_ad=_spec(fusion_lora, lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output and fusion_lora, *tail))

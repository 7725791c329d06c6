"""Llama-4 decoder (MoE, interleaved chunked-RoPE / global-NoPE attention) and vision encoder
(parity: torchtune/models/llama4/_component_builders.py:40-800)."""
from __future__ import annotations

from functools import partial
from typing import List, Optional

from torch import nn

from ...modules import FeedForward, Linear, Llama4ScaledRoPE, RotaryPositionalEmbeddings, TransformerDecoder, rms_norm
from ...modules.moe import GroupedExperts, LoRAGroupedExperts, MoE, TokenChoiceTopKRouter
from ...modules.peft import DoRALinear, LoRALinear
from .._factory import AdapterSpec, DecoderArch, adapter_from_kwargs, build_decoder, build_mlp
from ..clip import clip_vision_encoder
from ._chunked_attention import chunked_mask_mod
from ._encoder import Llama4VisionEncoder, Llama4VisionProjectionHead


class _UnitRMSNorm(nn.Module):
    """RMS normalisation without a learned scale (Llama-4 q/k norm)."""

    def __init__(self, eps: float):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        return rms_norm(x, self.eps)


def llama4_mlp(dim: int, hidden_dim: int, quantize_base: bool = False) -> FeedForward:
    return build_mlp(dim, hidden_dim, AdapterSpec(quantize_base=quantize_base))


def llama4_moe(dim: int, hidden_dim: int, num_experts: int = 8, experts_per_token: int = 1, use_shared_expert: bool = True) -> MoE:
    router = TokenChoiceTopKRouter(gate=Linear(dim, num_experts, bias=False), dim=dim, num_experts=num_experts, experts_per_token=experts_per_token)
    return MoE(experts=GroupedExperts(dim=dim, hidden_dim=hidden_dim, num_experts=num_experts), router=router, shared_expert=llama4_mlp(dim, hidden_dim) if use_shared_expert else None)


def lora_llama4_moe(dim: int, hidden_dim: int, num_experts: int = 8, experts_per_token: int = 1, use_shared_expert: bool = True, *, lora_rank: int, lora_alpha: float, lora_dropout: float = 0.0, ad: Optional[AdapterSpec] = None) -> MoE:
    """MoE whose experts and shared expert carry adapters; the router stays frozen and un-adapted."""
    ad = ad or AdapterSpec(apply_to_mlp=True, rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout)
    router = TokenChoiceTopKRouter(gate=Linear(dim, num_experts, bias=False), dim=dim, num_experts=num_experts, experts_per_token=experts_per_token)
    experts = LoRAGroupedExperts(dim=dim, hidden_dim=hidden_dim, rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, num_experts=num_experts)
    return MoE(experts=experts, router=router, shared_expert=build_mlp(dim, hidden_dim, ad) if use_shared_expert else None)


def _decoder(ad: Optional[AdapterSpec], *, vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, hidden_dim: int, max_seq_len: int, attn_dropout: float = 0.0,
             rope_base: int = 500_000, norm_eps: float = 1e-5, num_experts: int = 16, experts_per_token: int = 1, use_shared_expert: bool = True, use_qk_norm: bool = True,
             moe_every_n_layers: Optional[int] = None, mlp_hidden_dim: Optional[int] = None, skip_rope_interval: Optional[int] = None, attention_chunk_size: Optional[int] = None,
             use_scaled_rope: bool = False, rope_scale_factor: float = 16.0, rope_low_freq_factor: float = 1.0, rope_high_freq_factor: float = 1.0, old_context_len: int = 8192) -> TransformerDecoder:
    if skip_rope_interval is not None and attention_chunk_size is None:
        raise ValueError("Must pass local_chunk_size when enabling local chunked attention")
    if use_scaled_rope:
        rope = lambda hd, msl: Llama4ScaledRoPE(dim=hd, max_seq_len=msl, base=rope_base, scale_factor=rope_scale_factor, low_freq_factor=rope_low_freq_factor, high_freq_factor=rope_high_freq_factor, old_context_len=old_context_len)
    else:
        rope = lambda hd, msl: RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base)
    # layer i (0-based) is a local RoPE layer unless (i + 1) is a multiple of skip_rope_interval
    local = (lambda i: (i + 1) % skip_rope_interval != 0) if skip_rope_interval is not None else (lambda i: False)

    def mlp_factory(i: int, spec: AdapterSpec) -> nn.Module:
        if moe_every_n_layers is None or (i + 1) % moe_every_n_layers == 0:
            if spec.apply_to_mlp:
                return lora_llama4_moe(embed_dim, hidden_dim, num_experts, experts_per_token, use_shared_expert, lora_rank=spec.rank, lora_alpha=spec.alpha, lora_dropout=spec.dropout, ad=spec)
            return llama4_moe(embed_dim, hidden_dim, num_experts, experts_per_token, use_shared_expert)
        return build_mlp(embed_dim, mlp_hidden_dim, spec)

    arch = DecoderArch(
        vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads or num_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=hidden_dim,
        attn_dropout=attn_dropout, norm_eps=norm_eps, rope=rope, qk_norm=(lambda hd, eps: _UnitRMSNorm(eps)) if use_qk_norm else None,
        mlp_factory=mlp_factory, layer_uses_rope=local, layer_mask_mod=lambda i: chunked_mask_mod(attention_chunk_size) if local(i) else None,
    )
    return build_decoder(arch, ad)


def llama4_decoder(**kwargs) -> TransformerDecoder:
    """Keyword arguments: ``vocab_size, num_layers, num_heads, num_kv_heads, embed_dim, hidden_dim`` (expert
    width), ``max_seq_len, rope_base, norm_eps, num_experts, experts_per_token, use_shared_expert,
    use_qk_norm, moe_every_n_layers`` (+ ``mlp_hidden_dim`` for the dense layers in between),
    ``skip_rope_interval`` (every n-th layer is a global NoPE layer; the others use RoPE, unit q/k
    norm and attention restricted to ``attention_chunk_size`` blocks), ``use_scaled_rope`` and its
    scaling factors."""
    return _decoder(None, **kwargs)


def lora_llama4_decoder(lora_attn_modules: List[str], apply_lora_to_mlp: bool = False, apply_lora_to_output: bool = False, *, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0,
                        use_dora: bool = False, quantize_base: bool = False, **kwargs) -> TransformerDecoder:
    ad = adapter_from_kwargs(lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base)
    return _decoder(ad, **kwargs)


def llama4_vision_projection_head(*, decoder_embed_dim: int, clip_embed_dim: int, projection_embed_dim: int) -> Llama4VisionProjectionHead:
    factor = 0.5
    output = nn.Sequential(
        Linear(int(clip_embed_dim // (factor**2)), projection_embed_dim, bias=False), nn.GELU(),
        Linear(projection_embed_dim, projection_embed_dim, bias=False), nn.GELU(),
        Linear(projection_embed_dim, decoder_embed_dim, bias=False),
    )
    return Llama4VisionProjectionHead(output=output, pixel_shuffle_scaling_factor=factor)


def llama4_vision_encoder(*, patch_size: int, num_heads: int, clip_embed_dim: int, clip_num_layers: int, clip_hidden_states: Optional[List[int]] = None, projection_embed_dim: int,
                          decoder_embed_dim: int, tile_size: int, max_num_tiles: int = 1, in_channels: int = 3) -> Llama4VisionEncoder:
    clip = clip_vision_encoder(tile_size=tile_size, patch_size=patch_size, embed_dim=clip_embed_dim, num_layers=clip_num_layers, num_heads=num_heads, activation=nn.GELU, out_indices=clip_hidden_states,
                               max_num_tiles=max_num_tiles, in_channels=in_channels, attn_bias=True, output_cls_projection=False, append_cls_token=True, use_rope=True, use_tile_pos_embed=False)
    return Llama4VisionEncoder(clip=clip, projection_head=llama4_vision_projection_head(decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, projection_embed_dim=projection_embed_dim))


def lora_llama4_vision_projection_head(*, decoder_embed_dim: int, clip_embed_dim: int, projection_embed_dim: int, apply_lora_to_output: bool, lora_rank: int, lora_alpha: float,
                                       lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, **quantization_kwargs) -> Llama4VisionProjectionHead:
    """Projection head whose three linears carry adapters when ``apply_lora_to_output`` (they *are* the head's output path);
    otherwise the plain head (parity: torchtune/models/llama4/_component_builders.py:783-860)."""
    if not apply_lora_to_output:
        return llama4_vision_projection_head(decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, projection_embed_dim=projection_embed_dim)
    factor = 0.5
    cls = DoRALinear if use_dora else LoRALinear
    mk = lambda i, o: cls(i, o, rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_bias=False, quantize_base=quantize_base, **quantization_kwargs)
    output = nn.Sequential(mk(int(clip_embed_dim // (factor**2)), projection_embed_dim), nn.GELU(), mk(projection_embed_dim, projection_embed_dim), nn.GELU(),
                           mk(projection_embed_dim, decoder_embed_dim))
    return Llama4VisionProjectionHead(output=output, pixel_shuffle_scaling_factor=factor)


def lora_llama4_vision_encoder(encoder_lora: bool, fusion_lora: bool, lora_attn_modules: List[str], apply_lora_to_mlp: bool = False, apply_lora_to_output: bool = False, *, patch_size: int,
                               num_heads: int, clip_embed_dim: int, clip_num_layers: int, clip_hidden_states: Optional[List[int]] = None, projection_embed_dim: int, decoder_embed_dim: int,
                               tile_size: int, max_num_tiles: int = 1, in_channels: int = 3, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False,
                               quantize_base: bool = False, **quantization_kwargs) -> Llama4VisionEncoder:
    """Llama-4 vision encoder with adapters on the CLIP tower (``encoder_lora``) and / or the projection head (``fusion_lora``)
    (parity: torchtune/models/llama4/_component_builders.py:392-500)."""
    from ..clip._component_builders import _vision_encoder

    clip_kwargs = dict(tile_size=tile_size, patch_size=patch_size, embed_dim=clip_embed_dim, num_layers=clip_num_layers, num_heads=num_heads, activation=nn.GELU, cls_output_dim=512,
                       attn_bias=True, use_rope=True, out_indices=clip_hidden_states, output_cls_projection=False, max_num_tiles=max_num_tiles, in_channels=in_channels,
                       append_cls_token=True, use_tile_pos_embed=False)
    if encoder_lora:
        clip = _vision_encoder(**clip_kwargs, lora_modules=tuple(lora_attn_modules), lora=dict(rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora),
                               apply_lora_to_mlp=apply_lora_to_mlp, quantize_base=quantize_base)
    else:
        clip = _vision_encoder(**clip_kwargs)
    if fusion_lora:
        head = lora_llama4_vision_projection_head(decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, projection_embed_dim=projection_embed_dim,
                                                  apply_lora_to_output=apply_lora_to_output, lora_rank=lora_rank, lora_alpha=lora_alpha, lora_dropout=lora_dropout, use_dora=use_dora,
                                                  quantize_base=quantize_base, **quantization_kwargs)
    else:
        head = llama4_vision_projection_head(decoder_embed_dim=decoder_embed_dim, clip_embed_dim=clip_embed_dim, projection_embed_dim=projection_embed_dim)
    return Llama4VisionEncoder(clip=clip, projection_head=head)


def lora_llama4_self_attention(lora_modules: List[str], pos_embeddings: Optional[nn.Module], q_norm: Optional[nn.Module] = None, k_norm: Optional[nn.Module] = None, *,
                               head_dim: int, embed_dim: int, num_heads: int, num_kv_heads: int, max_seq_len: int, attn_dropout: float = 0.0,
                               lora_rank: int, lora_alpha: float, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False):
    """One decoder attention block with adapters on the listed projections; the caller passes the rotary embedding (``None`` on the
    layers that skip it) and the q/k norms (parity: torchtune/models/llama4/_component_builders.py:875-1017)."""
    from ...modules import MultiHeadAttention

    if not lora_modules:
        raise ValueError("lora_modules is empty: name at least one of q_proj, k_proj, v_proj, output_proj")
    ad = AdapterSpec(attn_modules=tuple(lora_modules), rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base)
    mods = set(lora_modules)
    unknown = mods - {"q_proj", "k_proj", "v_proj", "output_proj"}
    if unknown:
        raise ValueError(f"unknown attention modules for LoRA: {sorted(unknown)}")
    return MultiHeadAttention(
        embed_dim=embed_dim, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
        q_proj=ad.make(embed_dim, num_heads * head_dim, "q_proj" in mods), k_proj=ad.make(embed_dim, num_kv_heads * head_dim, "k_proj" in mods),
        v_proj=ad.make(embed_dim, num_kv_heads * head_dim, "v_proj" in mods), output_proj=ad.make(num_heads * head_dim, embed_dim, "output_proj" in mods),
        pos_embeddings=pos_embeddings, q_norm=q_norm, k_norm=k_norm, max_seq_len=max_seq_len, attn_dropout=attn_dropout,
    )


def lora_llama4_mlp(*, dim: int, hidden_dim: int, lora_rank: int, lora_alpha: float, lora_dropout: float = 0.0, quantize_base: bool = False, use_dora: bool = False) -> FeedForward:
    """Dense SwiGLU feed-forward with adapters on all three projections (parity: torchtune/models/llama4/_component_builders.py:1020-1060)."""
    return build_mlp(dim, hidden_dim, AdapterSpec(apply_to_mlp=True, rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base))

"""CLIP vision / text towers (parity: torchtune/models/clip/_component_builders.py:28-420)."""
from __future__ import annotations

from typing import Callable, List, Optional

from torch import nn

from ...modules import FeedForward, Fp32LayerNorm, FrozenNF4Linear, Linear, MultiHeadAttention, TransformerSelfAttentionLayer
from ...modules.peft import DoRALinear, LoRALinear
from ...modules.position_embeddings import VisionRotaryPositionalEmbeddings
from ...modules.vision_transformer import CLSProjection, VisionTransformer
from ._position_embeddings import TiledTokenPositionalEmbedding, TilePositionalEmbedding, TokenPositionalEmbedding
from ._text_encoder import CLIPTextEncoder, QuickGELU


def _proj(in_dim: int, out_dim: int, bias: bool, adapted: bool, lora: Optional[dict], quantize_base: bool = False) -> nn.Module:
    if adapted and lora is not None:
        cls = DoRALinear if lora.get("use_dora") else LoRALinear
        return cls(in_dim, out_dim, rank=lora["rank"], alpha=lora["alpha"], dropout=lora.get("dropout", 0.0), use_bias=bias, quantize_base=quantize_base)
    if quantize_base:
        return FrozenNF4Linear(in_dim, out_dim, bias=bias)
    return Linear(in_dim, out_dim, bias=bias)


def clip_mlp(in_dim: int, out_dim: int, hidden_dim: int, activation: nn.Module, quantize_base: bool = False, _lora: Optional[dict] = None) -> FeedForward:
    """Two-layer MLP ``down(act(gate(x)))`` with biases."""
    adapted = _lora is not None
    return FeedForward(
        gate_proj=_proj(in_dim, hidden_dim, True, adapted, _lora, quantize_base),
        down_proj=_proj(hidden_dim, out_dim, True, adapted, _lora, quantize_base),
        up_proj=None,
        activation=activation,
    )


def _vision_encoder(
    *, tile_size: int, patch_size: int, embed_dim: int, num_layers: int, num_heads: int, activation: Callable, cls_output_dim: int, attn_bias: bool, use_rope: bool,
    out_indices: Optional[List[int]], output_cls_projection: bool, max_num_tiles: int, in_channels: int, append_cls_token: bool, use_tile_pos_embed: bool,
    lora_modules: tuple = (), lora: Optional[dict] = None, apply_lora_to_mlp: bool = False, quantize_base: bool = False,
) -> VisionTransformer:
    if embed_dim % num_heads != 0:
        raise ValueError(f"embed_dim must be divisible by num_heads, got {embed_dim} and {num_heads}")
    head_dim = embed_dim // num_heads
    rope = VisionRotaryPositionalEmbeddings(patch_size=patch_size, tile_size=tile_size, max_num_tiles=max_num_tiles, dim=head_dim, base=10_000, append_cls_token=append_cls_token) if use_rope else None
    attn = MultiHeadAttention(
        embed_dim=embed_dim, num_heads=num_heads, num_kv_heads=num_heads, head_dim=head_dim,
        q_proj=_proj(embed_dim, embed_dim, attn_bias, "q_proj" in lora_modules, lora, quantize_base),
        k_proj=_proj(embed_dim, embed_dim, attn_bias, "k_proj" in lora_modules, lora, quantize_base),
        v_proj=_proj(embed_dim, embed_dim, attn_bias, "v_proj" in lora_modules, lora, quantize_base),
        output_proj=_proj(embed_dim, embed_dim, attn_bias, "output_proj" in lora_modules, lora, quantize_base),
        pos_embeddings=rope, attn_dropout=0.0, is_causal=False,
    )
    mlp = clip_mlp(embed_dim, embed_dim, 4 * embed_dim, activation(), quantize_base=quantize_base, _lora=lora if apply_lora_to_mlp else None)
    layer = TransformerSelfAttentionLayer(attn=attn, mlp=mlp, sa_norm=Fp32LayerNorm(embed_dim, eps=1e-5), mlp_norm=Fp32LayerNorm(embed_dim, eps=1e-5))
    if use_tile_pos_embed and max_num_tiles > 1:
        pre = TilePositionalEmbedding(max_num_tiles=max_num_tiles, embed_dim=embed_dim)
        post = TilePositionalEmbedding(max_num_tiles=max_num_tiles, embed_dim=embed_dim)
        tok = TiledTokenPositionalEmbedding(max_num_tiles=max_num_tiles, embed_dim=embed_dim, patch_size=patch_size, tile_size=tile_size)
    else:
        pre = post = None
        tok = TokenPositionalEmbedding(embed_dim=embed_dim, patch_size=patch_size, tile_size=tile_size)
    return VisionTransformer(
        num_layers=num_layers, layer=layer, token_pos_embedding=tok, pre_tile_pos_embed=pre, post_tile_pos_embed=post,
        cls_projection=CLSProjection(embed_dim=embed_dim, cls_output_dim=cls_output_dim) if output_cls_projection else None,
        out_indices=out_indices, tile_size=tile_size, patch_size=patch_size, embed_dim=embed_dim, in_channels=in_channels, append_cls_token=append_cls_token,
    )


def clip_vision_encoder(
    tile_size: int, patch_size: int, embed_dim: int, num_layers: int, num_heads: int, activation: Callable = nn.SiLU, cls_output_dim: int = 512, attn_bias: bool = True,
    use_rope: bool = False, out_indices: Optional[List[int]] = None, output_cls_projection: bool = False, max_num_tiles: int = 4, in_channels: int = 3,
    append_cls_token: bool = False, use_tile_pos_embed: bool = True,
) -> VisionTransformer:
    """Tiled ViT: patch GEMM → (+tile / token position embeddings, CLS) → ``num_layers`` bidirectional
    layers → optional CLS projection; ``out_indices`` selects intermediate hidden states to return."""
    return _vision_encoder(
        tile_size=tile_size, patch_size=patch_size, embed_dim=embed_dim, num_layers=num_layers, num_heads=num_heads, activation=activation, cls_output_dim=cls_output_dim,
        attn_bias=attn_bias, use_rope=use_rope, out_indices=out_indices, output_cls_projection=output_cls_projection, max_num_tiles=max_num_tiles, in_channels=in_channels,
        append_cls_token=append_cls_token, use_tile_pos_embed=use_tile_pos_embed,
    )


def lora_clip_vision_encoder(
    lora_modules: List[str], apply_lora_to_mlp: bool = False, *, tile_size: int, patch_size: int, embed_dim: int, num_layers: int, num_heads: int,
    activation: Callable = nn.SiLU, cls_output_dim: int = 512, attn_bias: bool = False, out_indices: Optional[List[int]] = None, output_cls_projection: bool = False,
    max_num_tiles: int = 4, in_channels: int = 3, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, **_,
) -> VisionTransformer:
    lora = dict(rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora)
    return _vision_encoder(
        tile_size=tile_size, patch_size=patch_size, embed_dim=embed_dim, num_layers=num_layers, num_heads=num_heads, activation=activation, cls_output_dim=cls_output_dim,
        attn_bias=attn_bias, use_rope=False, out_indices=out_indices, output_cls_projection=output_cls_projection, max_num_tiles=max_num_tiles, in_channels=in_channels,
        append_cls_token=False, use_tile_pos_embed=True, lora_modules=tuple(lora_modules), lora=lora, apply_lora_to_mlp=apply_lora_to_mlp, quantize_base=quantize_base,
    )


def clip_text_encoder(embed_dim: int, num_heads: int, num_layers: int, vocab_size: int = 49408, max_seq_len: int = 77, norm_eps: float = 1e-5) -> CLIPTextEncoder:
    attn = MultiHeadAttention(
        embed_dim=embed_dim, num_heads=num_heads, num_kv_heads=num_heads, head_dim=embed_dim // num_heads,
        q_proj=Linear(embed_dim, embed_dim), k_proj=Linear(embed_dim, embed_dim), v_proj=Linear(embed_dim, embed_dim), output_proj=Linear(embed_dim, embed_dim),
    )
    layer = TransformerSelfAttentionLayer(attn=attn, mlp=clip_mlp(embed_dim, embed_dim, embed_dim * 4, QuickGELU()), sa_norm=nn.LayerNorm(embed_dim, eps=norm_eps), mlp_norm=nn.LayerNorm(embed_dim, eps=norm_eps))
    return CLIPTextEncoder(layer=layer, final_norm=nn.LayerNorm(embed_dim, eps=norm_eps), vocab_size=vocab_size, max_seq_len=max_seq_len, embed_dim=embed_dim, num_layers=num_layers)


def _check_modules(lora_modules) -> tuple:
    if not lora_modules:
        raise ValueError("lora_modules is empty: name at least one of q_proj, k_proj, v_proj, output_proj")
    unknown = set(lora_modules) - {"q_proj", "k_proj", "v_proj", "output_proj"}
    if unknown:
        raise ValueError(f"unknown attention modules for LoRA: {sorted(unknown)}")
    return tuple(lora_modules)


def lora_clip_attention(lora_modules: List[str], *, embed_dim: int, head_dim: int, num_heads: int, num_kv_heads: int, attn_dropout: float = 0.0, attn_bias: bool = False,
                        lora_rank: int, lora_alpha: float, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False) -> MultiHeadAttention:
    """One bidirectional attention block of the vision tower with adapters on the listed projections
    (parity: torchtune/models/clip/_component_builders.py:440-600)."""
    mods = _check_modules(lora_modules)
    lora = dict(rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora)
    return MultiHeadAttention(
        embed_dim=embed_dim, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
        q_proj=_proj(embed_dim, num_heads * head_dim, attn_bias, "q_proj" in mods, lora, quantize_base),
        k_proj=_proj(embed_dim, num_kv_heads * head_dim, attn_bias, "k_proj" in mods, lora, quantize_base),
        v_proj=_proj(embed_dim, num_kv_heads * head_dim, attn_bias, "v_proj" in mods, lora, quantize_base),
        output_proj=_proj(num_heads * head_dim, embed_dim, attn_bias, "output_proj" in mods, lora, quantize_base),
        pos_embeddings=None, attn_dropout=attn_dropout, is_causal=False,
    )


def lora_clip_mlp(*, in_dim: int, out_dim: int, hidden_dim: int, activation: nn.Module, lora_rank: int, lora_alpha: float, lora_dropout: float = 0.0,
                  use_dora: bool = False, quantize_base: bool = False) -> FeedForward:
    """The tower's two-layer MLP with adapters on both projections (parity: torchtune/models/clip/_component_builders.py:603-660)."""
    return clip_mlp(in_dim, out_dim, hidden_dim, activation, quantize_base=quantize_base,
                    _lora=dict(rank=lora_rank, alpha=lora_alpha, dropout=lora_dropout, use_dora=use_dora))

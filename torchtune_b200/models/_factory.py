"""One parametric decoder factory shared by every dense decoder-only family.

The reference repeats a ``<family>()`` / ``lora_<family>()`` builder pair per model
family (e.g. torchtune/models/llama3_1/_component_builders.py:41-122 and :138-330,
torchtune/models/qwen2/_component_builders.py, torchtune/models/mistral/…).  Here a
single :func:`build_decoder` takes an architecture description plus an optional
adapter description and produces the same module tree / state-dict keys
(``layers.N.attn.q_proj.weight``, ``layers.N.mlp.w1.weight``, ``layers.N.sa_norm.scale``,
``tok_embeddings.weight``, ``norm.scale``, ``output.weight``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch
from torch import nn

from ..modules import (
    FeedForward,
    FrozenNF4Linear,
    Linear,
    MultiHeadAttention,
    RMSNorm,
    TiedLinear,
    TransformerDecoder,
    TransformerSelfAttentionLayer,
)
from ..modules.common_utils import _register_reparametrize_state_dict_hooks
from ..modules.peft import DoRALinear, LoRALinear


def scale_hidden_dim_for_mlp(dim: int, multiple_of: int = 256) -> int:
    """SwiGLU hidden size ``4·⌊2·dim/3⌋`` rounded up to ``multiple_of``
    (torchtune/models/llama3/_model_utils.py:8-23)."""
    hidden = 4 * int(2 * dim / 3)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


@dataclass
class AdapterSpec:
    """Which projections receive a low-rank adapter and how the base is stored."""

    attn_modules: Sequence[str] = ()
    apply_to_mlp: bool = False
    apply_to_output: bool = False
    rank: int = 8
    alpha: float = 16
    dropout: float = 0.0
    use_dora: bool = False
    quantize_base: bool = False

    def make(self, in_dim: int, out_dim: int, adapted: bool, bias: bool = False) -> nn.Module:
        if adapted:
            cls = DoRALinear if self.use_dora else LoRALinear
            return cls(in_dim, out_dim, rank=self.rank, alpha=self.alpha, dropout=self.dropout, use_bias=bias, quantize_base=self.quantize_base)
        if self.quantize_base and not bias:
            return FrozenNF4Linear(in_dim, out_dim, bias=False)
        return Linear(in_dim, out_dim, bias=bias)


@dataclass
class DecoderArch:
    vocab_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    embed_dim: int
    max_seq_len: int
    intermediate_dim: Optional[int] = None
    head_dim: Optional[int] = None
    attn_dropout: float = 0.0
    norm_eps: float = 1e-5
    rope: Optional[Callable[[int, int], nn.Module]] = None  # (head_dim, max_seq_len) -> module
    norm: Callable[[int, float], nn.Module] = lambda dim, eps: RMSNorm(dim, eps=eps)
    qkv_bias: bool = False
    qk_norm: Optional[Callable[[int, float], nn.Module]] = None  # per-head q/k norm (Qwen3)
    tie_embeddings: bool = False
    embedding: Callable[[int, int], nn.Module] = lambda v, d: nn.Embedding(v, d)
    activation: Callable[[], nn.Module] = nn.SiLU
    mlp_bias: bool = False
    qk_norm_before_rope: bool = False  # Qwen3 normalises q/k per head before the rotation
    post_norms: bool = False  # Gemma-2: extra norms on the attention / MLP outputs (sa_scale, mlp_scale)
    final_norm: Optional[Callable[[int, float], nn.Module]] = None  # defaults to `norm`
    attn_softcap: float = 0.0
    logit_softcap: float = 0.0  # cap·tanh(logits/cap) on the output logits (Gemma-2)
    attn_scale: Optional[float] = None
    sliding_window: Optional[Callable[[int], int]] = None  # layer index -> window (0 = global)
    # per-layer overrides (Llama-4): feed-forward module, whether the layer rotates/normalises q and k,
    # and an extra mask hook
    mlp_factory: Optional[Callable[[int, "AdapterSpec"], nn.Module]] = None
    layer_uses_rope: Optional[Callable[[int], bool]] = None
    layer_mask_mod: Optional[Callable[[int], Optional[Callable]]] = None

    def resolved_head_dim(self) -> int:
        return self.head_dim or self.embed_dim // self.num_heads

    def resolved_hidden(self) -> int:
        return self.intermediate_dim or scale_hidden_dim_for_mlp(self.embed_dim)


def build_attention(arch: DecoderArch, ad: AdapterSpec, rope: Optional[nn.Module], positional: bool = True) -> MultiHeadAttention:
    hd = arch.resolved_head_dim()
    qk_norm = arch.qk_norm if positional else None
    rope = rope if positional else None
    mods = set(ad.attn_modules)
    unknown = mods - {"q_proj", "k_proj", "v_proj", "output_proj"}
    if unknown:
        raise ValueError(f"unknown attention modules for LoRA: {sorted(unknown)}")
    return MultiHeadAttention(
        embed_dim=arch.embed_dim,
        num_heads=arch.num_heads,
        num_kv_heads=arch.num_kv_heads,
        head_dim=hd,
        q_proj=ad.make(arch.embed_dim, arch.num_heads * hd, "q_proj" in mods, arch.qkv_bias),
        k_proj=ad.make(arch.embed_dim, arch.num_kv_heads * hd, "k_proj" in mods, arch.qkv_bias),
        v_proj=ad.make(arch.embed_dim, arch.num_kv_heads * hd, "v_proj" in mods, arch.qkv_bias),
        output_proj=ad.make(arch.num_heads * hd, arch.embed_dim, "output_proj" in mods, False),
        pos_embeddings=rope,
        q_norm=qk_norm(hd, arch.norm_eps) if qk_norm else None,
        k_norm=qk_norm(hd, arch.norm_eps) if qk_norm else None,
        max_seq_len=arch.max_seq_len,
        attn_dropout=arch.attn_dropout,
        softcap=arch.attn_softcap,
        scale=arch.attn_scale,
        qk_norm_before_rope=arch.qk_norm_before_rope,
    )


def _window_mask_mod(window: int):
    """Per-layer mask hook adding a sliding window to whatever mask the batch carries."""
    from dataclasses import replace

    from ..ops.mask import AttentionMask

    def mod(mask, bsz, seq_len):
        if mask is None:
            return AttentionMask(causal=True, window=window)
        if isinstance(mask, AttentionMask) and mask.bool_mask is None:
            return replace(mask, window=window)
        dense = mask.bool_mask if isinstance(mask, AttentionMask) else mask
        q = torch.arange(dense.shape[-2], device=dense.device).view(-1, 1) + (dense.shape[-1] - dense.shape[-2])
        k = torch.arange(dense.shape[-1], device=dense.device).view(1, -1)
        return dense & ((q - k) < window)

    return mod


def build_mlp(dim: int, hidden: int, ad: AdapterSpec, activation: Optional[nn.Module] = None, bias: bool = False) -> FeedForward:
    return FeedForward(
        gate_proj=ad.make(dim, hidden, ad.apply_to_mlp, bias),
        down_proj=ad.make(hidden, dim, ad.apply_to_mlp, bias),
        up_proj=ad.make(dim, hidden, ad.apply_to_mlp, bias),
        activation=activation if activation is not None else nn.SiLU(),
    )


def build_decoder(arch: DecoderArch, adapter: Optional[AdapterSpec] = None) -> TransformerDecoder:
    ad = adapter or AdapterSpec()
    hd = arch.resolved_head_dim()
    rope = arch.rope(hd, arch.max_seq_len) if arch.rope else None  # one instance shared by all layers
    layers: List[nn.Module] = []
    for idx in range(arch.num_layers):
        window = arch.sliding_window(idx) if arch.sliding_window else 0
        positional = arch.layer_uses_rope(idx) if arch.layer_uses_rope else True
        mask_mod = _window_mask_mod(window) if window else None
        if arch.layer_mask_mod is not None and mask_mod is None:
            mask_mod = arch.layer_mask_mod(idx)
        mlp = arch.mlp_factory(idx, ad) if arch.mlp_factory else build_mlp(arch.embed_dim, arch.resolved_hidden(), ad, arch.activation(), arch.mlp_bias)
        layers.append(
            TransformerSelfAttentionLayer(
                attn=build_attention(arch, ad, rope, positional),
                mlp=mlp,
                sa_norm=arch.norm(arch.embed_dim, arch.norm_eps),
                mlp_norm=arch.norm(arch.embed_dim, arch.norm_eps),
                sa_scale=arch.norm(arch.embed_dim, arch.norm_eps) if arch.post_norms else None,
                mlp_scale=arch.norm(arch.embed_dim, arch.norm_eps) if arch.post_norms else None,
                mask_mod=mask_mod,
            )
        )
    tok = arch.embedding(arch.vocab_size, arch.embed_dim)
    if arch.tie_embeddings:
        if ad.apply_to_output:
            raise ValueError("apply_lora_to_output is incompatible with tied embeddings")
        output = TiedLinear(tok)
    elif ad.apply_to_output:
        # the output projection is never NF4-quantised
        cls = DoRALinear if ad.use_dora else LoRALinear
        output = cls(arch.embed_dim, arch.vocab_size, rank=ad.rank, alpha=ad.alpha, dropout=ad.dropout)
    else:
        output = Linear(arch.embed_dim, arch.vocab_size, bias=False)
    model = TransformerDecoder(
        tok_embeddings=tok,
        layers=layers,
        max_seq_len=arch.max_seq_len,
        num_heads=arch.num_heads,
        head_dim=hd,
        norm=(arch.final_norm or arch.norm)(arch.embed_dim, arch.norm_eps),
        output=output,
    )
    model.logit_softcap = float(arch.logit_softcap)
    if ad.quantize_base:
        # checkpoints of a quantised-base model are written in bf16 on CPU
        _register_reparametrize_state_dict_hooks(model, dtype=tok.weight.dtype)
    return model


def adapter_from_kwargs(
    lora_attn_modules: Sequence[str],
    apply_lora_to_mlp: bool = False,
    apply_lora_to_output: bool = False,
    lora_rank: int = 8,
    lora_alpha: float = 16,
    lora_dropout: float = 0.0,
    use_dora: bool = False,
    quantize_base: bool = False,
) -> AdapterSpec:
    return AdapterSpec(
        attn_modules=tuple(lora_attn_modules),
        apply_to_mlp=apply_lora_to_mlp,
        apply_to_output=apply_lora_to_output,
        rank=lora_rank,
        alpha=lora_alpha,
        dropout=lora_dropout,
        use_dora=use_dora,
        quantize_base=quantize_base,
    )

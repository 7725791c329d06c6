"""Gemma-2 HF ↔ native conversion (parity: torchtune/models/gemma2/_convert_weights.py:20-140):
the generic Llama-style map plus the two post-norms and the wrapped final norm."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..convert_weights import _FROM_HF, _invert, _to_half_split, _to_interleaved, get_mapped_key

_FROM_HF_GEMMA2 = {
    **_FROM_HF,
    "model.layers.{}.post_attention_layernorm.weight": "layers.{}.sa_scale.scale",
    "model.layers.{}.pre_feedforward_layernorm.weight": "layers.{}.mlp_norm.scale",
    "model.layers.{}.post_feedforward_layernorm.weight": "layers.{}.mlp_scale.scale",
    "model.norm.weight": "norm.rms_norm.scale",
}


def gemma2_hf_to_tune(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    out = {}
    for k, v in state_dict.items():
        if "rotary_emb.inv_freq" in k or k == "lm_head.weight":
            continue
        nk = get_mapped_key(k, _FROM_HF_GEMMA2)
        if nk.endswith("attn.q_proj.weight"):
            v = _to_interleaved(v, num_heads, head_dim)
        elif nk.endswith("attn.k_proj.weight"):
            v = _to_interleaved(v, num_kv_heads, head_dim)
        out[nk] = v
    return out


def gemma2_tune_to_hf(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    inv = _invert(_FROM_HF_GEMMA2)
    out = {}
    for k, v in state_dict.items():
        if k.endswith("attn.q_proj.weight"):
            v = _to_half_split(v, num_heads, head_dim)
        elif k.endswith("attn.k_proj.weight"):
            v = _to_half_split(v, num_kv_heads, head_dim)
        out[get_mapped_key(k, inv)] = v
    return out


def _register() -> None:
    from ...training.checkpointing._codecs import _llama_args, register_hf_codec
    from ...training.checkpointing._utils import ModelType

    register_hf_codec(ModelType.GEMMA2, lambda sd, cfg: gemma2_hf_to_tune(sd, **_llama_args(cfg)), lambda sd, cfg: gemma2_tune_to_hf(sd, **_llama_args(cfg)))


_register()

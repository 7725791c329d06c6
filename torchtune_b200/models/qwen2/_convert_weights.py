"""Qwen2 / Qwen3 HF ↔ native key conversion (parity: torchtune/models/qwen2/_convert_weights.py:13-137,
torchtune/models/qwen3/_convert_weights.py:19-140).  RoPE is half-split on both sides, so no
row permutation is needed; q/k/v biases and per-head q/k norms map one to one; a tied
``lm_head.weight`` is dropped on load and not written on save."""
from __future__ import annotations

from typing import Dict

import torch

from ..convert_weights import _FROM_HF, _invert, get_mapped_key

_EXTRA = {
    **{f"model.layers.{{}}.self_attn.{p}_proj.bias": f"layers.{{}}.attn.{p}_proj.bias" for p in ("q", "k", "v")},
    "model.layers.{}.self_attn.q_norm.weight": "layers.{}.attn.q_norm.scale",
    "model.layers.{}.self_attn.k_norm.weight": "layers.{}.attn.k_norm.scale",
}
_FROM_HF_QWEN = {**_FROM_HF, **_EXTRA}
QWEN2_TIED_KEY = "lm_head.weight"


def qwen2_hf_to_tune(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: int = None, tie_word_embeddings: bool = False) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in state_dict.items():
        if "rotary_emb.inv_freq" in k or (tie_word_embeddings and k == QWEN2_TIED_KEY):
            continue
        nk = get_mapped_key(k, _FROM_HF_QWEN)
        if nk is not None:
            out[nk] = v
    return out


def qwen2_tune_to_hf(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: int = None, tie_word_embeddings: bool = False) -> Dict[str, torch.Tensor]:
    inv = _invert(_FROM_HF_QWEN)
    out = {}
    for k, v in state_dict.items():
        if tie_word_embeddings and k == "output.weight":
            continue
        out[get_mapped_key(k, inv)] = v
    return out


qwen3_hf_to_tune = qwen2_hf_to_tune
qwen3_tune_to_hf = qwen2_tune_to_hf


def _register() -> None:
    from ...training.checkpointing._codecs import register_hf_codec
    from ...training.checkpointing._utils import ModelType

    def to_native(sd, cfg):
        return qwen2_hf_to_tune(sd, tie_word_embeddings=cfg.get("tie_word_embeddings", False))

    def from_native(sd, cfg):
        return qwen2_tune_to_hf(sd, tie_word_embeddings=cfg.get("tie_word_embeddings", False))

    register_hf_codec(ModelType.QWEN2, to_native, from_native)
    register_hf_codec(ModelType.QWEN3, to_native, from_native)


_register()

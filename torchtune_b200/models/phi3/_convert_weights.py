"""Phi-3 / Phi-4 HF ↔ native conversion (parity: torchtune/models/phi3/_convert_weights.py:15-104).
HF stores ``qkv_proj`` and ``gate_up_proj`` fused; they are split on load and re-fused on save.
RoPE is half-split on both sides (no permutation)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..convert_weights import _invert, get_mapped_key

_PHI3_FROM_HF = {
    "model.embed_tokens.weight": "tok_embeddings.weight",
    "model.layers.{}.self_attn.qkv_proj.weight": "layers.{}.attn.q_proj.weight",
    "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attn.output_proj.weight",
    "model.layers.{}.mlp.gate_up_proj.weight": "layers.{}.mlp.w1.weight",
    "model.layers.{}.mlp.down_proj.weight": "layers.{}.mlp.w2.weight",
    "model.layers.{}.input_layernorm.weight": "layers.{}.sa_norm.scale",
    "model.layers.{}.post_attention_layernorm.weight": "layers.{}.mlp_norm.scale",
    "model.norm.weight": "norm.scale",
    "lm_head.weight": "output.weight",
}


def phi3_hf_to_tune(state_dict: Dict[str, torch.Tensor], num_heads: Optional[int] = None, num_kv_heads: Optional[int] = None, dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    out = {}
    gqa = num_heads is not None and num_kv_heads is not None and num_heads != num_kv_heads
    if gqa and dim is None:
        raise ValueError("Phi models with GQA require dim, num_heads and num_kv_heads to be specified")
    for k, v in state_dict.items():
        nk = get_mapped_key(k, _PHI3_FROM_HF)
        if "qkv" in k:
            if gqa:
                q_rows = dim
                kv_rows = dim // num_heads * num_kv_heads
                q, kk, vv = v.split([q_rows, kv_rows, kv_rows], dim=0)
            else:
                q, kk, vv = v.chunk(3, dim=0)
            out[nk] = q
            out[nk.replace("q_proj", "k_proj")] = kk
            out[nk.replace("q_proj", "v_proj")] = vv
        elif "gate" in k:
            w1, w3 = v.chunk(2, dim=0)
            out[nk] = w1
            out[nk.replace("w1", "w3")] = w3
        else:
            out[nk] = v
    return out


def phi3_tune_to_hf(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    inv = _invert(_PHI3_FROM_HF)
    out = {}
    for k, v in state_dict.items():
        if "k_proj" in k or "v_proj" in k or ".w3." in k:
            continue  # folded into the fused tensors below
        nk = get_mapped_key(k, inv)
        if "q_proj" in k:
            v = torch.cat([v, state_dict[k.replace("q_proj", "k_proj")], state_dict[k.replace("q_proj", "v_proj")]], dim=0)
        elif ".w1." in k:
            v = torch.cat([v, state_dict[k.replace("w1", "w3")]], dim=0)
        out[nk] = v
    return out


def _register() -> None:
    from ...training.checkpointing._codecs import register_hf_codec
    from ...training.checkpointing._utils import ModelType

    def to_native(sd, cfg):
        return phi3_hf_to_tune(sd, num_heads=cfg.get("num_attention_heads"), num_kv_heads=cfg.get("num_key_value_heads"), dim=cfg.get("hidden_size"))

    for mt in (ModelType.PHI3_MINI, ModelType.PHI4):
        register_hf_codec(mt, to_native, lambda sd, cfg: phi3_tune_to_hf(sd))


_register()

"""HF ↔ native conversion for reward models: a Llama-style trunk whose head is a single-row
``score.weight`` (parity: torchtune/rlhf/utils/_convert_weights.py:27-140)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ...models.convert_weights import _FROM_HF, _invert, _to_half_split, _to_interleaved, get_mapped_key

_REWARD = {k: v for k, v in _FROM_HF.items() if k != "lm_head.weight"}
_REWARD["score.weight"] = "output.weight"


def reward_hf_to_tune(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    out = {}
    for k, v in state_dict.items():
        if "rotary_emb.inv_freq" in k:
            continue
        nk = get_mapped_key(k, _REWARD)
        if nk.endswith("attn.q_proj.weight"):
            v = _to_interleaved(v, num_heads, head_dim)
        elif nk.endswith("attn.k_proj.weight"):
            v = _to_interleaved(v, num_kv_heads, head_dim)
        out[nk] = v
    return out


def reward_tune_to_hf(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    inv = _invert(_REWARD)
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

    register_hf_codec(ModelType.REWARD, lambda sd, cfg: reward_hf_to_tune(sd, **_llama_args(cfg)), lambda sd, cfg: reward_tune_to_hf(sd, **_llama_args(cfg)))


_register()

"""Checkpoint key/layout conversion between this package's state dicts and the HF
``transformers`` and Meta ("consolidated") formats, plus PEFT adapter export.

Parity: torchtune/models/convert_weights.py:14-309.  RoPE here rotates interleaved
pairs, HF rotates half-split pairs, so q/k projection rows are permuted per head when
crossing the HF boundary; the two permutations are exact inverses.
"""
from __future__ import annotations

import re
from typing import Any, Dict, Iterable, Optional, Tuple

import torch

# (external name, internal name); "{}" stands for the layer index
_ATTN = (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("o", "output_proj"))
_META_PAIRS: Tuple[Tuple[str, str], ...] = (
    ("tok_embeddings.weight", "tok_embeddings.weight"),
    ("norm.weight", "norm.scale"),
    ("output.weight", "output.weight"),
    ("layers.{}.attention_norm.weight", "layers.{}.sa_norm.scale"),
    ("layers.{}.ffn_norm.weight", "layers.{}.mlp_norm.scale"),
    *((f"layers.{{}}.attention.w{m}.weight", f"layers.{{}}.attn.{t}.weight") for m, t in _ATTN),
    *((f"layers.{{}}.feed_forward.w{i}.weight", f"layers.{{}}.mlp.w{i}.weight") for i in (1, 2, 3)),
    *(
        (f"layers.{{}}.attention.w{m}.lora_{ab}.weight", f"layers.{{}}.attn.{t}.lora_{ab}.weight")
        for m, t in _ATTN
        for ab in ("a", "b")
    ),
)
_HF_PAIRS: Tuple[Tuple[str, Optional[str]], ...] = (
    ("model.embed_tokens.weight", "tok_embeddings.weight"),
    ("model.norm.weight", "norm.scale"),
    ("lm_head.weight", "output.weight"),
    ("model.layers.{}.input_layernorm.weight", "layers.{}.sa_norm.scale"),
    ("model.layers.{}.post_attention_layernorm.weight", "layers.{}.mlp_norm.scale"),
    ("model.layers.{}.self_attn.rotary_emb.inv_freq", None),
    *((f"model.layers.{{}}.self_attn.{m}_proj.weight", f"layers.{{}}.attn.{t}.weight") for m, t in _ATTN),
    ("model.layers.{}.mlp.gate_proj.weight", "layers.{}.mlp.w1.weight"),
    ("model.layers.{}.mlp.down_proj.weight", "layers.{}.mlp.w2.weight"),
    ("model.layers.{}.mlp.up_proj.weight", "layers.{}.mlp.w3.weight"),
)
_FROM_META: Dict[str, Optional[str]] = dict(_META_PAIRS)
_FROM_HF: Dict[str, Optional[str]] = dict(_HF_PAIRS)

_NUM = re.compile(r"(?<=\.)\d+(?=\.)")


def get_mapped_key(key: str, mapping_dict: Dict[str, Optional[str]]) -> Optional[str]:
    """Translate ``key`` through ``mapping_dict`` whose entries use ``{}`` for every numeric
    path component (layer / expert index)."""
    numbers = _NUM.findall(key)
    template = _NUM.sub("{}", key) if numbers else key
    if template not in mapping_dict:
        raise Exception(
            f'Error converting the state dict. Found unexpected key: "{key}". '
            "Please make sure you're loading a checkpoint with the right format. "
        )
    target = mapping_dict[template]
    return None if target is None else target.format(*numbers) if numbers else target


def _invert(mapping: Dict[str, Optional[str]]) -> Dict[str, str]:
    return {v: k for k, v in mapping.items() if v is not None}


def meta_to_tune(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in state_dict.items():
        if k == "rope.freqs":
            continue
        out[get_mapped_key(k, _FROM_META)] = v
    return out


def tune_to_meta(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    inv = _invert(_FROM_META)
    return {get_mapped_key(k, inv): v for k, v in state_dict.items()}


def _to_interleaved(w: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """HF rows ``[h][half][i]`` → interleaved rows ``[h][i][half]``."""
    rest = w.shape[1:]
    return w.view(n_heads, 2, head_dim // 2, *rest).transpose(1, 2).reshape(n_heads * head_dim, *rest)


def _to_half_split(w: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    rest = w.shape[1:]
    return w.view(n_heads, head_dim // 2, 2, *rest).transpose(1, 2).reshape(n_heads * head_dim, *rest)


def hf_to_tune(
    state_dict: Dict[str, torch.Tensor],
    num_heads: int = 32,
    num_kv_heads: int = 32,
    dim: int = 4096,
    head_dim: Optional[int] = None,
) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    out: Dict[str, torch.Tensor] = {}
    for k, v in state_dict.items():
        if "rotary_emb.inv_freq" in k:
            continue
        nk = get_mapped_key(k, _FROM_HF)
        if nk is None:
            continue
        if nk.endswith("attn.q_proj.weight"):
            v = _to_interleaved(v, num_heads, head_dim)
        elif nk.endswith("attn.k_proj.weight"):
            v = _to_interleaved(v, num_kv_heads, head_dim)
        out[nk] = v
    return out


def tune_to_hf(
    state_dict: Dict[str, torch.Tensor],
    num_heads: int = 32,
    num_kv_heads: int = 32,
    dim: int = 4096,
    head_dim: Optional[int] = None,
) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    inv = _invert(_FROM_HF)
    out: Dict[str, torch.Tensor] = {}
    for k, v in state_dict.items():
        nk = get_mapped_key(k, inv)
        if k.endswith("attn.q_proj.weight"):
            v = _to_half_split(v, num_heads, head_dim)
        elif k.endswith("attn.k_proj.weight"):
            v = _to_half_split(v, num_kv_heads, head_dim)
        out[nk] = v
    return out


# ---------------------------------------------------------------------------
# PEFT export
# ---------------------------------------------------------------------------
_TO_PEFT_KEYS = {"lora_a": "lora_A", "lora_b": "lora_B", "magnitude": "lora_magnitude_vector"}
_TO_PEFT_TARGET_MODULES = {
    "q_proj": "q_proj",
    "k_proj": "k_proj",
    "v_proj": "v_proj",
    "output_proj": "o_proj",
    "w1": "gate_proj",
    "w2": "down_proj",
    "w3": "up_proj",
    "output": "lm_head",
}
_PEFT_CONFIG_EXPECTED_KEYS = ["target_modules", "r", "lora_alpha"]


def tune_to_peft_adapter_config(adapter_config: Dict[str, Any], base_model_name_or_path: Optional[str] = None) -> Dict[str, Any]:
    if not all(k in adapter_config for k in _PEFT_CONFIG_EXPECTED_KEYS):
        raise ValueError(f"PEFT adapter config requires {_PEFT_CONFIG_EXPECTED_KEYS}, found {adapter_config.keys()}")
    bad = [m for m in adapter_config["target_modules"] if m not in _TO_PEFT_TARGET_MODULES]
    if bad:
        raise ValueError(f"Unknown target module {bad[0]}")
    adapter_config["target_modules"] = [_TO_PEFT_TARGET_MODULES[m] for m in adapter_config["target_modules"]]
    if base_model_name_or_path:
        adapter_config["base_model_name_or_path"] = base_model_name_or_path
    return adapter_config


def _peft_key_map() -> Dict[str, str]:
    table: Dict[str, str] = {}
    for hf_name, ours in _FROM_HF.items():
        if ours is None or not ours.endswith(".weight"):
            continue
        for mine, theirs in _TO_PEFT_KEYS.items():
            if mine == "magnitude":
                table[ours[: -len("weight")] + mine] = hf_name[: -len("weight")] + theirs
            else:
                table[ours[: -len("weight")] + f"{mine}.weight"] = hf_name[: -len("weight")] + f"{theirs}.weight"
    return table


def tune_to_peft_adapter_weights(
    state_dict: Dict[str, torch.Tensor],
    num_heads: int = 32,
    num_kv_heads: int = 32,
    dim: int = 4096,
    head_dim: Optional[int] = None,
) -> Dict[str, torch.Tensor]:
    """Rename adapter tensors to PEFT's names (prefixed ``base_model.model.``); the B
    matrices of q/k adapters get the same head permutation as the base weights."""
    head_dim = head_dim or dim // num_heads
    table = _peft_key_map()
    out = {}
    for k, v in state_dict.items():
        nk = get_mapped_key(k, table)
        if "lora_B" in nk and "q_proj" in nk:
            v = _to_half_split(v, num_heads, head_dim)
        elif "lora_B" in nk and "k_proj" in nk:
            v = _to_half_split(v, num_kv_heads, head_dim)
        out["base_model.model." + nk] = v
    return out

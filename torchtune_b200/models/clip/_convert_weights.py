"""HF CLIP text-model checkpoint → native keys (parity: torchtune/models/clip/_convert_weights.py:9-60)."""
from __future__ import annotations

import re
from typing import Dict

import torch

_LAYER = re.compile(r"^text_model\.encoder\.layers\.(\d+)\.(.+)$")
_SUB = {"layer_norm1": "sa_norm", "layer_norm2": "mlp_norm", "self_attn.q_proj": "attn.q_proj", "self_attn.k_proj": "attn.k_proj", "self_attn.v_proj": "attn.v_proj",
        "self_attn.out_proj": "attn.output_proj", "mlp.fc1": "mlp.w1", "mlp.fc2": "mlp.w2"}
_TOP = {"text_model.embeddings.token_embedding.weight": "token_embedding.weight", "text_model.embeddings.position_embedding.weight": "position_embedding",
        "text_model.final_layer_norm.weight": "final_norm.weight", "text_model.final_layer_norm.bias": "final_norm.bias"}
_IGNORE = ("logit_scale", "text_model.embeddings.position_ids", "text_projection.weight", "visual_projection.weight")


def clip_text_hf_to_tune(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Text tower only; the vision tower, projections and logit scale of the HF checkpoint are skipped."""
    out = {}
    for key, value in state_dict.items():
        if key.startswith("vision_model.") or key in _IGNORE:
            continue
        if key in _TOP:
            out[_TOP[key]] = value
            continue
        m = _LAYER.match(key)
        if m is None:
            raise KeyError(f'Error converting the state dict. Found unexpected key: "{key}".')
        stem, leaf = m.group(2).rsplit(".", 1)
        out[f"layers.{m.group(1)}.{_SUB[stem]}.{leaf}"] = value
    return out


def _register() -> None:
    from ...training.checkpointing._codecs import register_hf_codec
    from ...training.checkpointing._utils import ModelType

    def _no_export(sd, cfg):
        raise NotImplementedError("CLIP text checkpoints are read-only")

    register_hf_codec(ModelType.CLIP_TEXT, lambda sd, cfg: clip_text_hf_to_tune(sd), _no_export)


_register()

"""HF ↔ native weights for Llama 4 (parity: torchtune/models/llama4/_convert_weights.py:63-270).

Specifics: HF fuses the experts' gate and up projections into ``gate_up_proj [E, dim, 2·hidden]``;
the patch embedding is stored as a flat linear ``[embed, 3·p·p]``; q/k projections need no
permutation (both sides use interleaved rotary pairs)."""
from __future__ import annotations

import math
import re
from typing import Dict, List, Optional, Tuple

import torch


def _rules() -> List[Tuple[str, Optional[str]]]:
    lm, dec = "language_model.model.layers.{}.", "decoder.layers.{}."
    r: List[Tuple[str, Optional[str]]] = [
        ("language_model.model.embed_tokens.weight", "decoder.tok_embeddings.weight"),
        ("language_model.model.norm.weight", "decoder.norm.scale"),
        ("language_model.lm_head.weight", "decoder.output.weight"),
        (lm + "self_attn.rotary_emb.inv_freq", None),
        (lm + "input_layernorm.weight", dec + "sa_norm.scale"),
        (lm + "post_attention_layernorm.weight", dec + "mlp_norm.scale"),
        (lm + "feed_forward.experts.down_proj", dec + "mlp.experts.down_proj"),
        (lm + "feed_forward.experts.gate_up_proj", dec + "mlp.experts.gate_proj"),  # split / fused in code
        (lm + "feed_forward.router.weight", dec + "mlp.router.gate.weight"),
    ]
    for hf, nat in (("q_proj", "q_proj"), ("k_proj", "k_proj"), ("v_proj", "v_proj"), ("o_proj", "output_proj")):
        r.append((lm + f"self_attn.{hf}.weight", dec + f"attn.{nat}.weight"))
    for hf, nat in (("gate_proj", "w1"), ("down_proj", "w2"), ("up_proj", "w3")):
        r.append((lm + f"feed_forward.shared_expert.{hf}.weight", dec + f"mlp.shared_expert.{nat}.weight"))
        r.append((lm + f"feed_forward.{hf}.weight", dec + f"mlp.{nat}.weight"))  # dense layers of the 128-expert model
    vm, clip = "vision_model.", "encoders.vision.clip."
    r += [
        (vm + "class_embedding", clip + "cls_token_embedding.weight"),
        (vm + "positional_embedding_vlm", clip + "token_pos_embedding.positional_embedding"),
        (vm + "patch_embedding.linear.weight", clip + "conv.weight"),
        (vm + "vision_adapter.mlp.fc1.weight", "encoders.vision.projection.output.0.weight"),
        (vm + "vision_adapter.mlp.fc2.weight", "encoders.vision.projection.output.2.weight"),
        ("multi_modal_projector.linear_1.weight", "encoders.vision.projection.output.4.weight"),
    ]
    vl, cl = vm + "model.layers.{}.", clip + "layers.{}."
    for wb in ("weight", "bias"):
        r += [(vm + f"layernorm_pre.{wb}", clip + f"ln_pre.{wb}"), (vm + f"layernorm_post.{wb}", clip + f"ln_post.{wb}")]
        for hf, nat in (("q_proj", "q_proj"), ("k_proj", "k_proj"), ("v_proj", "v_proj"), ("o_proj", "output_proj")):
            r.append((vl + f"self_attn.{hf}.{wb}", cl + f"attn.{nat}.{wb}"))
        r += [(vl + f"mlp.fc1.{wb}", cl + f"mlp.w1.{wb}"), (vl + f"mlp.fc2.{wb}", cl + f"mlp.w2.{wb}"), (vl + f"input_layernorm.{wb}", cl + f"sa_norm.{wb}"), (vl + f"post_attention_layernorm.{wb}", cl + f"mlp_norm.{wb}")]
    return r


_HF2NAT = dict(_rules())
_NAT2HF = {v: k for k, v in _HF2NAT.items() if v is not None}
_IDX = re.compile(r"\.layers\.(\d+)\.")


def _map(key: str, table: Dict[str, Optional[str]]) -> Optional[str]:
    m = _IDX.search(key)
    tmpl = key if m is None else key[: m.start()] + ".layers.{}." + key[m.end() :]
    if tmpl not in table:
        raise KeyError(f'Error converting the state dict. Found unexpected key: "{key}".')
    target = table[tmpl]
    return None if target is None else (target if m is None else target.format(m.group(1)))


def llama4_hf_to_tune(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for key, value in state_dict.items():
        new = _map(key, _HF2NAT)
        if new is None:
            continue
        if key.endswith("experts.gate_up_proj"):
            gate, up = torch.chunk(value, 2, dim=-1)
            out[new], out[new.replace("gate_proj", "up_proj")] = gate, up
            continue
        if "patch_embedding" in key:
            d, flat = value.shape
            p = math.isqrt(flat // 3)
            assert 3 * p * p == flat, "conversion assumes 3-channel inputs and square patches"
            value = value.reshape(d, 3, p, p)
        out[new] = value
    return out


def llama4_tune_to_hf(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for key, value in state_dict.items():
        if key.endswith("experts.up_proj"):
            continue  # written together with gate_proj
        new = _map(key, _NAT2HF)
        if key.endswith("experts.gate_proj"):
            value = torch.cat([value, state_dict[key.replace("gate_proj", "up_proj")]], dim=-1)
        elif key.endswith("clip.conv.weight"):
            value = value.reshape(value.shape[0], -1)
        out[new] = value
    return out


def _register() -> None:
    from ...training.checkpointing._codecs import register_hf_codec
    from ...training.checkpointing._utils import ModelType

    register_hf_codec(ModelType.LLAMA4, lambda sd, cfg: llama4_hf_to_tune(sd), lambda sd, cfg: llama4_tune_to_hf(sd))


_register()

"""Original Flux autoencoder checkpoint → native keys (parity: torchtune/models/flux/_convert_weights.py:8-140).

Original layout: ``{encoder,decoder}.{conv_in,norm_out,conv_out}``, ``mid.{block_1,attn_1,block_2}``,
``down.N.block.M`` / ``down.N.downsample`` and ``up.N.block.M`` / ``up.N.upsample`` with the up blocks
numbered in reverse; attention projections are stored as 1×1 convolutions."""
from __future__ import annotations

import re
from typing import Dict

import torch

_RESNET = {"norm1": "main.0", "conv1": "main.2", "norm2": "main.3", "conv2": "main.5", "nin_shortcut": "shortcut"}
_ATTN = {"q": "attn.q_proj", "k": "attn.k_proj", "v": "attn.v_proj", "proj_out": "attn.output_proj", "norm": "norm"}
_MID = {"block_1": ("0", _RESNET), "attn_1": ("1", _ATTN), "block_2": ("2", _RESNET)}


class ConversionError(Exception):
    pass


def _convert_key(key: str, n_up_blocks: int = 4) -> str:
    m = re.match(r"^(encoder|decoder)\.(conv_in|norm_out|conv_out)\.(weight|bias)$", key)
    if m:
        part = {"conv_in": "conv_in", "norm_out": "end.0", "conv_out": "end.2"}[m.group(2)]
        return f"{m.group(1)}.{part}.{m.group(3)}"
    p = key.split(".")
    try:
        model, section = p[0], p[1]
        if model not in ("encoder", "decoder"):
            raise ConversionError(key)
        if section == "mid":
            idx, table = _MID[p[2]]
            return ".".join([model, "mid", idx, table[p[3]], p[4]])
        if section in ("down", "up"):
            block = p[2] if section == "down" else str(n_up_blocks - 1 - int(p[2]))
            if p[3] == "block":
                return ".".join([model, section, block, "layers", p[4], _RESNET[p[5]], p[6]])
            if p[3] in ("downsample", "upsample"):
                return ".".join([model, section, block] + p[3:])
    except (KeyError, IndexError) as exc:
        raise ConversionError(key) from exc
    raise ConversionError(key)


def flux_ae_hf_to_tune(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for key, value in state_dict.items():
        new = _convert_key(key)
        if "proj" in new:  # 1×1 conv weight [out, in, 1, 1] → linear weight [out, in]
            value = value.squeeze()
        out[new] = value
    return out

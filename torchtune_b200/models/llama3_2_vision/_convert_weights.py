"""HF ↔ native weights for Llama 3.2 Vision
(parity: torchtune/models/llama3_2_vision/_convert_weights.py:14-420).

What differs from the text-only conversion:

* HF numbers self- and cross-attention layers in one sequence; natively a cross-attention layer is
  the ``fusion_layer`` of the self-attention layer that follows it, so layer indices are compacted.
* The token embedding holds the 8 extra (image) rows at the end; natively they live in
  ``tok_embeddings.fusion_embedding``.
* HF stores tile / global position tables pre-gathered per supported aspect ratio (row 0 = padding);
  natively they are ``[tiles, tiles, tokens, dim]`` grids indexed by tile row and column.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..convert_weights import _to_half_split, _to_interleaved

_ATTN = (("q_proj", "q_proj"), ("k_proj", "k_proj"), ("v_proj", "v_proj"), ("o_proj", "output_proj"))


def _rules() -> List[Tuple[str, str]]:
    """(HF pattern, native pattern) pairs; ``{}`` stands for a layer index."""
    lm, dec = "language_model.model.layers.{}.", "decoder.layers.{}."
    r = [
        ("language_model.model.embed_tokens.weight", "decoder.tok_embeddings.weight"),
        ("language_model.model.norm.weight", "decoder.norm.scale"),
        ("language_model.lm_head.weight", "decoder.output.weight"),
        (lm + "input_layernorm.weight", dec + "sa_norm.scale"),
        (lm + "post_attention_layernorm.weight", dec + "mlp_norm.scale"),
        (lm + "cross_attn_attn_gate", dec + "fusion_layer.ca_scale.scale"),
        (lm + "cross_attn_mlp_gate", dec + "fusion_layer.mlp_scale.scale"),
        (lm + "cross_attn.q_norm.weight", dec + "fusion_layer.attn.q_norm.scale"),
        (lm + "cross_attn.k_norm.weight", dec + "fusion_layer.attn.k_norm.scale"),
    ]
    for hf, nat in _ATTN:
        r.append((lm + f"self_attn.{hf}.weight", dec + f"attn.{nat}.weight"))
        r.append((lm + f"cross_attn.{hf}.weight", dec + f"fusion_layer.attn.{nat}.weight"))
    for hf, nat in (("gate_proj", "w1"), ("down_proj", "w2"), ("up_proj", "w3")):
        r.append((lm + f"mlp.{hf}.weight", dec + f"mlp.{nat}.weight"))
    vm, clip = "vision_model.", "encoder.clip."
    r += [
        (vm + "gated_positional_embedding.embedding", clip + "token_pos_embedding.local_token_positional_embedding"),
        (vm + "gated_positional_embedding.tile_embedding.weight", clip + "token_pos_embedding.global_token_positional_embedding"),
        (vm + "gated_positional_embedding.gate", clip + "token_pos_embedding.gate"),
        (vm + "pre_tile_positional_embedding.embedding.weight", clip + "pre_tile_pos_embed.embedding"),
        (vm + "pre_tile_positional_embedding.gate", clip + "pre_tile_pos_embed.gate"),
        (vm + "post_tile_positional_embedding.embedding.weight", clip + "post_tile_pos_embed.embedding"),
        (vm + "post_tile_positional_embedding.gate", clip + "post_tile_pos_embed.gate"),
        (vm + "class_embedding", clip + "cls_token_embedding.weight"),
        (vm + "patch_embedding.weight", clip + "conv.weight"),
        ("multi_modal_projector.weight", "encoder.projection.output.weight"),
        ("multi_modal_projector.bias", "encoder.projection.output.bias"),
    ]
    for wb in ("weight", "bias"):
        r.append((vm + f"layernorm_pre.{wb}", clip + f"ln_pre.{wb}"))
        r.append((vm + f"layernorm_post.{wb}", clip + f"ln_post.{wb}"))
    for hf_stack, nat_stack in (("transformer", "encoder.clip"), ("global_transformer", "encoder.projection")):
        h, n = vm + hf_stack + ".layers.{}.", nat_stack + ".layers.{}."
        for hf, nat in _ATTN:
            r.append((h + f"self_attn.{hf}.weight", n + f"attn.{nat}.weight"))
        for wb in ("weight", "bias"):
            r += [(h + f"mlp.fc1.{wb}", n + f"mlp.w1.{wb}"), (h + f"mlp.fc2.{wb}", n + f"mlp.w2.{wb}"), (h + f"input_layernorm.{wb}", n + f"sa_norm.{wb}"), (h + f"post_attention_layernorm.{wb}", n + f"mlp_norm.{wb}")]
    r += [(vm + "global_transformer.layers.{}.gate_attn", "encoder.projection.layers.{}.sa_scale.scale"), (vm + "global_transformer.layers.{}.gate_ffn", "encoder.projection.layers.{}.mlp_scale.scale")]
    return r


_HF2NAT = dict(_rules())
_NAT2HF = {v: k for k, v in _HF2NAT.items()}
_IDX = re.compile(r"\.layers\.(\d+)\.")


def _template(key: str) -> Tuple[str, Optional[int]]:
    m = _IDX.search(key)
    return (key, None) if m is None else (key[: m.start()] + ".layers.{}." + key[m.end() :], int(m.group(1)))


def _grid_from_hf(value: torch.Tensor, num_tiles: int, dim: int, ratios: Sequence[Tuple[int, int]]) -> torch.Tensor:
    n_tok = value.shape[-1] // dim // num_tiles
    grid = torch.zeros(num_tiles, num_tiles, n_tok, dim, dtype=value.dtype, device=value.device)
    for i, (h, w) in enumerate(ratios):
        if h * w == num_tiles:  # smaller canvases are sub-grids of these
            grid[:h, :w] = value[i + 1].reshape(h, w, n_tok, dim)
    return grid


def _grid_to_hf(grid: torch.Tensor, num_tiles: int, ratios: Sequence[Tuple[int, int]]) -> torch.Tensor:
    n_tok, dim = grid.shape[-2:]
    out = torch.zeros(len(ratios) + 1, num_tiles, n_tok, dim, dtype=grid.dtype, device=grid.device)
    for i, (h, w) in enumerate(ratios):
        out[i + 1, : h * w] = grid[:h, :w].reshape(h * w, n_tok, dim)
    return out.reshape(len(ratios) + 1, -1)


def llama3_vision_hf_to_tune(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: Optional[int] = None, vocab_size: int = 128256,
                             cross_attention_layers: Optional[List[int]] = None, encoder_dim: int = 1280, tile_size: int = 448, num_tiles: int = 4,
                             supported_aspect_ratios: Optional[List[Tuple[int, int]]] = None) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    cross = sorted(cross_attention_layers or [])
    ratios = supported_aspect_ratios or []
    out: Dict[str, torch.Tensor] = {}
    for key, value in state_dict.items():
        if "rotary_emb.inv_freq" in key:
            continue
        tmpl, idx = _template(key)
        if tmpl not in _HF2NAT:
            raise KeyError(f'Error converting the state dict. Found unexpected key: "{key}".')
        new = _HF2NAT[tmpl]
        if key.startswith("language_model") and idx is not None:
            native_idx = idx - sum(idx > c for c in cross)
            if idx in cross and "fusion_layer" not in new:
                # norms / MLP of a cross-attention block share HF names with self-attention blocks
                new = new.replace("layers.{}.", "layers.{}.fusion_layer.").replace("sa_norm", "ca_norm")
            new = new.format(native_idx)
            if "cross_attn" not in key:
                if ".self_attn.q_proj." in key:
                    value = _to_interleaved(value, num_heads, head_dim)
                elif ".self_attn.k_proj." in key:
                    value = _to_interleaved(value, num_kv_heads, head_dim)
        elif idx is not None:
            new = new.format(idx)
        if new == "decoder.tok_embeddings.weight":
            out["decoder.tok_embeddings.fusion_embedding.weight"] = value[vocab_size:]
            value = value[:vocab_size]
        elif new.endswith("tile_pos_embed.embedding") or new.endswith("global_token_positional_embedding"):
            value = _grid_from_hf(value, num_tiles, encoder_dim, ratios)
        out[new] = value
    return out


def llama3_vision_tune_to_hf(state_dict: Dict[str, torch.Tensor], num_heads: int = 32, num_kv_heads: int = 32, dim: int = 4096, head_dim: Optional[int] = None, vocab_size: int = 128256,
                             cross_attention_layers: Optional[List[int]] = None, encoder_dim: int = 1280, tile_size: int = 448, num_tiles: int = 4,
                             supported_aspect_ratios: Optional[List[Tuple[int, int]]] = None) -> Dict[str, torch.Tensor]:
    head_dim = head_dim or dim // num_heads
    cross = sorted(cross_attention_layers or [])
    ratios = supported_aspect_ratios or []
    # native layer i that owns a fusion layer ↔ HF cross layer c and self layer c + 1
    n_hf_layers = 1 + max([int(m.group(1)) for k in state_dict if k.startswith("decoder.") for m in [_IDX.search(k)] if m] + [-1]) + len(cross)
    self_hf = [i for i in range(n_hf_layers) if i not in cross]
    out: Dict[str, torch.Tensor] = {}
    fusion_rows = state_dict.get("decoder.tok_embeddings.fusion_embedding.weight")
    for key, value in state_dict.items():
        if key == "decoder.tok_embeddings.fusion_embedding.weight":
            continue
        tmpl, idx = _template(key)
        lookup = tmpl
        in_fusion = ".fusion_layer." in key and key.startswith("decoder.")
        if in_fusion and tmpl not in _NAT2HF:
            lookup = tmpl.replace(".fusion_layer.", ".").replace("ca_norm", "sa_norm")
        if lookup not in _NAT2HF:
            raise KeyError(f'Error converting the state dict. Found unexpected key: "{key}".')
        new = _NAT2HF[lookup]
        if key.startswith("decoder.") and idx is not None:
            hf_self = self_hf[idx]
            new = new.format(hf_self - 1 if in_fusion else hf_self)
            if not in_fusion:
                if key.endswith("attn.q_proj.weight"):
                    value = _to_half_split(value, num_heads, head_dim)
                elif key.endswith("attn.k_proj.weight"):
                    value = _to_half_split(value, num_kv_heads, head_dim)
        elif idx is not None:
            new = new.format(idx)
        if key == "decoder.tok_embeddings.weight" and fusion_rows is not None:
            value = torch.cat([value, fusion_rows.to(value.dtype)], dim=0)
        elif key.endswith("tile_pos_embed.embedding") or key.endswith("global_token_positional_embedding"):
            value = _grid_to_hf(value, num_tiles, ratios)
        out[new] = value
    return out


def _vision_args(cfg):
    text, vis = cfg["text_config"], cfg["vision_config"]
    return dict(
        num_heads=text["num_attention_heads"], num_kv_heads=text["num_key_value_heads"], dim=text["hidden_size"], head_dim=text.get("head_dim"), vocab_size=text["vocab_size"],
        cross_attention_layers=text.get("cross_attention_layers"), encoder_dim=vis["hidden_size"], tile_size=vis["image_size"], num_tiles=vis["max_num_tiles"],
        supported_aspect_ratios=[tuple(r) for r in vis.get("supported_aspect_ratios", [])],
    )


def _register() -> None:
    from ...training.checkpointing._codecs import register_hf_codec
    from ...training.checkpointing._utils import ModelType

    register_hf_codec(ModelType.LLAMA3_VISION, lambda sd, cfg: llama3_vision_hf_to_tune(sd, **_vision_args(cfg)), lambda sd, cfg: llama3_vision_tune_to_hf(sd, **_vision_args(cfg)))


_register()

"""Llama-4 Scout (17B active, 16 experts) and Maverick (17B active, 128 experts)
(parity: torchtune/models/llama4/_model_builders.py:30-400)."""
from __future__ import annotations

from typing import List, Optional

from ...modules.model_fusion import EarlyFusionModel
from ._component_builders import llama4_decoder, llama4_vision_encoder, lora_llama4_decoder
from ._tokenizer import LLAMA4_SPECIAL_TOKENS
from ._transform import Llama4Transform

_VISION = dict(patch_size=14, num_heads=16, clip_embed_dim=1408, clip_num_layers=34, decoder_embed_dim=5120, projection_embed_dim=4096, max_num_tiles=16, in_channels=3)
_COMMON = dict(vocab_size=202_048, num_layers=48, num_heads=40, num_kv_heads=8, embed_dim=5120, hidden_dim=8192, attn_dropout=0.0, rope_base=500_000, norm_eps=1e-5, use_shared_expert=True, skip_rope_interval=4, attention_chunk_size=8192)
_SCOUT = dict(_COMMON, max_seq_len=10485760, num_experts=16, use_scaled_rope=True)
_MAVERICK = dict(_COMMON, max_seq_len=1048576, num_experts=128, use_qk_norm=False, moe_every_n_layers=2, mlp_hidden_dim=16384)


def _fuse(decoder, image_size: int, decoder_trainable: bool, encoder_trainable: bool, fusion_trainable: bool) -> EarlyFusionModel:
    vision = llama4_vision_encoder(**_VISION, tile_size=image_size)
    return EarlyFusionModel(decoder, encoders={"vision": vision}, encoder_tokens={"vision": LLAMA4_SPECIAL_TOKENS["<|patch|>"]}, encoders_trainable={"vision": encoder_trainable},
                            decoder_trainable=decoder_trainable, fusion_trainable=fusion_trainable)


def llama4_scout_17b_16e(decoder_trainable: bool = True, encoder_trainable: bool = False, fusion_trainable: bool = True, image_size: int = 336) -> EarlyFusionModel:
    return _fuse(llama4_decoder(**_SCOUT), image_size, decoder_trainable, encoder_trainable, fusion_trainable)


def llama4_maverick_17b_128e(decoder_trainable: bool = True, encoder_trainable: bool = False, fusion_trainable: bool = True, image_size: int = 336) -> EarlyFusionModel:
    return _fuse(llama4_decoder(**_MAVERICK), image_size, decoder_trainable, encoder_trainable, fusion_trainable)


def _lora(preset: dict, lora_attn_modules: List[str], decoder_trainable: str, encoder_trainable: str, fusion_trainable: str, apply_lora_to_mlp: bool, apply_lora_to_output: bool, lora_rank: int,
          lora_alpha: float, lora_dropout: float, use_dora: bool, quantize_base: bool, image_size: int) -> EarlyFusionModel:
    for flag in (decoder_trainable, encoder_trainable, fusion_trainable):
        if flag.lower() not in ("lora", "frozen"):
            raise ValueError("mixed LoRA + full fine-tuning is not supported: trainable flags must be 'lora' or 'frozen'")
    if decoder_trainable.lower() == "lora":
        decoder = lora_llama4_decoder(lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, lora_rank=lora_rank, lora_alpha=lora_alpha, lora_dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base, **preset)
    else:
        decoder = llama4_decoder(**preset)
    # the vision tower stays un-adapted (frozen or trained through the fusion projector only)
    return _fuse(decoder, image_size, decoder_trainable.lower() != "frozen", False, fusion_trainable.lower() != "frozen")


def lora_llama4_scout_17b_16e(lora_attn_modules: List[str], decoder_trainable: str = "lora", encoder_trainable: str = "frozen", fusion_trainable: str = "lora", apply_lora_to_mlp: bool = False,
                              apply_lora_to_output: bool = False, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, image_size: int = 336) -> EarlyFusionModel:
    return _lora(_SCOUT, lora_attn_modules, decoder_trainable, encoder_trainable, fusion_trainable, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base, image_size)


def lora_llama4_maverick_17b_128e(lora_attn_modules: List[str], decoder_trainable: str = "lora", encoder_trainable: str = "frozen", fusion_trainable: str = "lora", apply_lora_to_mlp: bool = False,
                                  apply_lora_to_output: bool = False, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, image_size: int = 336) -> EarlyFusionModel:
    return _lora(_MAVERICK, lora_attn_modules, decoder_trainable, encoder_trainable, fusion_trainable, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base, image_size)


def llama4_transform(path: str, max_seq_len: int = 8192, image_size: int = 336, max_num_tiles: int = 16, special_tokens_path: Optional[str] = None, prompt_template=None) -> Llama4Transform:
    return Llama4Transform(path=path, special_tokens_path=special_tokens_path, tile_size=image_size, patch_size=14, max_num_tiles=max_num_tiles, max_seq_len=max_seq_len,
                           image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5], prompt_template=prompt_template)

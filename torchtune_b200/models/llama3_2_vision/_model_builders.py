"""Llama 3.2 Vision 11B / 90B (parity: torchtune/models/llama3_2_vision/_model_builders.py:24-390)."""
from __future__ import annotations

from typing import List, Optional

from ...modules.model_fusion import DeepFusionModel
from ._component_builders import LoRATrainable, llama3_2_vision_decoder, llama3_2_vision_encoder, lora_llama3_2_vision_decoder, lora_llama3_2_vision_encoder
from ._transform import Llama3VisionTransform

_ENC = dict(patch_size=14, num_heads=16, clip_embed_dim=1280, clip_num_layers=32, clip_hidden_states=[3, 7, 15, 23, 30], num_layers_projection=8, max_num_tiles=4, in_channels=3)
_DEC = {
    "11b": dict(vocab_size=128_256, num_layers=32, fusion_interval=4, num_special_tokens=8, num_heads=32, num_kv_heads=8, embed_dim=4096, max_seq_len=131_072, encoder_max_seq_len=128_080, rope_base=500_000, intermediate_dim=14336),
    "90b": dict(vocab_size=128_256, num_layers=80, fusion_interval=4, num_special_tokens=8, num_heads=64, num_kv_heads=8, embed_dim=8192, max_seq_len=131_072, encoder_max_seq_len=128_080, rope_base=500_000, intermediate_dim=28672),
}


def llama3_2_vision_transform(path: str, max_seq_len: int = 8192, image_size: int = 560, special_tokens_path: Optional[str] = None, prompt_template=None) -> Llama3VisionTransform:
    """Transform with the image statistics the released checkpoints were trained with."""
    return Llama3VisionTransform(path=path, special_tokens_path=special_tokens_path, tile_size=image_size, patch_size=14, max_num_tiles=4, max_seq_len=max_seq_len,
                                 image_mean=(0.48145466, 0.4578275, 0.40821073), image_std=(0.26862954, 0.26130258, 0.27577711), prompt_template=prompt_template)


def _full(size: str, decoder_trainable: bool, encoder_trainable: bool, fusion_trainable: bool, image_size: int) -> DeepFusionModel:
    dec = _DEC[size]
    encoder = llama3_2_vision_encoder(**_ENC, decoder_embed_dim=dec["embed_dim"], tile_size=image_size)
    decoder = llama3_2_vision_decoder(**dec)
    return DeepFusionModel(encoder=encoder, decoder=decoder, encoder_trainable=encoder_trainable, decoder_trainable=decoder_trainable, fusion_trainable=fusion_trainable)


def _lora(size: str, lora_attn_modules: List[str], decoder_trainable: str, encoder_trainable: str, fusion_trainable: str, apply_lora_to_mlp: bool, apply_lora_to_output: bool, lora_rank: int,
          lora_alpha: float, lora_dropout: float, use_dora: bool, quantize_base: bool, image_size: int) -> DeepFusionModel:
    d, e, f = (LoRATrainable(x.lower()) for x in (decoder_trainable, encoder_trainable, fusion_trainable))
    assert LoRATrainable.FULL not in (d, e, f), "mixed LoRA + full fine-tuning is not supported: use the non-LoRA builder for full fine-tuning"
    dec = _DEC[size]
    lora_kw = dict(lora_rank=lora_rank, lora_alpha=lora_alpha, lora_dropout=lora_dropout, use_dora=use_dora, quantize_base=quantize_base)
    encoder = lora_llama3_2_vision_encoder(e == LoRATrainable.LORA, f == LoRATrainable.LORA, lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, **_ENC, decoder_embed_dim=dec["embed_dim"], tile_size=image_size, **lora_kw)
    decoder = lora_llama3_2_vision_decoder(d == LoRATrainable.LORA, f == LoRATrainable.LORA, lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output, **dec, **lora_kw)
    return DeepFusionModel(encoder=encoder, decoder=decoder, encoder_trainable=e != LoRATrainable.FROZEN, decoder_trainable=d != LoRATrainable.FROZEN, fusion_trainable=f != LoRATrainable.FROZEN)


def llama3_2_vision_11b(decoder_trainable: bool = False, encoder_trainable: bool = True, fusion_trainable: bool = True, image_size: int = 560) -> DeepFusionModel:
    return _full("11b", decoder_trainable, encoder_trainable, fusion_trainable, image_size)


def llama3_2_vision_90b(decoder_trainable: bool = False, encoder_trainable: bool = True, fusion_trainable: bool = True, image_size: int = 560) -> DeepFusionModel:
    return _full("90b", decoder_trainable, encoder_trainable, fusion_trainable, image_size)


def lora_llama3_2_vision_11b(lora_attn_modules: List[str], decoder_trainable: str = "frozen", encoder_trainable: str = "lora", fusion_trainable: str = "lora", apply_lora_to_mlp: bool = False,
                             apply_lora_to_output: bool = False, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, image_size: int = 560) -> DeepFusionModel:
    return _lora("11b", lora_attn_modules, decoder_trainable, encoder_trainable, fusion_trainable, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base, image_size)


def lora_llama3_2_vision_90b(lora_attn_modules: List[str], decoder_trainable: str = "frozen", encoder_trainable: str = "lora", fusion_trainable: str = "lora", apply_lora_to_mlp: bool = False,
                             apply_lora_to_output: bool = False, lora_rank: int = 8, lora_alpha: float = 16, lora_dropout: float = 0.0, use_dora: bool = False, quantize_base: bool = False, image_size: int = 560) -> DeepFusionModel:
    return _lora("90b", lora_attn_modules, decoder_trainable, encoder_trainable, fusion_trainable, apply_lora_to_mlp, apply_lora_to_output, lora_rank, lora_alpha, lora_dropout, use_dora, quantize_base, image_size)


def qlora_llama3_2_vision_11b(*args, **kwargs) -> DeepFusionModel:
    return lora_llama3_2_vision_11b(*args, **{**kwargs, "quantize_base": True})


def qlora_llama3_2_vision_90b(*args, **kwargs) -> DeepFusionModel:
    return lora_llama3_2_vision_90b(*args, **{**kwargs, "quantize_base": True})

"""CLIP towers, tokenizer and image transform (parity: torchtune/models/clip/__init__.py)."""
from ._component_builders import clip_mlp, clip_text_encoder, clip_vision_encoder, lora_clip_vision_encoder
from ._model_builders import clip_text_vit_large_patch14, clip_tokenizer, clip_vit_224_transform
from ._position_embeddings import TiledTokenPositionalEmbedding, TilePositionalEmbedding, TokenPositionalEmbedding
from ._text_encoder import CLIPTextEncoder, QuickGELU
from ._tokenizer import CLIPTokenizer
from ._transform import CLIPImageTransform

__all__ = [
    "clip_mlp",
    "clip_text_encoder",
    "clip_vision_encoder",
    "lora_clip_vision_encoder",
    "clip_text_vit_large_patch14",
    "clip_tokenizer",
    "CLIPImageTransform",
    "CLIPTextEncoder",
    "CLIPTokenizer",
    "QuickGELU",
    "TokenPositionalEmbedding",
    "TiledTokenPositionalEmbedding",
    "TilePositionalEmbedding",
]

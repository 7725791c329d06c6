"""CLIP presets (parity: torchtune/models/clip/_model_builders.py:9-60)."""
from ._component_builders import clip_text_encoder
from ._text_encoder import CLIPTextEncoder
from ._tokenizer import CLIPTokenizer


def clip_tokenizer(vocab_path: str = "/tmp/clip-vit-large-patch14/merges.txt", max_seq_len: int = 77, truncate: bool = True) -> CLIPTokenizer:
    """Tokenizer of CLIP ViT-L/14 from its ``merges.txt``."""
    return CLIPTokenizer(vocab_path, max_seq_len=max_seq_len, truncate=truncate)


def clip_text_vit_large_patch14() -> CLIPTextEncoder:
    """Text tower of CLIP ViT-L/14: 12 layers, width 768, 12 heads, 49408 tokens, 77 positions."""
    return clip_text_encoder(embed_dim=768, num_heads=12, num_layers=12, vocab_size=49408, max_seq_len=77, norm_eps=1e-5)


def clip_vit_224_transform():
    """Image transform of the 224-pixel CLIP ViT checkpoints: one tile, resize to the canvas, CLIP mean / std."""
    from ._transform import CLIPImageTransform

    return CLIPImageTransform(image_mean=[0.48145466, 0.4578275, 0.40821073], image_std=[0.26862954, 0.26130258, 0.27577711], tile_size=224, possible_resolutions=None,
                              max_num_tiles=1, resample="bilinear", resize_to_max_canvas=True)

"""Tokenizer + image transform of Llama 3.2 Vision
(parity: torchtune/models/llama3_2_vision/_transform.py:18-230)."""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Tuple

from ...data import Message
from ...modules.transforms import Transform, VisionCrossAttentionMask
from ...modules.transforms.tokenizers import ModelTokenizer
from ..clip import CLIPImageTransform
from ..llama3 import llama3_tokenizer


class Llama3VisionTransform(ModelTokenizer, Transform):
    """For every image in the messages: best-fit canvas, resize, normalise, tile.  Then tokenise the
    conversation (images become the image placeholder token) and build, per image, the mask that lets
    the text tokens following it attend to its tiles.  Adds ``encoder_input`` (``images``,
    ``aspect_ratio``), ``tokens``, ``mask`` and ``encoder_mask`` to the sample."""

    def __init__(self, path: str, *, tile_size: int, patch_size: int, max_num_tiles: int = 4, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None,
                 image_mean: Optional[List[float]] = None, image_std: Optional[List[float]] = None, prompt_template: Any = None):
        self.tokenizer = llama3_tokenizer(path, special_tokens_path=special_tokens_path, max_seq_len=max_seq_len, prompt_template=prompt_template)
        self.transform_image = CLIPImageTransform(image_mean=image_mean, image_std=image_std, tile_size=tile_size, possible_resolutions=None, max_num_tiles=max_num_tiles, resample="bilinear", resize_to_max_canvas=False)
        self.xattn_mask = VisionCrossAttentionMask(tile_size=tile_size, patch_size=patch_size, image_token_id=self.tokenizer.image_id)
        self.stop_tokens = self.tokenizer.stop_tokens
        self.special_tokens = self.tokenizer.special_tokens
        self.max_seq_len, self.max_num_tiles = max_seq_len, max_num_tiles
        self.image_seq_len = max_num_tiles * (self.xattn_mask.patches_per_tile + 1)
        self.prompt_template = prompt_template
        self.pad_id = self.tokenizer.pad_id

    @property
    def base_vocab_size(self) -> int:
        return self.tokenizer.base_vocab_size

    @property
    def vocab_size(self) -> int:
        return self.tokenizer.vocab_size

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        return self.tokenizer.encode(text=text, add_bos=add_bos, add_eos=add_eos)

    def decode(self, token_ids: List[int], truncate_at_eos: bool = True, skip_special_tokens: bool = True) -> str:
        return self.tokenizer.decode(token_ids, truncate_at_eos=truncate_at_eos, skip_special_tokens=skip_special_tokens)

    def tokenize_message(self, message: Message, add_start_tokens: bool = True, add_end_tokens: bool = True) -> List[int]:
        return self.tokenizer.tokenize_message(message=message, add_start_tokens=add_start_tokens, add_end_tokens=add_end_tokens)

    def tokenize_messages(self, messages: List[Message], *, add_end_tokens: bool = True) -> Tuple[List[int], List[bool]]:
        return self.tokenizer.tokenize_messages(messages=messages, add_end_tokens=add_end_tokens)

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        sample = dict(sample)
        images, ratios = [], []
        for message in sample["messages"]:
            for image in message.get_media():
                out = self.transform_image({"image": image}, inference=inference)
                images.append(out["image"])
                ratios.append(out["aspect_ratio"])
        sample["encoder_input"] = {"images": images, "aspect_ratio": ratios}
        sample = self.tokenizer(sample, inference=inference)
        return self.xattn_mask(sample, inference=inference)

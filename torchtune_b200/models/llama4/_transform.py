"""Tokenizer + image transform of Llama 4 (parity: torchtune/models/llama4/_transform.py:24-240)."""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Tuple

import torch

from ...data import Message
from ...modules.transforms.vision_utils import resize
from ..clip import CLIPImageTransform
from ..clip._transform import to_float_image
from ._tokenizer import Llama4Tokenizer


class Llama4Transform:
    """Images are cut into at most ``max_num_tiles`` tiles plus — when there is more than one tile — a
    down-scaled global view; text gets one ``<|patch|>`` placeholder per projected vision token."""

    def __init__(self, path: str, *, tile_size: int, patch_size: int, max_num_tiles: int = 4, pixel_shuffle_scaling_factor: float = 0.5, special_tokens_path: Optional[str] = None,
                 max_seq_len: Optional[int] = None, image_mean: Optional[List[float]] = None, image_std: Optional[List[float]] = None, dtype: torch.dtype = torch.bfloat16, prompt_template: Any = None):
        special_tokens = None
        if special_tokens_path is not None:
            from ...modules.transforms.tokenizers import parse_hf_tokenizer_json

            special_tokens = parse_hf_tokenizer_json(special_tokens_path)
        if prompt_template is not None and not callable(prompt_template):
            from ...data._prompt_templates import _get_prompt_template

            prompt_template = _get_prompt_template(prompt_template)
        self.tokenizer = Llama4Tokenizer(path=path, special_tokens=special_tokens, max_seq_len=max_seq_len, prompt_template=prompt_template)
        self.clip_transform = CLIPImageTransform(image_mean=image_mean, image_std=image_std, tile_size=tile_size, possible_resolutions=None, max_num_tiles=max_num_tiles, resample="bilinear", resize_to_max_canvas=False, dtype=dtype)
        self.tile_size, self.dtype, self.mean, self.std = tile_size, dtype, image_mean, image_std
        self.stop_tokens, self.special_tokens = self.tokenizer.stop_tokens, self.tokenizer.special_tokens
        self.max_seq_len, self.max_num_tiles = max_seq_len, max_num_tiles
        self.patches_per_tile = (tile_size // patch_size) ** 2
        self.image_seq_len = max_num_tiles * self.patches_per_tile
        self.pixel_shuffle_scaling_factor = pixel_shuffle_scaling_factor
        self.patch_tokens_per_tile = int(self.patches_per_tile * pixel_shuffle_scaling_factor**2)
        self.prompt_template, self.pad_id = prompt_template, self.tokenizer.pad_id

    @property
    def base_vocab_size(self) -> int:
        return self.tokenizer.base_vocab_size

    @property
    def vocab_size(self) -> int:
        return self.tokenizer.vocab_size

    def _thumbnail(self, image: Any) -> torch.Tensor:
        x = resize(to_float_image(image, torch.float32), (self.tile_size, self.tile_size), "bilinear")
        if self.mean:
            x = (x - torch.tensor(self.mean).view(-1, 1, 1)) / torch.tensor(self.std).view(-1, 1, 1)
        return x.to(self.dtype)

    def transform_image(self, image: Any, inference: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        out = self.clip_transform({"image": image}, inference=inference)
        tiles, ar = out["image"], out["aspect_ratio"]
        if tiles.shape[0] > 1:
            tiles = torch.cat([tiles, self._thumbnail(image).unsqueeze(0)], dim=0)
        return tiles, ar

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
        images = []
        for message in sample["messages"]:
            for content in message.content:
                if content["type"] == "image":
                    tiles, ar = self.transform_image(content["content"], inference=inference)
                    images.append(tiles)
                    content["patch_tokens_per_tile"] = self.patch_tokens_per_tile
                    content["aspect_ratio"] = ar
        sample["encoder_input"] = {"vision": {"images": images}}
        return self.tokenizer(sample, inference=inference)

"""Llama-4 tokenizer (parity: torchtune/models/llama4/_tokenizer.py:24-470): o200k-style tiktoken BPE
with the Llama-4 header / vision / reasoning special tokens.  Images expand to a tile grid of patch
placeholders: ``<|image_start|>`` [rows of ``<|patch|>``·n separated by x / y tile separators] then
the global view ``<|image|>`` ``<|patch|>``·n ``<|image_end|>``."""
from __future__ import annotations

import re
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ...data._messages import Message
from ...data._utils import truncate
from ...modules.transforms.tokenizers import TikTokenBaseTokenizer

O200K_PATTERN = r"""[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+"""  # noqa: E501


def get_reserved_special_tokens(start_id: int, end_id: int, name: Optional[str] = None, start_reserved: int = 0) -> Dict[str, int]:
    stem = f"{name}_reserved_special_token" if name else "reserved_special_token"
    return {f"<|{stem}_{start_reserved + i}|>": tid for i, tid in enumerate(range(start_id, end_id))}


def _consecutive(first_id: int, names: List[str]) -> Dict[str, int]:
    return {n: first_id + i for i, n in enumerate(names)}


BASIC_SPECIAL_TOKENS = _consecutive(200000, ["<|begin_of_text|>", "<|end_of_text|>", "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>"])
TEXT_SPECIAL_TOKENS = {
    **_consecutive(200005, ["<|header_start|>", "<|header_end|>", "<|eom|>", "<|eot|>", "<|step|>"]),
    **get_reserved_special_tokens(200010, 200018, "text_post_train", 0),
    "<|finetune_right_pad|>": 200018,
    **get_reserved_special_tokens(200019, 200080, "text_post_train", 8),
}
VISION_SPECIAL_TOKENS = {
    **_consecutive(200080, ["<|image_start|>", "<|image_end|>", "<|vision_reserved_special_token_0|>", "<|vision_reserved_special_token_1|>", "<|tile_x_separator|>", "<|tile_y_separator|>"]),
    **get_reserved_special_tokens(200086, 200090, "vision", 2),
    "<|image|>": 200090,
    "<|vision_reserved_special_token_6|>": 200091,
    "<|patch|>": 200092,
    **get_reserved_special_tokens(200093, 201134, "vision", 7),
}
REASONING_SPECIAL_TOKENS = {**get_reserved_special_tokens(201134, 201142, "reasoning", 0), "<|reasoning_thinking_start|>": 201142, "<|reasoning_thinking_end|>": 201143}
SPECIAL_TOKENS = {**BASIC_SPECIAL_TOKENS, **TEXT_SPECIAL_TOKENS, **VISION_SPECIAL_TOKENS, **REASONING_SPECIAL_TOKENS}
NUM_RESERVED_SPECIAL_TOKENS = 2048
RESERVED_TOKENS = get_reserved_special_tokens(201144, 202048)
LLAMA4_SPECIAL_TOKENS = {**SPECIAL_TOKENS, **RESERVED_TOKENS}


class Llama4Tokenizer:
    def __init__(self, path: str, special_tokens: Optional[Dict[str, int]] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
        self.special_tokens = special_tokens if special_tokens is not None else LLAMA4_SPECIAL_TOKENS
        for tok in SPECIAL_TOKENS:
            if "_reserved_special_token_" not in tok and tok not in self.special_tokens:
                raise ValueError(f"{tok} missing from special_tokens")
        st = self.special_tokens
        self.bos_id, self.eos_id, self.pad_id, self.step_id = st["<|begin_of_text|>"], st["<|end_of_text|>"], st["<|finetune_right_pad|>"], st["<|step|>"]
        self.start_header_id, self.end_header_id, self.eom_id, self.eot_id = st["<|header_start|>"], st["<|header_end|>"], st["<|eom|>"], st["<|eot|>"]
        self.image_id, self.patch_id, self.image_start, self.image_end = st["<|image|>"], st["<|patch|>"], st["<|image_start|>"], st["<|image_end|>"]
        self.tile_x_separator, self.tile_y_separator = st["<|tile_x_separator|>"], st["<|tile_y_separator|>"]
        self.reasoning_start, self.reasoning_end = st["<|reasoning_thinking_start|>"], st["<|reasoning_thinking_end|>"]
        self.stop_tokens = [self.eos_id, self.eot_id, self.eom_id]
        self.tt_model = TikTokenBaseTokenizer(path=path, name="llama4_tiktoken", pattern=O200K_PATTERN, bos_id=self.bos_id, eos_id=self.eos_id, special_tokens=self.special_tokens)
        self.max_seq_len, self.prompt_template, self.truncation_type = max_seq_len, prompt_template, truncation_type
        self._special_re = re.compile(r"<\|.*?\|>")
        self._header_re = re.compile(r"<\|header_start\|>.*?<\|header_end\|>\n\n")

    @property
    def base_vocab_size(self) -> int:
        return self.tt_model.base_vocab_size

    @property
    def vocab_size(self) -> int:
        return self.tt_model.vocab_size

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        return self.tt_model.encode(text=text, add_bos=add_bos, add_eos=add_eos)

    def decode(self, token_ids: List[int], truncate_at_eos: bool = True, skip_special_tokens: bool = True) -> str:
        text = self.tt_model.decode(token_ids, truncate_at_eos=truncate_at_eos)
        return self._special_re.sub("", self._header_re.sub("", text)) if skip_special_tokens else text

    def _image_tokens(self, patches_per_tile: int, aspect_ratio: torch.Tensor) -> List[int]:
        rows, cols = (int(v) for v in aspect_ratio.tolist())
        global_view = [self.image_id] + [self.patch_id] * patches_per_tile + [self.image_end]
        out = [self.image_start]
        if (rows, cols) != (1, 1):
            for _ in range(rows):
                for c in range(cols):
                    out += [self.patch_id] * patches_per_tile
                    if c < cols - 1:
                        out.append(self.tile_x_separator)
                out.append(self.tile_y_separator)
        return out + global_view

    def _body(self, message: Message) -> List[int]:
        out: List[int] = []
        for part in message.content:
            if part["type"] == "text":
                out += self.encode(part["content"].strip(), add_bos=False, add_eos=False)
            elif part["type"] == "image":
                out += self._image_tokens(part.get("patch_tokens_per_tile", 1), part.get("aspect_ratio", torch.tensor([1, 1])))
        return out

    def tokenize_message(self, message: Message, *, add_start_tokens: bool = True, add_end_tokens: bool = True) -> List[int]:
        head = ([self.start_header_id] + self.encode(message.role.strip(), add_bos=False, add_eos=False) + [self.end_header_id] + self.encode("\n\n", add_bos=False, add_eos=False)) if add_start_tokens else []
        tail = ([self.eot_id] if message.eot else [self.eom_id]) if add_end_tokens else []
        return head + self._body(message) + tail

    def tokenize_messages(self, messages: List[Message], *, add_end_tokens: bool = True) -> Tuple[List[int], List[bool]]:
        if self.prompt_template is not None:
            messages = self.prompt_template(messages)
        tokens, mask = [self.bos_id], [True]
        for i, m in enumerate(messages):
            ids = self.tokenize_message(m, add_end_tokens=add_end_tokens if i == len(messages) - 1 else True)
            tokens += ids
            mask += [m.masked] * len(ids)
            if self.max_seq_len and len(tokens) >= self.max_seq_len:
                break
        if add_end_tokens:
            tokens.append(self.eos_id)
            mask.append(True)
        if self.max_seq_len:
            tokens = truncate(tokens, self.max_seq_len, self.eos_id if add_end_tokens else None, self.truncation_type)
            mask = truncate(mask, self.max_seq_len, True if add_end_tokens else None, self.truncation_type)
        return tokens, mask

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        sample = dict(sample)
        tokens, mask = self.tokenize_messages(sample.pop("messages"), add_end_tokens=not inference)
        sample["tokens"], sample["mask"] = tokens, mask
        return sample

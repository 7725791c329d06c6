"""Qwen2.5 tokenizer: Qwen2 BPE plus tool-call / tool-response markup
(parity: torchtune/models/qwen2_5/_tokenizer.py:20-260)."""
from __future__ import annotations

from typing import List

from ...data._messages import Message
from ..qwen2._tokenizer import QWEN2_SPECIAL_TOKENS, Qwen2Tokenizer

_NAMES = ["<|object_ref_start|>", "<|object_ref_end|>", "<|box_start|>", "<|box_end|>", "<|quad_start|>", "<|quad_end|>", "<|vision_start|>", "<|vision_end|>", "<|vision_pad|>", "<|image_pad|>", "<|video_pad|>", "<tool_call>", "</tool_call>", "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>", "<|fim_pad|>", "<|repo_name|>", "<|file_sep|>"]
QWEN2_5_SPECIAL_TOKENS = {**QWEN2_SPECIAL_TOKENS, **{name: 151646 + i for i, name in enumerate(_NAMES)}}


class Qwen2_5Tokenizer(Qwen2Tokenizer):
    """Tool calls by the assistant are wrapped in ``<tool_call>…</tool_call>``; consecutive tool
    returns are grouped into one ``user`` turn, each inside ``<tool_response>…</tool_response>``."""

    def __init__(self, path: str, merges_file: str, special_tokens=QWEN2_5_SPECIAL_TOKENS, max_seq_len=None, **kwargs):
        super().__init__(path, merges_file, special_tokens=special_tokens, max_seq_len=max_seq_len, **kwargs)
        self.tool_call_start_id = self.special_tokens["<tool_call>"]
        self.tool_call_end_id = self.special_tokens["</tool_call>"]

    def _plain(self, text: str) -> List[int]:
        return self.encode(text, add_bos=False, add_eos=False)

    def _header(self, messages: List[Message], i: int) -> List[int]:
        m = messages[i]
        if m.role == "ipython":
            first = i == 0 or messages[i - 1].role != "ipython"
            return (self._open("user") + self._plain("<tool_response>\n")) if first else self._plain("\n<tool_response>\n")
        ids = self._open(m.role)
        if m.role == "assistant" and m.ipython:
            ids += [self.tool_call_start_id] + self._plain("\n")
        return ids

    def _footer(self, messages: List[Message], i: int) -> List[int]:
        m = messages[i]
        if m.role == "ipython":
            last = i == len(messages) - 1 or messages[i + 1].role != "ipython"
            return self._plain("\n</tool_response>") + (self._close() if last else [])
        ids: List[int] = []
        if m.role == "assistant" and m.ipython:
            ids += self._plain("\n") + [self.tool_call_end_id]
        if m.role != "assistant" or i != len(messages) - 1:
            ids += self._close()
        return ids

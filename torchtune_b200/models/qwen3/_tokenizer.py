"""Qwen3 tokenizer: the Qwen2.5 layout with the ``<tool_response>`` / ``<think>`` specials
(parity: torchtune/models/qwen3/_tokenizer.py)."""
from ..qwen2_5._tokenizer import QWEN2_5_SPECIAL_TOKENS, Qwen2_5Tokenizer

QWEN3_SPECIAL_TOKENS = {**QWEN2_5_SPECIAL_TOKENS, "<tool_response>": 151665, "</tool_response>": 151666, "<think>": 151667, "</think>": 151668}


class Qwen3Tokenizer(Qwen2_5Tokenizer):
    def __init__(self, path: str, merges_file: str, special_tokens=QWEN3_SPECIAL_TOKENS, max_seq_len=None, **kwargs):
        super().__init__(path, merges_file, special_tokens=special_tokens, max_seq_len=max_seq_len, **kwargs)

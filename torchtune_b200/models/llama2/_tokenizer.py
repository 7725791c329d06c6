"""Llama-2 tokenizer (parity: torchtune/models/llama2/_tokenizer.py:21-190)."""
from .._sp_tokenizer import SentencePieceModelTokenizer


class Llama2Tokenizer(SentencePieceModelTokenizer):
    pass

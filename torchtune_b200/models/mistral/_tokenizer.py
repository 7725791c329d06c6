"""Mistral tokenizer (parity: torchtune/models/mistral/_tokenizer.py)."""
from .._sp_tokenizer import SentencePieceModelTokenizer


class MistralTokenizer(SentencePieceModelTokenizer):
    pass

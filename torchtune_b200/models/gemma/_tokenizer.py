"""Gemma tokenizer (parity: torchtune/models/gemma/_tokenizer.py)."""
from .._sp_tokenizer import SentencePieceModelTokenizer


class GemmaTokenizer(SentencePieceModelTokenizer):
    pass

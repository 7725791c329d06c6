from ._gpt2 import GPT2BaseTokenizer
from ._hf_tokenizer import HuggingFaceBaseTokenizer, HuggingFaceModelTokenizer
from ._sentencepiece import SentencePieceBaseTokenizer
from ._tiktoken import TikTokenBaseTokenizer
from ._utils import BaseTokenizer, ModelTokenizer, parse_hf_tokenizer_json, tokenize_messages_no_special_tokens

__all__ = [
    "SentencePieceBaseTokenizer",
    "TikTokenBaseTokenizer",
    "ModelTokenizer",
    "GPT2BaseTokenizer",
    "BaseTokenizer",
    "tokenize_messages_no_special_tokens",
    "parse_hf_tokenizer_json",
    "HuggingFaceBaseTokenizer",
    "HuggingFaceModelTokenizer",
]

"""Old import path of the tokenizer base classes (parity: torchtune/modules/tokenizers/__init__.py:9-31).  They live in
``torchtune_b200.modules.transforms.tokenizers``; importing from here works and warns."""
import warnings

from ..transforms.tokenizers import (  # noqa: F401
    BaseTokenizer,
    ModelTokenizer,
    SentencePieceBaseTokenizer,
    TikTokenBaseTokenizer,
    parse_hf_tokenizer_json,
    tokenize_messages_no_special_tokens,
)

__all__ = ["BaseTokenizer", "ModelTokenizer", "SentencePieceBaseTokenizer", "TikTokenBaseTokenizer", "parse_hf_tokenizer_json",
           "tokenize_messages_no_special_tokens"]

warnings.warn("torchtune_b200.modules.tokenizers moved to torchtune_b200.modules.transforms.tokenizers; update the import",
              DeprecationWarning, stacklevel=2)

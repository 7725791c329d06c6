"""SentencePiece wrapper (parity: torchtune/modules/transforms/tokenizers/_sentencepiece.py:15-118)."""
from __future__ import annotations

from typing import List, Optional

WHITESPACE_CHARS = [" ", "\n", "\t", "\r", "\v"]


class SentencePieceBaseTokenizer:
    def __init__(self, path: str):
        from sentencepiece import SentencePieceProcessor

        spm = SentencePieceProcessor()
        spm.load(path)
        self.spm_model = spm
        self.vocab_size = spm.vocab_size()
        self.bos_id = spm.bos_id()
        self.eos_id = spm.eos_id()
        self.pad_id = spm.pad_id()
        # does the vocabulary itself contain tokens with whitespace glued on?
        self.encodes_whitespace = any(spm.encode(c) for c in WHITESPACE_CHARS)

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, trim_leading_whitespace: bool = False, prefix: Optional[str] = None) -> List[int]:
        """With ``trim_leading_whitespace`` the text is encoded behind a known prefix and the
        prefix tokens are dropped, which removes the leading-space token SentencePiece would
        otherwise put in front of a continuation message."""
        if trim_leading_whitespace and self.encodes_whitespace:
            if not hasattr(self, "prefix"):
                self.prefix = prefix or "\n"
                self.encoded_prefix = self.spm_model.encode(self.prefix, add_bos=False, add_eos=False)
            start = len(self.encoded_prefix) + int(add_bos)
            return self.spm_model.encode(self.prefix + text, add_bos=add_bos, add_eos=add_eos, out_type=int)[start:]
        return self.spm_model.encode(text, add_bos=add_bos, add_eos=add_eos, out_type=int)

    def decode(self, ids: List[int]) -> str:
        return self.spm_model.decode(ids)

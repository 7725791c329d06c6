"""tiktoken BPE wrapper (parity: torchtune/modules/transforms/tokenizers/_tiktoken.py:14-160)."""
from __future__ import annotations

from typing import Dict, Iterator, List

MAX_ENCODE_CHARS = 400_000
MAX_NO_WHITESPACE_CHARS = 25_000


class TikTokenBaseTokenizer:
    """Encodes text that contains no special tokens.  Very long inputs are cut into pieces of
    at most ``MAX_ENCODE_CHARS`` and runs of more than ``MAX_NO_WHITESPACE_CHARS`` consecutive
    (non-)whitespace characters are split, which keeps tiktoken's regex from going quadratic."""

    def __init__(self, path: str, name: str, pattern: str, bos_id: int, eos_id: int, special_tokens: Dict[str, int]):
        from tiktoken import Encoding
        from tiktoken.load import load_tiktoken_bpe

        ranks = load_tiktoken_bpe(path)
        self.tt_model = Encoding(name=name, pat_str=pattern, mergeable_ranks=ranks, special_tokens=special_tokens)
        self.base_vocab_size = len(ranks)
        self.vocab_size = self.tt_model.n_vocab
        self.bos_id = bos_id
        self.eos_id = eos_id

    @staticmethod
    def _split_long_repetitions(s: str, max_run: int) -> Iterator[str]:
        run_is_space = s[0].isspace() if s else False
        run_len = 0
        start = 0
        for i, ch in enumerate(s):
            if ch.isspace() != run_is_space:
                run_is_space = not run_is_space
                run_len = 1
            else:
                run_len += 1
                if run_len > max_run:
                    yield s[start:i]
                    start = i
                    run_len = 1
        yield s[start:]

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, **_) -> List[int]:
        if not text:
            return []
        ids: List[int] = []
        for off in range(0, len(text), MAX_ENCODE_CHARS):
            for piece in self._split_long_repetitions(text[off : off + MAX_ENCODE_CHARS], MAX_NO_WHITESPACE_CHARS):
                # specials are never matched here: text is encoded as plain text
                ids.extend(self.tt_model.encode(piece, allowed_special=set(), disallowed_special=()))
        if add_bos:
            ids = [self.bos_id] + ids
        if add_eos:
            ids = ids + [self.eos_id]
        return ids

    def decode(self, token_ids: List[int], truncate_at_eos: bool = True) -> str:
        if truncate_at_eos and self.eos_id in token_ids:
            token_ids = token_ids[: token_ids.index(self.eos_id)]
        return self.tt_model.decode(token_ids)

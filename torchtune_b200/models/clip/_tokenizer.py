"""CLIP byte-level BPE tokenizer (parity: torchtune/models/clip/_tokenizer.py:15-240).

Vocabulary layout (fixed by the original model): the 256 byte symbols, the same 256 symbols
with the end-of-word marker, one entry per merge rule in file order, then the start and end
of text specials.  Text is lower-cased, split by CLIP's pattern, and every word is merged with
its last symbol carrying the end-of-word marker.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Tuple

import regex as re

from ...modules.transforms.tokenizers._gpt2 import bytes_to_unicode
from ...modules.transforms.tokenizers._utils import BaseTokenizer

WORD_BOUNDARY = "</w>"
_SOT, _EOT = "<|startoftext|>", "<|endoftext|>"


def _read_merges(path: str) -> List[Tuple[str, str]]:
    rules = []
    with open(path, encoding="utf-8") as f:
        for i, line in enumerate(f):
            line = line.strip()
            if not line or (i == 0 and line.startswith("#version:")):
                continue
            rules.append(tuple(line.split()))
    return rules


class CLIPTokenizer(BaseTokenizer):
    def __init__(self, path: str, max_seq_len: int = 77, truncate: bool = True):
        self.max_seq_len, self.truncate = max_seq_len, truncate
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {v: k for k, v in self.byte_encoder.items()}
        merges = _read_merges(path)
        symbols = list(self.byte_encoder.values())
        vocab = symbols + [s + WORD_BOUNDARY for s in symbols] + ["".join(m) for m in merges] + [_SOT, _EOT]
        self.encoder: Dict[str, int] = {w: i for i, w in enumerate(vocab)}
        self.decoder = {i: w for w, i in self.encoder.items()}
        self.bpe_ranks = {m: i for i, m in enumerate(merges)}
        self.pat = re.compile(r"""<\|startoftext\|>|<\|endoftext\|>|'s|'t|'re|'ve|'m|'ll|'d|[\p{L}]+|[\p{N}]|[^\s\p{L}\p{N}]+""", re.IGNORECASE)
        self.sot_token, self.eot_token = self.encoder[_SOT], self.encoder[_EOT]
        self.pad_token = self.eot_token
        self._cache: Dict[str, List[str]] = {_SOT: [_SOT], _EOT: [_EOT]}

    def _merge_word(self, word: str) -> List[str]:
        if word in self._cache:
            return self._cache[word]
        parts = list(word[:-1]) + [word[-1] + WORD_BOUNDARY]
        while len(parts) > 1:
            ranked = [(self.bpe_ranks.get((a, b), None), i) for i, (a, b) in enumerate(zip(parts, parts[1:]))]
            ranked = [(r, i) for r, i in ranked if r is not None]
            if not ranked:
                break
            best_rank = min(ranked)[0]
            pair = next((parts[i], parts[i + 1]) for r, i in ranked if r == best_rank)
            merged, i = [], 0
            while i < len(parts):
                if i + 1 < len(parts) and (parts[i], parts[i + 1]) == pair:
                    merged.append(parts[i] + parts[i + 1])
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        self._cache[word] = parts
        return parts

    def encode(self, text: str) -> List[int]:
        text = text.replace("’", "'").lower()
        tokens = [self.sot_token]
        for piece in re.findall(self.pat, text):
            word = "".join(self.byte_encoder[b] for b in piece.encode("utf-8"))
            tokens.extend(self.encoder[t] for t in self._merge_word(word))
            if len(tokens) >= self.max_seq_len:
                break
        tokens.append(self.eot_token)
        if len(tokens) > self.max_seq_len:
            assert self.truncate, "Tokenized text is larger than the maximum sequence length but truncate is set to False."
            tokens = tokens[: self.max_seq_len]
            tokens[-1] = self.eot_token
        return tokens

    def decode(self, tokens: List[int]) -> str:
        text = "".join(self.decoder[t] for t in tokens)
        out, i = bytearray(), 0
        while i < len(text):
            if text.startswith(WORD_BOUNDARY, i):
                out.extend(b" ")
                i += len(WORD_BOUNDARY)
            elif text[i] in self.byte_decoder:
                out.append(self.byte_decoder[text[i]])
                i += 1
            else:  # characters of the special tokens
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out.decode("utf-8", errors="replace")

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        sample = dict(sample)
        sample["tokens"] = self.encode(sample.pop("text"))
        return sample

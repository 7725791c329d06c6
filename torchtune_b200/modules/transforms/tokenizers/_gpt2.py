"""Byte-level BPE tokenizer in the GPT-2 file format (``vocab.json`` + ``merges.txt``)
(parity: torchtune/modules/transforms/tokenizers/_gpt2.py:15-230)."""
from __future__ import annotations

import json
import re
from functools import lru_cache
from typing import Dict, List, Optional, Tuple


@lru_cache()
def bytes_to_unicode() -> Dict[int, str]:
    """Reversible byte → printable-unicode table: printable Latin-1 bytes map to themselves,
    the remaining bytes to code points from 256 upwards (so merges never see whitespace or
    control characters)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    table = {b: chr(b) for b in keep}
    extra = 0
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + extra)
            extra += 1
    return table


def get_pairs(word: Tuple[str, ...]) -> set:
    return set(zip(word[:-1], word[1:]))


class GPT2BaseTokenizer:
    def __init__(self, vocab_path: str, merges_path: str, unk_id: Optional[int] = None, bos_id: Optional[int] = None, eos_id: Optional[int] = None, pad_id: Optional[int] = None):
        with open(vocab_path, encoding="utf-8") as f:
            self.encoder: Dict[str, int] = json.load(f)
        self.decoder = {i: t for t, i in self.encoder.items()}
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {c: b for b, c in self.byte_encoder.items()}
        with open(merges_path, encoding="utf-8") as f:
            lines = f.read().split("\n")[1:-1]
        self.bpe_ranks = {tuple(line.split()): rank for rank, line in enumerate(lines)}
        self.cache: Dict[str, str] = {}
        self.pat = re.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?[\w]+| ?\d+| ?[^\s\w\d]+|\s+(?!\S)|\s+""", re.UNICODE)
        self.unk_id, self.bos_id, self.eos_id, self.pad_id = unk_id, bos_id, eos_id, pad_id

    @property
    def vocab_size(self) -> int:
        return len(self.encoder)

    def bpe(self, token: str) -> str:
        """Apply merges greedily by rank; returns the space-joined sub-tokens."""
        if token in self.cache:
            return self.cache[token]
        word = tuple(token)
        while len(word) > 1:
            ranked = [(self.bpe_ranks.get(pair, float("inf")), pair) for pair in get_pairs(word)]
            rank, (a, b) = min(ranked)
            if rank == float("inf"):
                break
            merged: List[str] = []
            i = 0
            while i < len(word):
                if i < len(word) - 1 and word[i] == a and word[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            word = tuple(merged)
        out = " ".join(word)
        self.cache[token] = out
        return out

    def _tokenize(self, text: str) -> List[str]:
        pieces: List[str] = []
        for chunk in self.pat.findall(text):
            mapped = "".join(self.byte_encoder[b] for b in chunk.encode("utf-8"))
            pieces.extend(self.bpe(mapped).split(" "))
        return pieces

    def _convert_token_to_id(self, token: str) -> int:
        return self.encoder.get(token, self.unk_id)

    def _convert_id_to_token(self, index: int) -> str:
        return self.decoder.get(index)

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, **_) -> List[int]:
        ids = [self._convert_token_to_id(t) for t in self._tokenize(text)]
        if add_bos and self.bos_id is not None:
            ids = [self.bos_id] + ids
        if add_eos and self.eos_id is not None:
            ids = ids + [self.eos_id]
        return ids

    def decode(self, tokens: List[int]) -> str:
        text = "".join(self._convert_id_to_token(t) or "" for t in tokens)
        return bytearray(self.byte_decoder[c] for c in text if c in self.byte_decoder).decode("utf-8", errors="replace")

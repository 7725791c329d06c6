"""Qwen2 byte-level BPE tokenizer with ChatML-style turn markers
(parity: torchtune/models/qwen2/_tokenizer.py:21-430)."""
from __future__ import annotations

import unicodedata
from typing import Any, Dict, List, Mapping, Optional, Tuple

import regex as re

from ...data._messages import Message
from ...data._utils import truncate
from ...modules.transforms.tokenizers import GPT2BaseTokenizer

PRETOKENIZE_REGEX = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
ENDOFTEXT, IM_START, IM_END = "<|endoftext|>", "<|im_start|>", "<|im_end|>"
QWEN2_SPECIAL_TOKENS = {ENDOFTEXT: 151643, IM_START: 151644, IM_END: 151645}


class Qwen2Tokenizer(GPT2BaseTokenizer):
    """``path`` is ``vocab.json``, ``merges_file`` is ``merges.txt``.  Text is NFC-normalised,
    split at special tokens (which map straight to their ids) and BPE-encoded in between.
    Every turn is ``<|im_start|>role\\n … <|im_end|>\\n``; a final assistant turn is left open
    and the sequence ends with ``eos`` (``<|im_end|>``)."""

    def __init__(self, path: str, merges_file: str, special_tokens: Dict[str, int] = QWEN2_SPECIAL_TOKENS, max_seq_len: Optional[int] = None, *, prompt_template=None, errors: str = "replace", unk_token: Optional[str] = None, bos_token: Optional[str] = None, eos_token: str = IM_END, pad_token: Optional[str] = ENDOFTEXT, bpe_cache_size: int = 152064, truncation_type: str = "right"):
        super().__init__(path, merges_file)
        self.pat = re.compile(PRETOKENIZE_REGEX)
        self.errors = errors
        self.special_tokens = dict(special_tokens)
        self._special_by_id = {i: t for t, i in self.special_tokens.items()}
        pick = lambda tok: None if tok is None else self.special_tokens[tok]  # noqa: E731
        self.unk_id, self.bos_id, self.eos_id, self.pad_id = pick(unk_token), pick(bos_token), pick(eos_token), pick(pad_token)
        self.im_start_id, self.im_end_id = self.special_tokens[IM_START], self.special_tokens[IM_END]
        self.stop_tokens = [self.eos_id, self.pad_id]
        alternation = "|".join(re.escape(t) for t in sorted(self.special_tokens, key=len, reverse=True))
        self._split_specials = re.compile(f"({alternation})")
        self.max_seq_len = max_seq_len
        self.prompt_template = prompt_template
        self.truncation_type = truncation_type

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, **_) -> List[int]:
        text = unicodedata.normalize("NFC", text)
        ids: List[int] = []
        if add_bos and self.bos_id is not None:
            ids.append(self.bos_id)
        for piece in self._split_specials.split(text):
            if not piece:
                continue
            if piece in self.special_tokens:
                ids.append(self.special_tokens[piece])
            else:
                ids.extend(self._convert_token_to_id(t) for t in self._tokenize(piece))
        if add_eos and self.eos_id is not None:
            ids.append(self.eos_id)
        return ids

    def decode(self, token_ids: List[int], skip_special_tokens: bool = False) -> str:
        out, run = [], []

        def flush():
            if run:
                text = "".join(run)
                out.append(bytearray(self.byte_decoder[c] for c in text).decode("utf-8", errors=self.errors))
                run.clear()

        for t in token_ids:
            if t in self._special_by_id:
                flush()
                if not skip_special_tokens:
                    out.append(self._special_by_id[t])
            else:
                run.append(self._convert_id_to_token(t) or "")
        flush()
        return "".join(out)

    # -- conversation layout -----------------------------------------------------------
    def _open(self, role: str) -> List[int]:
        return [self.im_start_id] + self.encode(f"{role}\n", add_bos=False, add_eos=False)

    def _close(self) -> List[int]:
        return [self.im_end_id] + self.encode("\n", add_bos=False, add_eos=False)

    def _header(self, messages: List[Message], i: int) -> List[int]:
        return [] if messages[i].role == "ipython" else self._open(messages[i].role)

    def _footer(self, messages: List[Message], i: int) -> List[int]:
        m = messages[i]
        if m.role == "ipython" or (m.role == "assistant" and i == len(messages) - 1):
            return []
        return self._close()

    def tokenize_messages(self, messages: List[Message], *, add_end_tokens: bool = True) -> Tuple[List[int], List[bool]]:
        if self.prompt_template is not None:
            messages = self.prompt_template(messages)
        tokens: List[int] = []
        mask: List[bool] = []
        for i, m in enumerate(messages):
            ids = self._header(messages, i)
            for part in m.content:
                if part["type"] != "text":
                    raise RuntimeError(f"Unsupported message content type: {part['type']}")
                ids += self.encode(part["content"], add_bos=False, add_eos=False)
            ids += self._footer(messages, i)
            tokens += ids
            mask += [m.masked] * len(ids)
            if self.max_seq_len and len(tokens) >= self.max_seq_len:
                break
        if add_end_tokens:
            tokens.append(self.eos_id)
            mask.append(mask[-1] if mask else True)
        if self.max_seq_len:
            tokens = truncate(tokens, self.max_seq_len, self.eos_id if add_end_tokens else None, self.truncation_type)
            mask = truncate(mask, self.max_seq_len, True if add_end_tokens else None, self.truncation_type)
        return tokens, mask

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        messages = sample.pop("messages")
        tokens, mask = self.tokenize_messages(messages, add_end_tokens=not inference)
        sample["tokens"], sample["mask"] = tokens, mask
        return sample

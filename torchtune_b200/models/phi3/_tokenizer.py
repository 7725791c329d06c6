"""Phi-3 mini tokenizer: SentencePiece plus role markers
(parity: torchtune/models/phi3/_tokenizer.py:18-290)."""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Tuple

from ...data._messages import Message
from ...data._utils import truncate
from ...modules.transforms.tokenizers import SentencePieceBaseTokenizer

_NAMES = ["<|endoftext|>", "<|assistant|>", "<|placeholder1|>", "<|placeholder2|>", "<|placeholder3|>", "<|placeholder4|>", "<|system|>", "<|end|>", "<|placeholder5|>", "<|placeholder6|>", "<|user|>"]
PHI3_SPECIAL_TOKENS = {name: 32000 + i for i, name in enumerate(_NAMES)}


class Phi3MiniTokenizer:
    """Each message becomes ``<|role|>\\n text <|end|>\\n``; BOS opens every turn and EOS
    (``<|endoftext|>``) follows each assistant message when ``add_end_tokens`` is set."""

    def __init__(self, path: str, special_tokens: Optional[Dict[str, int]] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
        self._spm_model = SentencePieceBaseTokenizer(path)
        self.special_tokens = special_tokens if special_tokens is not None else PHI3_SPECIAL_TOKENS
        self.eos_id = self.special_tokens["<|endoftext|>"]
        self.pad_id = self.special_tokens["<|endoftext|>"]
        self.stop_tokens = [self.eos_id, self.special_tokens["<|end|>"]]
        self.max_seq_len = max_seq_len
        self.prompt_template = prompt_template
        self.truncation_type = truncation_type

    vocab_size = property(lambda self: self._spm_model.vocab_size)
    bos_id = property(lambda self: self._spm_model.bos_id)

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, trim_leading_whitespace: bool = False) -> List[int]:
        return self._spm_model.encode(text, add_bos=add_bos, add_eos=add_eos, trim_leading_whitespace=trim_leading_whitespace)

    def decode(self, ids: List[int]) -> str:
        return self._spm_model.decode([i for i in ids if not 32_000 <= i <= 32_064])

    def tokenize_messages(self, messages: List[Message], *, add_end_tokens: bool = False, ignore_system_prompt: bool = False, add_eos: Optional[bool] = None) -> Tuple[List[int], List[bool]]:
        if add_eos is not None:
            add_end_tokens = add_eos
        if self.prompt_template is not None:
            messages = self.prompt_template(messages)
        newline = self.encode("\n", add_bos=False, add_eos=False)
        role_token = {"user": "<|user|>", "assistant": "<|assistant|>", "system": "<|system|>"}
        tokens: List[int] = []
        mask: List[bool] = []
        turn_start = True
        for m in messages:
            if ignore_system_prompt and m.role == "system":
                continue
            if m.role not in role_token:
                raise ValueError(f"Unknown role '{m.role}' for message: '{m.content}'")
            ids: List[int] = [self.bos_id] if turn_start else []
            ids.append(self.special_tokens[role_token[m.role]])
            ids += newline
            for part in m.content:
                if part["type"] != "text":
                    raise RuntimeError(f"Unsupported message content type: {part['type']}")
                ids += self.encode(part["content"].rstrip(" "), add_bos=False, add_eos=False, trim_leading_whitespace=True)
            ids += [self.special_tokens["<|end|>"]] + newline
            if m.role == "assistant" and add_end_tokens:
                ids.append(self.eos_id)
                turn_start = True
            else:
                turn_start = False
            tokens += ids
            mask += [m.masked] * len(ids)
            if self.max_seq_len and len(tokens) >= self.max_seq_len:
                break
        if self.max_seq_len and len(tokens) >= self.max_seq_len:
            tokens = truncate(tokens, self.max_seq_len, self.eos_id if add_end_tokens else None, self.truncation_type)
            mask = truncate(mask, self.max_seq_len, True if add_end_tokens else None, self.truncation_type)
        return tokens, mask

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        messages = sample.pop("messages")
        tokens, mask = self.tokenize_messages(messages, add_end_tokens=not inference)
        sample["tokens"], sample["mask"] = tokens, mask
        return sample

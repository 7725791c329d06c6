"""Tokenizer protocols and shared helpers
(parity: torchtune/modules/transforms/tokenizers/_utils.py:18-230)."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Protocol, Tuple

from ....data._messages import Message
from ....data._utils import truncate


class BaseTokenizer(Protocol):
    """String ↔ token ids."""

    def encode(self, text: str, **kwargs: Dict[str, Any]) -> List[int]: ...

    def decode(self, token_ids: List[int], **kwargs: Dict[str, Any]) -> str: ...


class ModelTokenizer(Protocol):
    """Model-specific tokenizer: knows its special tokens and how to lay out a conversation."""

    special_tokens: Dict[str, int]
    max_seq_len: Optional[int]

    def tokenize_messages(self, messages: List[Message], **kwargs: Dict[str, Any]) -> Tuple[List[int], List[bool]]: ...


def tokenize_messages_no_special_tokens(
    tokenizer: ModelTokenizer,
    messages: List[Message],
    *,
    bos_id: Optional[int] = None,
    eos_id: Optional[int] = None,
    truncation_type: str = "right",
) -> Tuple[List[int], List[bool]]:
    """Encode messages one by one and concatenate, adding only BOS at the start of each turn
    and EOS after each assistant message.  Leading whitespace of a continuation message is
    trimmed unless the previous message ended with a space.  Returns ``(tokens, mask)``;
    the result is truncated to ``tokenizer.max_seq_len``."""
    tokens: List[int] = []
    mask: List[bool] = []
    turn_start = True
    prev_trailing_space = False
    limit = tokenizer.max_seq_len
    last_masked = False
    for msg in messages:
        last_masked = msg.masked
        if turn_start and bos_id is not None:
            tokens.append(bos_id)
            mask.append(msg.masked)
        trim = (not turn_start) and not prev_trailing_space
        piece: List[int] = []
        text = ""
        for part in msg.content:
            if part["type"] != "text":
                raise RuntimeError(f"Unsupported message content type: {part['type']}")
            text = part["content"]
            piece += tokenizer.encode(text.rstrip(" "), add_bos=False, add_eos=False, trim_leading_whitespace=trim)
        prev_trailing_space = text.endswith(" ")
        tokens += piece
        mask += [msg.masked] * len(piece)
        if msg.role == "assistant":
            if eos_id is not None:
                tokens.append(eos_id)
                mask.append(msg.masked)
            turn_start = True
        else:
            turn_start = False
        if limit is not None and len(tokens) >= limit:
            break
    if limit is not None:
        tokens = truncate(tokens, limit, eos_id, truncation_type=truncation_type)
        mask = truncate(mask, limit, last_masked if eos_id is not None else None, truncation_type=truncation_type)
    return tokens, mask


def parse_hf_tokenizer_json(tokenizer_json_path: str) -> Dict[str, int]:
    """``added_tokens`` of a HF ``tokenizer.json`` as ``{token string: id}``."""
    with open(tokenizer_json_path, "r") as f:
        data = json.load(f)
    return {tok["content"]: tok["id"] for tok in data["added_tokens"]}

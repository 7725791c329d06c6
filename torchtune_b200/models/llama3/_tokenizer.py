"""Llama-3 tokenizer (parity: torchtune/models/llama3/_tokenizer.py:18-380): tiktoken BPE plus
the header / end-of-turn special tokens."""
from __future__ import annotations

import re
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ...data._messages import Message
from ...data._utils import truncate
from ...modules.transforms.tokenizers import TikTokenBaseTokenizer

CL100K_PATTERN = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""  # noqa: E501

_NAMED = {
    "<|begin_of_text|>": 128000,
    "<|end_of_text|>": 128001,
    "<|reserved_special_token_0|>": 128002,
    "<|reserved_special_token_1|>": 128003,
    "<|finetune_right_pad_id|>": 128004,
    "<|step_id|>": 128005,
    "<|start_header_id|>": 128006,
    "<|end_header_id|>": 128007,
    "<|eom_id|>": 128008,
    "<|eot_id|>": 128009,
    "<|python_tag|>": 128010,
    "<|image|>": 128256,
    "<|video|>": 128012,
    "<|reserved_special_token_245|>": 128011,
}
NUM_RESERVED_SPECIAL_TOKENS = 257
SPECIAL_TOKENS = dict(_NAMED)
RESERVED_TOKENS = {f"<|reserved_special_token_{2 + i}|>": 128013 + i for i in range(NUM_RESERVED_SPECIAL_TOKENS - len(_NAMED))}
LLAMA3_SPECIAL_TOKENS = {**SPECIAL_TOKENS, **RESERVED_TOKENS}
_REQUIRED = ("<|begin_of_text|>", "<|end_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eom_id|>", "<|eot_id|>", "<|python_tag|>")


class Llama3Tokenizer:
    """Conversation layout: ``<|begin_of_text|>`` (masked) then, per message,
    ``<|start_header_id|>role<|end_header_id|>\\n\\n body <|eot_id|>`` (``<|eom_id|>`` when the
    message does not end the turn), and a masked ``<|end_of_text|>`` at the end."""

    def __init__(self, path: str, special_tokens: Optional[Dict[str, int]] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
        self.special_tokens = special_tokens if special_tokens is not None else LLAMA3_SPECIAL_TOKENS
        for tok in _REQUIRED:
            if tok not in self.special_tokens:
                raise ValueError(f"{tok} missing from special_tokens")
        st = self.special_tokens
        self.bos_id, self.eos_id = st["<|begin_of_text|>"], st["<|end_of_text|>"]
        self.pad_id = st.get("<|finetune_right_pad_id|>", 128004)
        self.step_id = st.get("<|step_id|>", 128005)
        self.start_header_id, self.end_header_id = st["<|start_header_id|>"], st["<|end_header_id|>"]
        self.eom_id, self.eot_id, self.python_tag = st["<|eom_id|>"], st["<|eot_id|>"], st["<|python_tag|>"]
        self.image_id = st.get("<|image|>", 128256)
        self.stop_tokens = [self.eos_id, self.eot_id, self.eom_id]
        self.tt_model = TikTokenBaseTokenizer(path=path, name="llama3_tiktoken", pattern=CL100K_PATTERN, bos_id=self.bos_id, eos_id=self.eos_id, special_tokens=self.special_tokens)
        self.max_seq_len = max_seq_len
        self.prompt_template = prompt_template
        self.truncation_type = truncation_type
        self._special_re = re.compile(r"<\|.*?\|>")
        self._header_re = re.compile(r"<\|start_header_id\|>.*?<\|end_header_id\|>\n\n")

    @property
    def base_vocab_size(self) -> int:
        return self.tt_model.base_vocab_size

    @property
    def vocab_size(self) -> int:
        return self.tt_model.vocab_size

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        return self.tt_model.encode(text=text, add_bos=add_bos, add_eos=add_eos)

    def decode(self, token_ids: List[int], truncate_at_eos: bool = True, skip_special_tokens: bool = True) -> str:
        text = self.tt_model.decode(token_ids, truncate_at_eos=truncate_at_eos)
        if skip_special_tokens:
            # headers first ("user\n\n" would otherwise stay behind), then any remaining special token
            text = self._special_re.sub("", self._header_re.sub("", text))
        return text

    def _header(self, message: Message) -> List[int]:
        return [self.start_header_id] + self.encode(message.role.strip(), add_bos=False, add_eos=False) + [self.end_header_id] + self.encode("\n\n", add_bos=False, add_eos=False)

    def _body(self, message: Message) -> List[int]:
        out: List[int] = []
        for part in message.content:
            if part["type"] == "text":
                out += self.encode(part["content"].strip(), add_bos=False, add_eos=False)
            elif part["type"] == "image":
                out.append(self.image_id)
            else:
                raise RuntimeError(f"Unsupported message content type: {part['type']}")
        if message.ipython:
            out = [self.python_tag] + out
        return out

    def tokenize_message(self, message: Message, *, add_start_tokens: bool = True, add_end_tokens: bool = True) -> List[int]:
        start = self._header(message) if add_start_tokens else []
        end = ([self.eot_id] if message.eot else [self.eom_id]) if add_end_tokens else []
        return start + self._body(message) + end

    def tokenize_messages(self, messages: List[Message], *, add_end_tokens: bool = True) -> Tuple[List[int], List[bool]]:
        if self.prompt_template is not None:
            messages = self.prompt_template(messages)
        tokens, mask = [self.bos_id], [True]
        for i, m in enumerate(messages):
            # only the final message may be left open (generation prompt)
            closing = add_end_tokens if i == len(messages) - 1 else True
            ids = self.tokenize_message(m, add_end_tokens=closing)
            tokens += ids
            mask += [m.masked] * len(ids)
            if self.max_seq_len and len(tokens) >= self.max_seq_len:
                break
        if add_end_tokens:
            tokens.append(self.eos_id)
            mask.append(True)
        if self.max_seq_len:
            tokens = truncate(tokens, self.max_seq_len, self.eos_id if add_end_tokens else None, self.truncation_type)
            mask = truncate(mask, self.max_seq_len, True if add_end_tokens else None, self.truncation_type)
        return tokens, mask

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        messages = sample.pop("messages")
        tokens, mask = self.tokenize_messages(messages, add_end_tokens=not inference)
        sample["tokens"], sample["mask"] = tokens, mask
        return sample

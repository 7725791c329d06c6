"""Phi-4 tokenizer: byte-level BPE (GPT-2 file format) with ``<|im_start|>role<|im_sep|> … <|im_end|>``
turns (parity: torchtune/models/phi4/_tokenizer.py:13-180)."""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Tuple

from ...data._messages import Message
from ...data._utils import truncate
from ...modules.transforms.tokenizers import GPT2BaseTokenizer

_HEAD = ["<|dummy_0|>", "<|endoftext|>", "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>", "<|dummy_1|>", "<|dummy_2|>", "<|dummy_3|>", "<|im_start|>", "<|im_end|>", "<|im_sep|>"]
PHI4_SPECIAL_TOKENS = {name: 100256 + i for i, name in enumerate(_HEAD)}
PHI4_SPECIAL_TOKENS["<|endofprompt|>"] = 100276
_next = 4
for _tid in range(100267, 100352):
    if _tid != 100276:
        PHI4_SPECIAL_TOKENS[f"<|dummy_{_next}|>"] = _tid
        _next += 1


class Phi4Tokenizer:
    def __init__(self, vocab_path: str = None, merges_path: str = None, special_tokens: Optional[Dict[str, int]] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
        self.special_tokens = special_tokens if special_tokens is not None else PHI4_SPECIAL_TOKENS
        self.eos_id = self.special_tokens["<|im_end|>"]
        self.bos_id = self.special_tokens["<|endoftext|>"]
        self.pad_id = self.special_tokens["<|dummy_85|>"] if "<|dummy_85|>" in self.special_tokens else self.bos_id
        self.stop_tokens = [self.eos_id]
        self.max_seq_len = max_seq_len
        self.prompt_template = prompt_template
        self.truncation_type = truncation_type
        self.tokenizer_model = GPT2BaseTokenizer(vocab_path, merges_path, self.eos_id, self.bos_id, self.eos_id, self.pad_id)

    vocab_size = property(lambda self: self.tokenizer_model.vocab_size)

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        return self.tokenizer_model.encode(text=text, add_bos=add_bos, add_eos=add_eos)

    def decode(self, ids: List[int], skip_special_tokens: bool = True) -> str:
        return self.tokenizer_model.decode([i for i in ids if not (skip_special_tokens and 100_256 <= i <= 100_351)])

    def _tokenize_header(self, role: str) -> List[int]:
        return [self.special_tokens["<|im_start|>"]] + self.encode(role, add_bos=False, add_eos=False) + [self.special_tokens["<|im_sep|>"]]

    def tokenize_messages(self, messages: List[Message], *, add_end_tokens: bool = True, ignore_system_prompt: bool = False) -> Tuple[List[int], List[bool]]:
        if self.prompt_template is not None:
            messages = self.prompt_template(messages)
        tokens: List[int] = []
        mask: List[bool] = []
        for m in messages:
            if ignore_system_prompt and m.role == "system":
                continue
            ids = self._tokenize_header(m.role)
            for part in m.content:
                if part["type"] != "text":
                    raise RuntimeError(f"Unsupported message content type: {part['type']}")
                ids += self.encode(part["content"].rstrip(" "), add_bos=False, add_eos=False)
            if m.role != "assistant" or add_end_tokens:
                ids.append(self.special_tokens["<|im_end|>"])
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

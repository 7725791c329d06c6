"""SentencePiece-based model tokenizer shared by Llama-2, Mistral and Gemma
(parity: torchtune/models/llama2/_tokenizer.py:21-190, torchtune/models/mistral/_tokenizer.py,
torchtune/models/gemma/_tokenizer.py): BOS at each turn start, EOS after each assistant
message, no other special tokens."""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Tuple

from ..data._messages import Message
from ..modules.transforms.tokenizers import SentencePieceBaseTokenizer, tokenize_messages_no_special_tokens


class SentencePieceModelTokenizer:
    default_pad_id = 0

    def __init__(self, path: str, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
        self._spm_model = SentencePieceBaseTokenizer(path)
        # the underlying model has no pad piece; pad with id 0 as the original checkpoints do
        self._spm_model.pad_id = self.default_pad_id
        self.stop_tokens = [self.eos_id]
        self.special_tokens = {}
        self.max_seq_len = max_seq_len
        self.prompt_template = prompt_template
        self.truncation_type = truncation_type

    eos_id = property(lambda self: self._spm_model.eos_id)
    bos_id = property(lambda self: self._spm_model.bos_id)
    pad_id = property(lambda self: self._spm_model.pad_id)
    vocab_size = property(lambda self: self._spm_model.vocab_size)

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, trim_leading_whitespace: bool = False) -> List[int]:
        return self._spm_model.encode(text, add_bos=add_bos, add_eos=add_eos, trim_leading_whitespace=trim_leading_whitespace)

    def decode(self, token_ids: List[int]) -> str:
        return self._spm_model.decode(token_ids)

    def tokenize_messages(self, messages: List[Message], *, add_start_tokens: bool = True, add_end_tokens: bool = True, add_eos: Optional[bool] = None) -> Tuple[List[int], List[bool]]:
        if add_eos is not None:
            add_end_tokens = add_eos
        if self.prompt_template is not None:
            messages = self.prompt_template(messages)
        return tokenize_messages_no_special_tokens(
            tokenizer=self,
            messages=messages,
            bos_id=self.bos_id if add_start_tokens else None,
            eos_id=self.eos_id if add_end_tokens else None,
            truncation_type=self.truncation_type,
        )

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        messages = sample.pop("messages")
        tokens, mask = self.tokenize_messages(messages, add_end_tokens=not inference)
        sample["tokens"], sample["mask"] = tokens, mask
        return sample

"""Named dataset builders referenced from configs (parity: torchtune/datasets/_alpaca.py,
_chat.py, _instruct.py, _grammar.py, _samsum.py, _slimorca.py, _hh_rlhf_helpful.py,
_stack_exchange_paired.py, _cnn_dailymail.py, _wikitext.py).  Every builder takes the tokenizer
positionally and forwards unknown keyword arguments to ``datasets.load_dataset``."""
from __future__ import annotations

from functools import partial
from typing import Any, Callable, Dict, Mapping, Optional, Union

from ..data._messages import AlpacaToMessages, ChosenRejectedToMessages, InputOutputToMessages, Message, OpenAIToMessages, ShareGPTToMessages
from ._packed import PackedDataset
from ._preference import PreferenceDataset
from ._sft import SFTDataset
from ._text_completion import TextCompletionDataset, text_completion_dataset


def _strategy(train_on_input: bool) -> str:
    return "train_on_all" if train_on_input else "train_on_assistant"


def _maybe_pack(ds: SFTDataset, tokenizer, packed: bool) -> Union[SFTDataset, PackedDataset]:
    if not packed:
        return ds
    if tokenizer.max_seq_len is None:
        raise ValueError("PackedDataset requires a max_seq_len to be set on the tokenizer.")
    return PackedDataset(ds, max_seq_len=tokenizer.max_seq_len, padding_idx=getattr(tokenizer, "pad_id", 0) or 0)


def _sft(tokenizer, source, transform, packed, filter_fn, split, kwargs):
    ds = SFTDataset(source=source, message_transform=transform, model_transform=tokenizer, filter_fn=filter_fn, split=split, **kwargs)
    return _maybe_pack(ds, tokenizer, packed)


def alpaca_dataset(tokenizer, *, source: str = "tatsu-lab/alpaca", column_map: Optional[Dict[str, str]] = None, train_on_input: bool = True, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """Alpaca-style instruction data; the prompt is trained on by default."""
    return _sft(tokenizer, source, AlpacaToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map), packed, filter_fn, split, load_dataset_kwargs)


alpaca_cleaned_dataset = partial(alpaca_dataset, source="yahma/alpaca-cleaned")
alpaca_cleaned_dataset.__doc__ = "``alpaca_dataset`` on the cleaned release ``yahma/alpaca-cleaned``."


def instruct_dataset(tokenizer, *, source: str, column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """Custom ``input`` / ``output`` column data."""
    transform = InputOutputToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map, new_system_prompt=new_system_prompt)
    return _sft(tokenizer, source, transform, packed, filter_fn, split, load_dataset_kwargs)


def chat_dataset(tokenizer, *, source: str, conversation_column: str, conversation_style: str, train_on_input: bool = False, new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """Multi-turn chat data in ``sharegpt`` or ``openai`` layout."""
    if conversation_style == "sharegpt":
        transform = ShareGPTToMessages(masking_strategy=_strategy(train_on_input), column_map={"conversations": conversation_column}, new_system_prompt=new_system_prompt)
    elif conversation_style == "openai":
        transform = OpenAIToMessages(masking_strategy=_strategy(train_on_input), column_map={"messages": conversation_column}, new_system_prompt=new_system_prompt)
    else:
        raise ValueError(f"Unsupported conversation style: {conversation_style}")
    return _sft(tokenizer, source, transform, packed, filter_fn, split, load_dataset_kwargs)


def grammar_dataset(tokenizer, *, source: str = "liweili/c4_200m", column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """Grammar-correction pairs (pair with ``GrammarErrorCorrectionTemplate``)."""
    transform = InputOutputToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map, new_system_prompt=new_system_prompt)
    return _sft(tokenizer, source, transform, packed, filter_fn, split, load_dataset_kwargs)


def samsum_dataset(tokenizer, *, source: str = "Samsung/samsum", column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """Dialogue summarisation (pair with ``SummarizeTemplate``)."""
    transform = InputOutputToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map or {"input": "dialogue", "output": "summary"}, new_system_prompt=new_system_prompt)
    return _sft(tokenizer, source, transform, packed, filter_fn, split, load_dataset_kwargs)


def slimorca_dataset(tokenizer, *, source: str = "Open-Orca/SlimOrca-Dedup", column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """SlimOrca ShareGPT-format conversations."""
    transform = ShareGPTToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map, new_system_prompt=new_system_prompt)
    return _sft(tokenizer, source, transform, packed, filter_fn, split, load_dataset_kwargs)


def hh_rlhf_helpful_dataset(tokenizer, *, source: str = "RLHFlow/HH-RLHF-Helpful-standard", column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, new_system_prompt: Optional[str] = None, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> PreferenceDataset:
    """Anthropic helpful/harmless pairs (standardised helpful subset)."""
    transform = ChosenRejectedToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map, new_system_prompt=new_system_prompt)
    return PreferenceDataset(source=source, message_transform=transform, tokenizer=tokenizer, filter_fn=filter_fn, split=split, **load_dataset_kwargs)


class StackExchangePairedToMessages:
    """Rows with one ``prompt`` and two answers (``chosen`` / ``rejected``) → a pair of
    two-message conversations; the prompt is masked unless ``train_on_input``."""

    def __init__(self, train_on_input: bool = False, column_map: Optional[Dict[str, str]] = None):
        self.train_on_input = train_on_input
        self._column_map = column_map or {}

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        cm = self._column_map
        prompt = sample[cm.get("prompt", "prompt")]

        def side(answer_key: str):
            return [Message(role="user", content=prompt, masked=not self.train_on_input), Message(role="assistant", content=sample[answer_key])]

        return {"chosen": side(cm.get("chosen", "chosen")), "rejected": side(cm.get("rejected", "rejected"))}


def stack_exchange_paired_dataset(tokenizer, *, source: str = "lvwerra/stack-exchange-paired", column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> PreferenceDataset:
    column_map = column_map or {"prompt": "question", "chosen": "response_j", "rejected": "response_k"}
    transform = StackExchangePairedToMessages(train_on_input=train_on_input, column_map=column_map)
    load_dataset_kwargs.setdefault("data_dir", "data/rl")
    return PreferenceDataset(source=source, message_transform=transform, tokenizer=tokenizer, filter_fn=filter_fn, split=split, **load_dataset_kwargs)


def cnn_dailymail_articles_dataset(tokenizer, source: str = "ccdv/cnn_dailymail", max_seq_len: Optional[int] = None, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> TextCompletionDataset:
    """News articles as plain text (dataset version 3.0.0)."""
    load_dataset_kwargs.setdefault("name", "3.0.0")
    return TextCompletionDataset(tokenizer=tokenizer, source=source, column="article", filter_fn=filter_fn, split=split, **load_dataset_kwargs)


def wikitext_dataset(tokenizer, source: str = "EleutherAI/wikitext_document_level", subset: str = "wikitext-103-v1", max_seq_len: Optional[int] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any):
    """Document-level WikiText for continued pre-training."""
    return text_completion_dataset(tokenizer=tokenizer, source=source, column="page", name=subset, packed=packed, filter_fn=filter_fn, split=split, **load_dataset_kwargs)

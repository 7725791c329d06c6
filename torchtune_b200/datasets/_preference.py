"""Preference (chosen / rejected) datasets (parity: torchtune/datasets/_preference.py:19-320)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Mapping, Optional

from torch.utils.data import Dataset

from ..data._common import CROSS_ENTROPY_IGNORE_IDX
from ..data._messages import ChosenRejectedToMessages
from ._sft import _load


def _strategy(train_on_input: bool) -> str:
    return "train_on_all" if train_on_input else "train_on_assistant"


class PreferenceDataset(Dataset):
    """Tokenises both sides of each pair; labels are *unshifted* copies of the ids with masked
    (prompt) positions set to the ignore index — the shift happens in the log-prob reduction."""

    def __init__(self, *, source: str, message_transform: Callable, tokenizer, filter_fn: Optional[Callable] = None, packed: bool = False, **load_dataset_kwargs: Any) -> None:
        if packed:
            raise ValueError("Packed is currently not supported for preference datasets.")
        self._tokenizer = tokenizer
        self._message_transform = message_transform
        self._data = _load(source, **load_dataset_kwargs)
        if filter_fn is not None:
            self._data = self._data.filter(filter_fn)

    def __len__(self) -> int:
        return len(self._data)

    def __getitem__(self, index: int) -> Dict[str, List[int]]:
        return self._prepare_sample(self._data[index])

    def _side(self, messages) -> tuple:
        ids, mask = self._tokenizer.tokenize_messages(messages)
        labels = [CROSS_ENTROPY_IGNORE_IDX if m else t for t, m in zip(ids, mask)]
        assert len(ids) == len(labels)
        return ids, labels

    def _prepare_sample(self, sample: Mapping[str, Any]) -> Dict[str, List[int]]:
        pair = self._message_transform(sample)
        c_ids, c_labels = self._side(pair["chosen"])
        r_ids, r_labels = self._side(pair["rejected"])
        return dict(chosen_input_ids=c_ids, chosen_labels=c_labels, rejected_input_ids=r_ids, rejected_labels=r_labels)


def preference_dataset(tokenizer, *, source: str, column_map: Optional[Dict[str, str]] = None, train_on_input: bool = False, new_system_prompt: Optional[str] = None, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> PreferenceDataset:
    """Pairs stored as two conversations (lists of ``{role, content}``) per row."""
    transform = ChosenRejectedToMessages(masking_strategy=_strategy(train_on_input), column_map=column_map, new_system_prompt=new_system_prompt)
    return PreferenceDataset(source=source, message_transform=transform, tokenizer=tokenizer, filter_fn=filter_fn, split=split, **load_dataset_kwargs)

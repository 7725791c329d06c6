"""Unstructured text datasets for continued pre-training (parity: torchtune/datasets/_text_completion.py:18-171)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Union

from torch.utils.data import Dataset

from ..data._common import CROSS_ENTROPY_IGNORE_IDX
from ..data._utils import truncate
from ._packed import PackedDataset
from ._sft import _load


class TextCompletionDataset(Dataset):
    """Encodes ``sample[column]`` with BOS (and EOS when ``add_eos``), truncates to
    ``max_seq_len - 1`` and emits ``labels = tokens[1:] + [ignore]``."""

    def __init__(self, tokenizer, source: str, column: str = "text", add_eos: bool = True, filter_fn: Optional[Callable] = None, **load_dataset_kwargs: Any) -> None:
        self._tokenizer = tokenizer
        self._data = _load(source, **load_dataset_kwargs)
        self._column = column
        self.add_eos = add_eos
        if filter_fn is not None:
            self._data = self._data.filter(filter_fn)

    def __len__(self) -> int:
        return len(self._data)

    def __getitem__(self, index: int) -> Dict[str, List[int]]:
        return self._prepare_sample(self._data[index])

    def _prepare_sample(self, sample) -> Dict[str, List[int]]:
        tokens = self._tokenizer.encode(text=sample[self._column], add_bos=True, add_eos=self.add_eos)
        if self._tokenizer.max_seq_len is not None:
            tokens = truncate(tokens, self._tokenizer.max_seq_len - 1)
        return {"tokens": tokens, "labels": tokens[1:] + [CROSS_ENTROPY_IGNORE_IDX]}


def text_completion_dataset(tokenizer, source: str, column: str = "text", add_eos: bool = True, packed: bool = False, split_across_pack: bool = True, split: str = "train", filter_fn: Optional[Callable] = None, **load_dataset_kwargs: Any) -> Union[TextCompletionDataset, PackedDataset]:
    ds = TextCompletionDataset(tokenizer=tokenizer, source=source, column=column, add_eos=add_eos, split=split, filter_fn=filter_fn, **load_dataset_kwargs)
    if packed:
        if tokenizer.max_seq_len is None:
            raise ValueError("PackedDataset requires a max_seq_len to be set on the tokenizer.")
        return PackedDataset(ds, max_seq_len=tokenizer.max_seq_len, padding_idx=getattr(tokenizer, "pad_id", 0) or 0, split_across_pack=split_across_pack)
    return ds

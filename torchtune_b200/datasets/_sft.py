"""Supervised fine-tuning dataset (parity: torchtune/datasets/_sft.py:19-180)."""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional

from torch.utils.data import Dataset

from ..data._common import CROSS_ENTROPY_IGNORE_IDX
from ..data._messages import validate_messages


def _load(source: str, **kwargs: Any):
    from datasets import load_dataset

    return load_dataset(source, **kwargs)


class SFTTransform:
    """``message_transform`` (row → messages) then ``model_transform`` (messages → tokens +
    mask); labels are the tokens shifted left by one with masked positions and the final
    position set to the ignore index, so no logit slicing is needed downstream."""

    def __init__(self, message_transform: Optional[Callable] = None, model_transform: Optional[Callable] = None):
        if message_transform is None and model_transform is None:
            raise ValueError("At least one of message_transform or model_transform must be provided.")
        self._message_transform = message_transform
        self._model_transform = model_transform

    def __call__(self, sample: Mapping[str, Any]) -> Dict[str, Any]:
        if self._message_transform is not None:
            sample = self._message_transform(sample)
            if "messages" in sample:
                validate_messages(sample["messages"])
        if self._model_transform is None:
            return sample
        out = self._model_transform(sample)
        if not ("tokens" in out and "mask" in out):
            raise ValueError(f"model_transform returned the following keys: {', '.join(out.keys())}. Must return 'tokens' and 'mask' as keys.")
        tokens, mask = out["tokens"], out["mask"]
        out["labels"] = [CROSS_ENTROPY_IGNORE_IDX if masked else tok for tok, masked in zip(tokens[1:], mask[1:])] + [CROSS_ENTROPY_IGNORE_IDX]
        assert len(out["tokens"]) == len(out["labels"])
        return out


class SFTDataset(Dataset):
    def __init__(self, *, source: str, message_transform: Callable, model_transform: Callable, filter_fn: Optional[Callable] = None, filter_kwargs: Optional[Dict[str, Any]] = None, **load_dataset_kwargs: Any) -> None:
        self._message_transform = message_transform
        self._model_transform = model_transform
        self._data = _load(source, **load_dataset_kwargs)
        if filter_fn is not None:
            self._data = self._data.filter(filter_fn, **(filter_kwargs or {}))
        self._prepare_sample = SFTTransform(message_transform=message_transform, model_transform=model_transform)

    def __len__(self) -> int:
        return len(self._data)

    def __getitem__(self, index: int) -> Dict[str, Any]:
        return self._prepare_sample(self._data[index])

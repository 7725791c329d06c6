"""Index-range concatenation of datasets (parity: torchtune/datasets/_concat.py:16-91)."""
from __future__ import annotations

import bisect
from typing import Any, List

from torch.utils.data import Dataset


class ConcatDataset(Dataset):
    """View several datasets as one.  Either all or none of them may be packed."""

    def __init__(self, datasets: List[Dataset]):
        self._datasets = list(datasets)
        packed = [getattr(d, "packed", False) or type(d).__name__ == "PackedDataset" for d in self._datasets]
        if any(packed) and not all(packed):
            raise ValueError("ConcatDataset can't process a mix of packed and non-packed datasets.")
        self.packed = all(packed) and bool(packed)
        self._ends: List[int] = []
        total = 0
        for d in self._datasets:
            total += len(d)
            self._ends.append(total)

    def __len__(self) -> int:
        return self._ends[-1] if self._ends else 0

    def __getitem__(self, index: int) -> Any:
        if index < 0:
            index += len(self)
        if not 0 <= index < len(self):
            raise IndexError(f"Index {index} out of range")
        which = bisect.bisect_right(self._ends, index)
        start = self._ends[which - 1] if which else 0
        return self._datasets[which][index - start]

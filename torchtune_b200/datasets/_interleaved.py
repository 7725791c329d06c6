"""Weighted interleaving of several map-style datasets (role of the multi-dataset sampler built from torchdata nodes at
torchtune/data/_utils.py:240-347, used by recipes/dev/lora_finetune_distributed_multi_dataset.py).

The mixture is a *map-style* dataset of fixed length: position ``i`` belongs to dataset ``d(i)`` drawn with the given
probabilities from a seeded generator, and is the ``k``-th visit of that dataset (its rows are visited in order and wrap
around).  Being a pure function of ``(seed, i)`` it composes with the resumable sampler / loader like any other dataset —
no iterator state has to be checkpointed."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch
from torch.utils.data import Dataset


class InterleavedDataset(Dataset):
    def __init__(self, datasets: Sequence[Dataset], weights: Optional[Sequence[float]] = None, seed: int = 0, length: Optional[int] = None, stop_criterion: str = "cycle_until_all_exhausted"):
        if not datasets:
            raise ValueError("need at least one dataset")
        self.datasets = list(datasets)
        w = torch.tensor([1.0] * len(datasets) if weights is None else [float(x) for x in weights], dtype=torch.float64)
        if (w <= 0).any():
            raise ValueError("dataset weights must be positive")
        self.weights = (w / w.sum()).tolist()
        sizes = [len(d) for d in self.datasets]
        if length is None:
            if stop_criterion == "first_exhausted":
                length = int(min(n / p for n, p in zip(sizes, self.weights)))
            elif stop_criterion in ("cycle_until_all_exhausted", "all_exhausted"):
                length = int(max(n / p for n, p in zip(sizes, self.weights)))
            else:
                raise ValueError(f"unknown stop_criterion {stop_criterion!r}")
        self._len = max(length, 1)
        g = torch.Generator().manual_seed(seed)
        choice = torch.multinomial(torch.tensor(self.weights), self._len, replacement=True, generator=g)
        self._which = choice.tolist()
        # k-th visit of each dataset at every position
        counts = [0] * len(datasets)
        self._local: List[int] = []
        for d in self._which:
            self._local.append(counts[d] % sizes[d])
            counts[d] += 1

    def __len__(self) -> int:
        return self._len

    def __getitem__(self, index: int) -> Dict[str, Any]:
        return self.datasets[self._which[index]][self._local[index]]

"""Resumable data loading: a distributed sampler and loader whose position can be saved
in ``recipe_state.pt`` and restored (parity with the stateful loader/sampler used at
recipes/full_finetune_distributed.py:825-849 and :936-941)."""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Iterator, Optional

import torch
from torch.utils.data import DataLoader, Dataset, Sampler


class StatefulDistributedSampler(Sampler[int]):
    """Rank-strided (optionally shuffled) index stream with ``state_dict`` support."""

    def __init__(self, dataset: Dataset, num_replicas: int = 1, rank: int = 0, shuffle: bool = True, seed: int = 0, drop_last: bool = False):
        self.dataset, self.num_replicas, self.rank = dataset, num_replicas, rank
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch = 0
        self.start_index = 0
        n = len(dataset)
        self.num_samples = n // num_replicas if drop_last else math.ceil(n / num_replicas)
        self.total_size = self.num_samples * num_replicas

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _indices(self):
        n = len(self.dataset)
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            idx = torch.randperm(n, generator=g).tolist()
        else:
            idx = list(range(n))
        if self.drop_last:
            idx = idx[: self.total_size]
        else:
            pad = self.total_size - len(idx)
            idx += (idx * math.ceil(pad / max(len(idx), 1)))[:pad]
        return idx[self.rank : self.total_size : self.num_replicas]

    def __iter__(self) -> Iterator[int]:
        idx = self._indices()[self.start_index :]
        self.start_index = 0
        return iter(idx)

    def __len__(self) -> int:
        return self.num_samples

    def state_dict(self) -> Dict[str, Any]:
        return {"epoch": self.epoch, "seed": self.seed}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.epoch = sd.get("epoch", 0)


class StatefulDataLoader:
    """``DataLoader`` wrapper that counts yielded batches; after ``load_state_dict`` the next
    iteration skips what was already consumed in the interrupted epoch."""

    def __init__(self, dataset: Dataset, batch_size: int, sampler: Optional[StatefulDistributedSampler] = None, collate_fn: Optional[Callable] = None, drop_last: bool = True, num_workers: int = 0, pin_memory: bool = False, **kwargs):
        self.sampler = sampler
        self.batch_size = batch_size
        self._loader = DataLoader(dataset, batch_size=batch_size, sampler=sampler, collate_fn=collate_fn, drop_last=drop_last, num_workers=num_workers, pin_memory=pin_memory, **kwargs)
        self._yielded = 0
        self._resume_batches = 0

    @property
    def dataset(self):
        return self._loader.dataset

    def __len__(self) -> int:
        return len(self._loader)

    def __iter__(self):
        if self._resume_batches and self.sampler is not None:
            self.sampler.start_index = self._resume_batches * self.batch_size
        self._yielded = self._resume_batches
        self._resume_batches = 0
        for batch in self._loader:
            self._yielded += 1
            yield batch
        self._yielded = 0

    def mark_epoch_end(self) -> None:
        """Call when an epoch is abandoned early (step cap): the saved position then means
        "start of the next epoch" rather than "inside this one"."""
        self._yielded = 0

    def state_dict(self) -> Dict[str, Any]:
        return {"batches_yielded": self._yielded, "sampler": self.sampler.state_dict() if self.sampler is not None else None}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self._resume_batches = sd.get("batches_yielded", 0)
        if self.sampler is not None and sd.get("sampler"):
            self.sampler.load_state_dict(sd["sampler"])

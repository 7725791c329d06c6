"""Synthetic token datasets for benchmarking and tests.

The reference has no counterpart (its tests use a ``DummyDataset``,
tests/recipes/utils.py:22-45).  These builders are ``_component_``-instantiable and
accept (and ignore) a tokenizer as first positional argument so they slot into
recipes exactly where a real dataset builder would.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.utils.data import Dataset

from ..data._common import CROSS_ENTROPY_IGNORE_IDX


class SyntheticSFTDataset(Dataset):
    """I.i.d. uniform tokens; ``labels[i] = tokens[i+1]`` with the last label and the first
    ``prompt_len`` label positions of each row set to the ignore index."""

    def __init__(self, vocab_size: int, seq_len: int, num_samples: int = 1024, prompt_len: int = 0, seed: int = 0):
        self.vocab_size, self.seq_len, self.num_samples, self.prompt_len, self.seed = vocab_size, seq_len, num_samples, prompt_len, seed

    def __len__(self) -> int:
        return self.num_samples

    def _tokens(self, idx: int, n: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        return torch.randint(0, self.vocab_size, (n,), generator=g, dtype=torch.long)

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        tokens = self._tokens(idx, self.seq_len)
        labels = torch.cat([tokens[1:], torch.tensor([CROSS_ENTROPY_IGNORE_IDX])])
        labels[: self.prompt_len] = CROSS_ENTROPY_IGNORE_IDX
        return {"tokens": tokens, "labels": labels}


class SyntheticPackedDataset(SyntheticSFTDataset):
    """Packed rows of ``seq_len`` tokens made of documents of ``doc_len`` tokens: positions
    restart at every boundary and the last label of each document is ignored."""

    def __init__(self, vocab_size: int, seq_len: int, doc_len: int, num_samples: int = 1024, seed: int = 0):
        super().__init__(vocab_size, seq_len, num_samples, 0, seed)
        if seq_len % doc_len:
            raise ValueError("seq_len must be a multiple of doc_len")
        self.doc_len = doc_len

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        tokens = self._tokens(idx, self.seq_len)
        labels = torch.cat([tokens[1:], torch.tensor([CROSS_ENTROPY_IGNORE_IDX])])
        labels[self.doc_len - 1 :: self.doc_len] = CROSS_ENTROPY_IGNORE_IDX
        n_docs = self.seq_len // self.doc_len
        return {
            "tokens": tokens,
            "labels": labels,
            "input_pos": torch.arange(self.doc_len).repeat(n_docs),
            "seq_lens": torch.full((n_docs,), self.doc_len, dtype=torch.long),
        }


class SyntheticPreferenceDataset(Dataset):
    """Chosen/rejected pairs of ``seq_len`` tokens sharing a ``prompt_len`` prefix, with
    independent uniform completions; labels are unshifted copies with the prompt masked."""

    def __init__(self, vocab_size: int, seq_len: int, prompt_len: int, num_samples: int = 1024, seed: int = 0):
        self.vocab_size, self.seq_len, self.prompt_len, self.num_samples, self.seed = vocab_size, seq_len, prompt_len, num_samples, seed

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, idx: int) -> Dict[str, List[int]]:
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        prompt = torch.randint(0, self.vocab_size, (self.prompt_len,), generator=g)
        out = {}
        for name in ("chosen", "rejected"):
            completion = torch.randint(0, self.vocab_size, (self.seq_len - self.prompt_len,), generator=g)
            ids = torch.cat([prompt, completion])
            labels = ids.clone()
            labels[: self.prompt_len] = CROSS_ENTROPY_IGNORE_IDX
            out[f"{name}_input_ids"] = ids.tolist()
            out[f"{name}_labels"] = labels.tolist()
        return out


def synthetic_sft_dataset(tokenizer: Any = None, *, vocab_size: int, seq_len: int, num_samples: int = 1024, prompt_len: int = 0, seed: int = 0, packed: bool = False, doc_len: Optional[int] = None, **_: Any) -> Dataset:
    if packed:
        return SyntheticPackedDataset(vocab_size, seq_len, doc_len or seq_len, num_samples, seed)
    return SyntheticSFTDataset(vocab_size, seq_len, num_samples, prompt_len, seed)


def synthetic_packed_dataset(tokenizer: Any = None, *, vocab_size: int, seq_len: int, doc_len: int, num_samples: int = 1024, seed: int = 0, **_: Any) -> Dataset:
    return SyntheticPackedDataset(vocab_size, seq_len, doc_len, num_samples, seed)


def synthetic_preference_dataset(tokenizer: Any = None, *, vocab_size: int, seq_len: int, prompt_len: int, num_samples: int = 1024, seed: int = 0, **_: Any) -> Dataset:
    return SyntheticPreferenceDataset(vocab_size, seq_len, prompt_len, num_samples, seed)

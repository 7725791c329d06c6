"""Offline greedy sample packing (parity: torchtune/datasets/_packed.py:17-274)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
from torch.utils.data import Dataset

from ..data._common import CROSS_ENTROPY_IGNORE_IDX, PACK_TYPE


class PackedDataset(Dataset):
    """Concatenates tokenised samples into rows of exactly ``max_seq_len`` tokens.

    Each pack keeps ``tokens``, ``labels``, ``input_pos`` (restarting at every sample) and
    ``seq_lens`` (one entry per sample, padding counted as a final pseudo-sample so the
    lengths sum to ``max_seq_len``).  A sample that does not fit starts the next pack, or —
    with ``split_across_pack`` — is cut at the boundary.  ``max_packs`` bounds the work.
    """

    packed = True

    def __init__(self, ds: Dataset, *, max_seq_len: int, padding_idx: int = 0, max_packs: Optional[int] = None, split_across_pack: bool = False) -> None:
        self.ds = ds
        self.max_seq_len = max_seq_len
        self.padding_idx = padding_idx
        self.max_packs = max_packs
        self.split_across_pack = split_across_pack
        self.packs: List[PACK_TYPE] = []
        self.previous_sample_boundary = 0
        self._pack()

    # ------------------------------------------------------------------
    def _full(self) -> bool:
        return self.max_packs is not None and len(self.packs) >= self.max_packs

    def _pack(self) -> None:
        cur: Dict[str, List[int]] = {"tokens": [], "labels": [], "input_pos": [], "seq_lens": []}
        for sample in self.ds:
            tokens, labels = list(sample["tokens"]), list(sample["labels"])
            n = len(tokens)
            if n > self.max_seq_len and not self.split_across_pack:
                raise ValueError(f"Dataset sample is too long ({n} > {self.max_seq_len}). Please set `split_across_pack=True` or increase `max_seq_len`.")
            cur["tokens"] += tokens
            cur["labels"] += labels
            cur["input_pos"] += [i % self.max_seq_len for i in range(n)]
            cur["seq_lens"].append(n)
            while len(cur["tokens"]) > self.max_seq_len and not self._full():
                cur = self._emit_and_carry(cur)
            self.previous_sample_boundary = len(cur["tokens"])
            if self._full():
                break
        if cur["tokens"] and not self._full():
            self._add(cur)

    def _emit_and_carry(self, cur: Dict[str, List[int]]) -> Dict[str, List[int]]:
        """Emit one full pack from the front of ``cur`` and return what is left over."""
        if self.split_across_pack:
            cut = self.max_seq_len
            head_of_last = cut - sum(cur["seq_lens"][:-1])
            head_lens = cur["seq_lens"][:-1] + ([head_of_last] if head_of_last > 0 else [])
            carried_len = cur["seq_lens"][-1] - head_of_last
        else:
            cut = self.previous_sample_boundary
            head_lens = cur["seq_lens"][:-1]
            carried_len = cur["seq_lens"][-1]
        self._add({"tokens": cur["tokens"][:cut], "labels": cur["labels"][:cut], "input_pos": cur["input_pos"][:cut], "seq_lens": head_lens})
        return {"tokens": cur["tokens"][cut:], "labels": cur["labels"][cut:], "input_pos": cur["input_pos"][cut:], "seq_lens": [carried_len]}

    def _add(self, pack: Dict[str, List[int]]) -> None:
        tokens = torch.tensor(pack["tokens"], dtype=torch.long)
        labels = torch.tensor(pack["labels"], dtype=torch.long)
        pos = torch.tensor(pack["input_pos"], dtype=torch.long)
        lens = torch.tensor(pack["seq_lens"], dtype=torch.long)
        pad = self.max_seq_len - tokens.numel()
        if pad > 0:
            tokens = torch.cat([tokens, torch.full((pad,), self.padding_idx, dtype=torch.long)])
            labels = torch.cat([labels, torch.full((pad,), CROSS_ENTROPY_IGNORE_IDX, dtype=torch.long)])
            last = int(pos[-1]) if pos.numel() else -1
            # positions simply keep counting through the padding (clamped to stay valid)
            pos = torch.cat([pos, torch.clamp(torch.arange(last + 1, last + 1 + pad), max=self.max_seq_len - 1)])
            lens = torch.cat([lens, torch.tensor([pad])])
        self.packs.append({"tokens": tokens, "labels": labels, "input_pos": pos, "seq_lens": lens})

    def __len__(self) -> int:
        return len(self.packs)

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        return self.packs[idx]

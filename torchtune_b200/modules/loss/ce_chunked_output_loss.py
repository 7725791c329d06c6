"""Cross entropy over a list of logit chunks (parity: torchtune/modules/loss/ce_chunked_output_loss.py:18-102)."""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F
from torch import nn


class CEWithChunkedOutputLoss(nn.Module):
    """Takes the list produced by ``model.set_num_output_chunks(n)``; each chunk is upcast
    to fp32 separately so only one fp32 chunk is alive at a time."""

    def __init__(self, num_output_chunks: int = 8, ignore_index: int = -100):
        super().__init__()
        self.num_output_chunks = num_output_chunks
        self.ignore_index = ignore_index

    def compute_cross_entropy(self, logits: torch.Tensor, labels: torch.Tensor, normalize: bool = True) -> torch.Tensor:
        return F.cross_entropy(logits.float(), labels, ignore_index=self.ignore_index, reduction="sum")

    def forward(self, logits: List[torch.Tensor], labels: torch.Tensor) -> torch.Tensor:
        n_valid = (labels != self.ignore_index).sum()
        label_chunks = labels.tensor_split(self.num_output_chunks, dim=1)
        total = 0.0
        for lg, lb in zip(logits, label_chunks):
            total = total + self.compute_cross_entropy(lg.reshape(-1, lg.size(-1)), lb.reshape(-1))
        return total / n_valid.clamp_min(1)

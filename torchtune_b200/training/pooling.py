"""Sequence-length helper (parity: torchtune/training/pooling.py:9-42)."""
import torch


def get_unmasked_sequence_lengths(mask: torch.Tensor) -> torch.Tensor:
    """Index of the last non-padding token per row of a right-padded batch; ``mask`` is
    True on padding.  Rows that are entirely padding give 0."""
    lengths = (~mask).sum(-1)
    return (lengths - 1).clamp(0, mask.shape[1] - 1)

"""Mask helpers for packed batches (API of torchtune/modules/attention_utils.py:55-176).

The attention kernel takes a *structured* mask (:class:`torchtune_b200.ops.mask.AttentionMask`: per-token document ids, causal
flag, chunk / window sizes) instead of a dense ``[b, s, s]`` tensor or a flex-attention block mask, so
:func:`packed_block_causal_mask` returns that; :func:`create_block_causal_mask` still materialises the dense boolean mask for
callers that want to look at it or run the eager reference path.
"""
from __future__ import annotations

from typing import List

import torch

from ..ops.mask import AttentionMask


def create_block_causal_mask(seq_lens: List[torch.Tensor]) -> torch.Tensor:
    """``seq_lens[i]``: lengths of the documents packed into sample ``i`` → boolean ``[b, s, s]`` mask that is lower triangular
    inside every document and False across documents (all samples must sum to the same ``s``)."""
    masks = []
    for lens in seq_lens:
        lens = torch.as_tensor(lens)
        doc = torch.repeat_interleave(torch.arange(lens.numel(), device=lens.device), lens)
        same = doc[:, None] == doc[None, :]
        pos = torch.arange(doc.numel(), device=lens.device)
        masks.append(same & (pos[:, None] >= pos[None, :]))
    return torch.stack(masks)


def packed_block_causal_mask(seq_lens: List[torch.Tensor]) -> AttentionMask:
    """Block-causal mask of a packed batch in the form the attention kernel consumes (document ids per token)."""
    return AttentionMask.from_seq_lens(seq_lens)


def causal_mask_flex(b, h, q_idx, kv_idx):
    """Mask predicate ``(batch, head, query index, key index) → visible?`` of a plain causal mask — the calling convention of
    flex-attention mask mods, usable with index tensors (broadcasting) to materialise a mask for the eager path."""
    return q_idx >= kv_idx


def kv_offset_mask_flex(b, h, q_idx, kv_idx, offset):
    """Mask predicate for decoding one token at cache position ``offset``: every key up to and including it is visible."""
    return kv_idx <= offset

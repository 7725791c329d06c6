"""Chunked (local) attention for the RoPE layers of Llama 4
(parity: torchtune/models/llama4/_chunked_attention.py:20-75): a query attends only to keys of the
same ``chunk_size`` block of positions, on top of whatever mask the batch carries.  Expressed as the
``chunk`` field of :class:`~torchtune_b200.ops.mask.AttentionMask`, which the attention kernel turns
into a per-query lower bound — no block-mask object or dense mask is built."""
from __future__ import annotations

from dataclasses import replace
from typing import Callable

import torch

from ...ops.mask import AttentionMask


def get_chunked_attention_mask(mask, chunk_size: int, bsz: int, seq_len: int):
    if mask is None:
        return AttentionMask(causal=True, chunk=chunk_size)
    if isinstance(mask, AttentionMask) and mask.bool_mask is None:
        return replace(mask, chunk=chunk_size)
    dense = mask.bool_mask if isinstance(mask, AttentionMask) else mask
    q = torch.arange(dense.shape[-2], device=dense.device).view(-1, 1) + (dense.shape[-1] - dense.shape[-2])
    k = torch.arange(dense.shape[-1], device=dense.device).view(1, -1)
    return dense & ((q // chunk_size) == (k // chunk_size))


def chunked_mask_mod(chunk_size: int) -> Callable:
    return lambda mask, bsz, seq_len: get_chunked_attention_mask(mask, chunk_size, bsz, seq_len)

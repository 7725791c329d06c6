"""Key/value cache for incremental decoding (parity: torchtune/modules/kv_cache.py:11-116).

Buffers are laid out ``[batch, max_seq_len, num_kv_heads, head_dim]`` — the layout the
attention kernels consume — rather than head-major.
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import nn


class KVCache(nn.Module):
    def __init__(self, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> None:
        super().__init__()
        shape = (batch_size, max_seq_len, num_kv_heads, head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        self.register_buffer("v_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        # positions of the *next* writes; kept as a tensor so updates are pure tensor ops
        self.register_buffer("cache_pos", torch.arange(0, max_seq_len), persistent=False)
        self.batch_size = batch_size
        self.max_seq_len = max_seq_len

    def reset(self) -> None:
        self.k_cache.zero_()
        self.v_cache.zero_()
        self.cache_pos -= self.size

    @property
    def size(self) -> int:
        return int(self.cache_pos[0].item())

    def update(self, k_val: torch.Tensor, v_val: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Append ``[b, s, n_kv, d]`` keys/values and return the full buffers."""
        bsz, seq_len = k_val.shape[0], k_val.shape[1]
        if bsz > self.k_cache.shape[0]:
            raise ValueError(
                f"The current cache has been setup with a batch size of {self.k_cache.shape[0]}"
                f", but found new key tensors with batch size {bsz}!"
            )
        if self.cache_pos[0] + seq_len > self.max_seq_len:
            raise AssertionError("KV cache is full: cannot write past max_seq_len")
        where = self.cache_pos[:seq_len]
        self.k_cache[:bsz].index_copy_(1, where, k_val)
        self.v_cache[:bsz].index_copy_(1, where, v_val)
        self.cache_pos.add_(seq_len)
        return self.k_cache[:bsz], self.v_cache[:bsz]

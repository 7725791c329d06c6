"""KV cache for exported graphs (parity: torchtune/modules/_export/kv_cache.py:12-130): ``[b, max_seq, n_kv, d]`` (or the
head-major ``[b, n_kv, max_seq, d]`` with ``transpose_cache``) buffers updated with ``index_copy_`` at explicit positions."""
from __future__ import annotations

from typing import Tuple

import torch
from torch import nn


class KVCache(nn.Module):
    def __init__(self, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype, transpose_cache: bool = True) -> None:
        super().__init__()
        self.transpose_cache = transpose_cache
        shape = (batch_size, num_kv_heads, max_seq_len, head_dim) if transpose_cache else (batch_size, max_seq_len, num_kv_heads, head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        self.register_buffer("v_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        self.register_buffer("cache_pos", torch.arange(0, max_seq_len), persistent=False)
        self.batch_size, self.max_seq_len = batch_size, max_seq_len

    @property
    def size(self) -> int:
        return int(self.cache_pos[0].item())

    def reset(self) -> None:
        self.k_cache.zero_()
        self.v_cache.zero_()
        self.cache_pos -= self.size

    def update(self, k_val: torch.Tensor, v_val: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``k_val`` / ``v_val`` are in the cache's layout; they are written at the next ``seq_len`` positions."""
        seq_dim = 2 if self.transpose_cache else 1
        seq_len = k_val.shape[seq_dim]
        pos = self.cache_pos[:seq_len]
        self.k_cache.index_copy_(seq_dim, pos, k_val)
        self.v_cache.index_copy_(seq_dim, pos, v_val)
        self.cache_pos.add_(seq_len)
        return self.k_cache, self.v_cache

"""Exportable attention (parity: torchtune/modules/_export/attention.py:21-440)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..attention import MultiHeadAttention as TrainingMHA
from .kv_cache import KVCache


class SDPA(nn.Module):
    """The attention core as its own module (a single node runtimes can swap): expands KV heads for grouped-query attention and
    calls ``scaled_dot_product_attention``."""

    def __init__(self, num_kv_heads: int, num_heads: int, head_dim: int, attn_dropout: float, is_causal: bool, kv_cache: Optional[KVCache]) -> None:
        super().__init__()
        self.num_kv_heads, self.num_heads, self.head_dim = num_kv_heads, num_heads, head_dim
        self.q_per_kv = num_heads // num_kv_heads
        self.attn_dropout, self.is_causal, self.kv_cache = attn_dropout, is_causal, kv_cache

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bsz: int, seq_len: int, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``q`` ``[b, n_h, s, d]``, ``k`` / ``v`` ``[b, n_kv, s_kv, d]`` → ``[b, s, n_h·d]``."""
        if self.q_per_kv > 1:
            k = k.unsqueeze(2).expand(-1, -1, self.q_per_kv, -1, -1).flatten(1, 2)
            v = v.unsqueeze(2).expand(-1, -1, self.q_per_kv, -1, -1).flatten(1, 2)
        if mask is not None and mask.dim() == 3:
            mask = mask[:, None, :, :]
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=0.0, is_causal=self.kv_cache is None and mask is None and self.is_causal)
        return out.transpose(1, 2).reshape(bsz, seq_len, -1)


class MultiHeadAttention(nn.Module):
    """Same projections / norms / RoPE as the training attention, with the cache update and the attention core expressed in
    traceable ops."""

    def __init__(self, *, embed_dim: int, num_heads: int, num_kv_heads: int, head_dim: int, q_proj: nn.Module, k_proj: nn.Module, v_proj: nn.Module, output_proj: nn.Module,
                 pos_embeddings: Optional[nn.Module] = None, q_norm: Optional[nn.Module] = None, k_norm: Optional[nn.Module] = None, kv_cache: Optional[KVCache] = None,
                 max_seq_len: int = 4096, is_causal: bool = True, attn_dropout: float = 0.0) -> None:
        super().__init__()
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        if bool(q_norm) ^ bool(k_norm):
            raise ValueError("q and k norm must be set together")
        self.num_heads, self.num_kv_heads, self.embed_dim, self.head_dim = num_heads, num_kv_heads, embed_dim, head_dim
        self.max_seq_len, self.is_causal, self.attn_dropout = max_seq_len, is_causal, attn_dropout
        self.kv_cache = kv_cache
        self.q_proj, self.k_proj, self.v_proj, self.output_proj = q_proj, k_proj, v_proj, output_proj
        self.q_norm, self.k_norm, self.pos_embeddings = q_norm, k_norm, pos_embeddings
        self._sdpa = SDPA(num_kv_heads, num_heads, head_dim, attn_dropout, is_causal, kv_cache)
        self.cache_enabled = False

    def setup_cache(self, batch_size: int, dtype: torch.dtype, max_seq_len: int) -> None:
        self.kv_cache = KVCache(batch_size=batch_size, max_seq_len=max_seq_len, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, dtype=dtype, transpose_cache=True)
        self._sdpa.kv_cache = self.kv_cache
        self.cache_enabled = True

    def reset_cache(self) -> None:
        if self.kv_cache is None:
            raise RuntimeError("Key value caches are not setup. Call ``setup_caches()`` first.")
        self.kv_cache.reset()

    def forward(self, x: torch.Tensor, y: Optional[torch.Tensor] = None, *, mask: Optional[torch.Tensor] = None, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, s_x, _ = x.shape
        q = self.q_proj(x).view(b, s_x, self.num_heads, self.head_dim)
        if self.pos_embeddings is not None:
            q = self.pos_embeddings(q, input_pos=input_pos)
        q = q.transpose(1, 2)
        if self.q_norm is not None:
            q = self.q_norm(q)
        if y is None:
            if self.kv_cache is None:
                raise ValueError("Must provide y input or use kv_cache to enable streaming decoding")
            k, v = self.kv_cache.k_cache, self.kv_cache.v_cache
        else:
            s_y = y.shape[1]
            k = self.k_proj(y).view(b, s_y, self.num_kv_heads, self.head_dim)
            v = self.v_proj(y).view(b, s_y, self.num_kv_heads, self.head_dim)
            if self.pos_embeddings is not None:
                k = self.pos_embeddings(k, input_pos=input_pos)
            k, v = k.transpose(1, 2), v.transpose(1, 2)
            if self.k_norm is not None:
                k = self.k_norm(k)
            if self.kv_cache is not None and self.cache_enabled:
                k, v = self.kv_cache.update(k, v)
        return self.output_proj(self._sdpa(q, k, v, b, s_x, mask=mask))


def _convert(mha: TrainingMHA) -> MultiHeadAttention:
    return MultiHeadAttention(embed_dim=mha.embed_dim, num_heads=mha.num_heads, num_kv_heads=mha.num_kv_heads, head_dim=mha.head_dim, q_proj=mha.q_proj, k_proj=mha.k_proj, v_proj=mha.v_proj,
                              output_proj=mha.output_proj, pos_embeddings=mha.pos_embeddings, q_norm=mha.q_norm, k_norm=mha.k_norm, kv_cache=None, max_seq_len=mha.max_seq_len,
                              is_causal=mha.is_causal, attn_dropout=mha.attn_dropout)


def replace_mha_with_inference_mha(module: nn.Module) -> nn.Module:
    """Swap every training attention module below ``module`` (in place) for the exportable variant sharing its sub-modules."""
    for name, child in list(module.named_children()):
        if isinstance(child, TrainingMHA):
            setattr(module, name, _convert(child))
        else:
            replace_mha_with_inference_mha(child)
    return module

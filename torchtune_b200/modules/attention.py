"""Multi-head / grouped-query attention (parity: torchtune/modules/attention.py:18-303)."""
from __future__ import annotations

import logging
from typing import Optional, Union

import torch
from torch import nn

from .. import ops
from ..ops.mask import AttentionMask
from .kv_cache import KVCache

logger = logging.getLogger(__name__)

MaskLike = Union[AttentionMask, torch.Tensor, None]


def _as_mask(mask: MaskLike, default_causal: bool) -> AttentionMask:
    if mask is None:
        return AttentionMask(causal=default_causal)
    if isinstance(mask, AttentionMask):
        return mask
    return AttentionMask(causal=False, bool_mask=mask)


class MultiHeadAttention(nn.Module):
    """Attention with ``num_kv_heads <= num_heads`` key/value heads.

    Tensors stay in ``[batch, seq, heads, head_dim]`` from the projections to the
    output projection; key/value heads are never expanded — the kernel maps query head
    ``h`` to KV head ``h // (num_heads // num_kv_heads)``.  ``mask`` may be an
    :class:`~torchtune_b200.ops.AttentionMask` (structured, used for training) or a
    boolean tensor ``[b, s_q, s_kv]`` with True = attend.  With ``y`` given this is
    cross attention; ``y=None`` on a cross-attention layer reads the KV cache.
    """

    def __init__(
        self,
        *,
        embed_dim: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        q_proj: nn.Module,
        k_proj: nn.Module,
        v_proj: nn.Module,
        output_proj: nn.Module,
        pos_embeddings: Optional[nn.Module] = None,
        q_norm: Optional[nn.Module] = None,
        k_norm: Optional[nn.Module] = None,
        kv_cache: Optional[KVCache] = None,
        max_seq_len: int = 4096,
        is_causal: bool = True,
        attn_dropout: float = 0.0,
        softcap: float = 0.0,
        scale: Optional[float] = None,
        qk_norm_before_rope: bool = False,
    ) -> None:
        super().__init__()
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        if attn_dropout < 0 or attn_dropout > 1:
            raise ValueError(f"attn_dropout ({attn_dropout}) must be between 0.0 and 1.0")
        if bool(q_norm) ^ bool(k_norm):
            raise ValueError("q and k norm must be set together")
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.embed_dim = embed_dim
        self.attn_dropout = attn_dropout
        self.head_dim = head_dim
        self.max_seq_len = max_seq_len
        self.is_causal = is_causal
        self.softcap = softcap
        self.scale = scale
        self.kv_cache = kv_cache
        self.q_proj = q_proj
        self.k_proj = k_proj
        self.v_proj = v_proj
        self.output_proj = output_proj
        self.q_norm = q_norm
        self.k_norm = k_norm
        self.pos_embeddings = pos_embeddings
        self.qk_norm_before_rope = qk_norm_before_rope
        self.cache_enabled = False

    def setup_cache(self, batch_size: int, dtype: torch.dtype, max_seq_len: int) -> None:
        if self.kv_cache is not None:
            logger.warning("Key value caches are already setup. You cannot call ``setup_caches()`` twice. Skipping.")
            return
        self.kv_cache = KVCache(batch_size, max_seq_len, self.num_kv_heads, self.head_dim, dtype)
        # a cache created outside a device context lands on the CPU; it belongs where this module's weights are
        home = next((t.device for t in list(self.parameters()) + list(self.buffers()) if t.device.type != "meta"), None)
        if home is not None and home.type != "cpu" and self.kv_cache.k_cache.device.type == "cpu":
            self.kv_cache.to(home)
        self.cache_enabled = True

    def reset_cache(self) -> None:
        if self.kv_cache is None:
            raise RuntimeError("Key value caches are not setup. Call ``setup_caches()`` first.")
        self.kv_cache.reset()

    def forward(
        self,
        x: torch.Tensor,
        y: Optional[torch.Tensor] = None,
        *,
        mask: MaskLike = None,
        input_pos: Optional[torch.Tensor] = None,
        residual: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        """``residual``: a tensor of the output's shape that is added to the result; with a plain output projection the addition
        happens in that projection's GEMM epilogue (a decoder layer passes its residual stream)."""
        b, s_x, _ = x.shape
        q = self.q_proj(x).view(b, s_x, self.num_heads, self.head_dim)
        if self.q_norm is not None and self.qk_norm_before_rope:
            q = self.q_norm(q)
        if self.pos_embeddings is not None:
            q = self.pos_embeddings(q, input_pos=input_pos)
        if self.q_norm is not None and not self.qk_norm_before_rope:
            q = self.q_norm(q)

        if y is None:
            if self.kv_cache is None or not self.cache_enabled:
                raise ValueError("Must provide y input or use kv_cache to enable streaming decoding")
            k, v = self.kv_cache.k_cache[:b], self.kv_cache.v_cache[:b]
        else:
            s_y = y.shape[1]
            k = self.k_proj(y).view(b, s_y, self.num_kv_heads, self.head_dim)
            v = self.v_proj(y).view(b, s_y, self.num_kv_heads, self.head_dim)
            if self.k_norm is not None and self.qk_norm_before_rope:
                k = self.k_norm(k)
            if self.pos_embeddings is not None:
                k = self.pos_embeddings(k, input_pos=input_pos)
            if self.k_norm is not None and not self.qk_norm_before_rope:
                k = self.k_norm(k)
            if self.kv_cache is not None and self.cache_enabled:
                k, v = self.kv_cache.update(k, v)

        plain = self.kv_cache is None or not self.cache_enabled
        attn_mask = _as_mask(mask, default_causal=self.is_causal and plain and mask is None)
        cp = getattr(self, "context_parallel", None)
        if cp is not None and plain:  # sequence-sharded activations: whole sequences for a subset of heads inside attention
            q, k, v = cp.seq_to_heads(q), cp.seq_to_heads(k), cp.seq_to_heads(v)
        out = ops.attention(
            q,
            k,
            v,
            attn_mask,
            scale=self.scale,
            softcap=self.softcap,
            dropout_p=self.attn_dropout if self.training else 0.0,
        )
        if cp is not None and plain:
            out = cp.heads_to_seq(out)
        out = out.reshape(b, s_x, self.num_heads * self.head_dim)
        if residual is None:
            return self.output_proj(out)
        if type(self.output_proj) is nn.Linear:
            return ops.linear_residual(out, self.output_proj.weight, self.output_proj.bias, residual)
        return self.output_proj(out) + residual

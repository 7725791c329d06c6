"""T5 v1.1 encoder (parity: torchtune/models/t5/_encoder.py:17-310): bidirectional transformer with
un-scaled dot-product attention plus a learned bias per (bucketed relative position, head) shared by
all layers, RMS pre-norms and gated-GELU feed-forward."""
from __future__ import annotations

import math
from typing import List

import torch
import torch.nn.functional as F
from torch import nn


def relative_position_buckets(num_buckets: int, max_dist: int, max_seq_len: int) -> torch.Tensor:
    """``[q, k]`` bucket ids for bidirectional attention: half of the buckets serve keys after the
    query; within each half small distances get their own bucket and larger ones share
    logarithmically sized buckets up to ``max_dist``."""
    rel = torch.arange(max_seq_len)[None, :] - torch.arange(max_seq_len)[:, None]
    dist = rel.abs()
    half = num_buckets // 2
    exact = half // 2
    log_bucket = exact + (torch.log(dist.float().clamp_min(1) / exact) / math.log(max_dist / exact) * (half - exact)).to(torch.long)
    log_bucket = log_bucket.clamp_max(half - 1)
    return (rel > 0).long() * half + torch.where(dist < exact, dist, log_bucket)


class T5EncoderRelativePositionBias(nn.Module):
    def __init__(self, num_buckets: int, max_dist: int, num_heads: int, max_seq_len: int):
        super().__init__()
        self.max_seq_len = max_seq_len
        self.embedding = nn.Embedding(num_buckets, num_heads)
        self.register_buffer("relative_position_to_bucket", relative_position_buckets(num_buckets, max_dist, max_seq_len), persistent=False)

    def forward(self) -> torch.Tensor:
        return self.embedding(self.relative_position_to_bucket).permute(2, 0, 1).unsqueeze(0)  # [1, heads, q, k]


class T5EncoderSelfAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, head_dim: int, q_proj: nn.Module, k_proj: nn.Module, v_proj: nn.Module, output_proj: nn.Module):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        if embed_dim // num_heads != head_dim:
            raise ValueError(f"head_dim ({head_dim}) must be equal to embed_dim // num_heads")
        self.num_heads, self.head_dim = num_heads, head_dim
        self.q_proj, self.k_proj, self.v_proj, self.output_proj = q_proj, k_proj, v_proj, output_proj

    def forward(self, x: torch.Tensor, rel_pos_bias: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        split = lambda t: t.view(b, s, self.num_heads, self.head_dim).transpose(1, 2)
        q, k, v = split(self.q_proj(x)), split(self.k_proj(x)), split(self.v_proj(x))
        bias = rel_pos_bias[:, :, :s, :s].to(q.dtype)
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, scale=1.0)  # T5 does not scale by 1/sqrt(d)
        return self.output_proj(out.transpose(1, 2).reshape(b, s, d))


class T5EncoderLayer(nn.Module):
    def __init__(self, attn: nn.Module, mlp: nn.Module, sa_norm: nn.Module, mlp_norm: nn.Module) -> None:
        super().__init__()
        self.attn, self.mlp, self.sa_norm, self.mlp_norm = attn, mlp, sa_norm, mlp_norm

    def forward(self, x: torch.Tensor, rel_pos_bias: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.sa_norm(x), rel_pos_bias)
        return x + self.mlp(self.mlp_norm(x))


class T5Encoder(nn.Module):
    def __init__(self, *, token_embedding: nn.Embedding, layers: List[nn.Module], final_norm: nn.Module, num_heads: int, rel_pos_num_buckets: int, rel_pos_max_dist: int, max_seq_len: int) -> None:
        super().__init__()
        self.token_embedding, self.final_norm, self.max_seq_len = token_embedding, final_norm, max_seq_len
        self.relative_position_bias = T5EncoderRelativePositionBias(rel_pos_num_buckets, rel_pos_max_dist, num_heads, max_seq_len)
        self.layers = layers if isinstance(layers, nn.ModuleList) else nn.ModuleList(layers)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if tokens.shape[1] > self.max_seq_len:
            raise ValueError(f"seq_len ({tokens.shape[1]}) of input tensor should be smaller than max_seq_len ({self.max_seq_len})")
        x = self.token_embedding(tokens)
        bias = self.relative_position_bias()
        for layer in self.layers:
            x = layer(x, bias)
        return self.final_norm(x)

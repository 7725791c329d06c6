"""CLIP text tower (parity: torchtune/models/clip/_text_encoder.py:16-110)."""
from __future__ import annotations

import copy
from typing import Optional

import torch
from torch import nn


class QuickGELU(nn.Module):
    """``x · sigmoid(1.702 x)`` — the GELU approximation CLIP was trained with."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * torch.sigmoid(1.702 * x)


class CLIPTextEncoder(nn.Module):
    """Causal transformer over at most ``max_seq_len`` tokens; the output is the final-norm hidden
    state at the first end-of-text token of every sequence (``[bsz, embed_dim]``)."""

    def __init__(self, *, layer: nn.Module, final_norm: nn.Module, vocab_size: int = 49408, max_seq_len: int = 77, embed_dim: int = 768, num_layers: int = 12, eot_token: int = 49407):
        super().__init__()
        self.layers = nn.ModuleList([copy.deepcopy(layer) for _ in range(num_layers)])
        self.final_norm = final_norm
        self.max_seq_len, self.eot_token = max_seq_len, eot_token
        self.token_embedding = nn.Embedding(vocab_size, embed_dim)
        self.position_embedding = nn.Parameter(torch.empty(max_seq_len, embed_dim).normal_(std=0.01))

    def forward(self, tokens: torch.Tensor, *, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        _, seq_len = tokens.shape
        if seq_len > self.max_seq_len:
            raise ValueError(f"seq_len ({seq_len}) of input tensor should be smaller than max_seq_len ({self.max_seq_len})")
        x = self.token_embedding(tokens) + self.position_embedding[:seq_len].to(self.token_embedding.weight.dtype)
        for layer in self.layers:
            x = layer(x, mask=mask)
        x = self.final_norm(x)
        eot = (tokens == self.eot_token).int().argmax(dim=-1)
        return x.take_along_dim(eot.view(-1, 1, 1), dim=1).squeeze(1)

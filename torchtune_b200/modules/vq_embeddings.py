"""Vector-quantised embedding table (parity: torchtune/modules/vq_embeddings.py:12-95; arXiv 1711.00937)."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F
from torch import nn


class VectorQuantizedEmbeddings(nn.Module):
    """Maps every input vector to its nearest (L2) codebook row; the output equals the codebook row in the
    forward pass and passes gradients straight through to the input in the backward pass."""

    def __init__(self, num_embeddings: int, embedding_dim: int) -> None:
        super().__init__()
        self.embedding = nn.Parameter(torch.empty(num_embeddings, embedding_dim).normal_())
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim

    def forward(self, z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        bsz, seq_len, dim = z.shape
        if dim != self.embedding_dim:
            raise ValueError(f"Expected last dimension of input tensor ({dim}) to be embedding size of {self.embedding_dim}")
        flat = z.reshape(-1, dim)
        # ‖z − e‖² = ‖z‖² − 2 z·e + ‖e‖²; the first term does not affect the argmin
        scores = (self.embedding.pow(2).sum(1) - 2.0 * flat @ self.embedding.t()) if flat.shape[0] else flat.new_zeros(0, self.num_embeddings)
        ids = scores.argmin(dim=1)
        q = self.decode(ids)
        q = flat + (q - flat).detach()
        return q.view(bsz, seq_len, dim), ids.view(bsz, seq_len)

    def extra_repr(self) -> str:
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}"

    def decode(self, token_ids: torch.Tensor) -> torch.Tensor:
        return F.embedding(token_ids, self.embedding)

"""Gemma building blocks (parity: torchtune/models/gemma/rms_norm.py:11-26,
torchtune/models/gemma/gemma_norm_embedding.py)."""
import math

import torch
from torch import nn


class GemmaRMSNorm(nn.Module):
    """RMS norm whose learnable gain is ``1 + scale`` (``scale`` starts at zero) and whose
    multiply happens in fp32 before the cast back."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.scale = nn.Parameter(torch.zeros(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (out * (1.0 + self.scale.float())).type_as(x)


class GemmaNormEmbeddings(nn.Embedding):
    """Token embedding scaled by ``sqrt(embedding_dim)``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return super().forward(x) * math.sqrt(self.embedding_dim)


class TanhSoftCapping(nn.Module):
    """``cap · tanh(x / cap)``."""

    def __init__(self, capping_value: float):
        super().__init__()
        self.capping_value = capping_value

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.tanh(x / self.capping_value) * self.capping_value


class Gemma2FinalNorm(nn.Module):
    """Final RMS norm of Gemma-2, optionally followed by soft capping of the normalised hidden state.

    The reference caps here, on the hidden state that then goes through the output projection
    (torchtune/models/gemma2/_component_builders.py:56-72).  The published model caps the *logits*, after the projection, which
    is not the same function; this package's builders therefore pass ``cap_hidden=False`` and set the decoder's
    ``logit_softcap`` instead.  ``cap_hidden=True`` reproduces the reference's graph.  The parameter name
    (``rms_norm.scale``) is the same either way, so checkpoints are interchangeable."""

    def __init__(self, capping_value: float, embed_dim: int, eps: float, cap_hidden: bool = True):
        super().__init__()
        self.capping_value = capping_value
        self.cap_hidden = cap_hidden
        self.rms_norm = GemmaRMSNorm(embed_dim, eps=eps)
        self.logit_capping = TanhSoftCapping(capping_value)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.rms_norm(x)
        return self.logit_capping(x) if self.cap_hidden else x
